"""The data-parallel kernels on ONE GPU: `world` local buffers stand in for the peers.

sf_adam_step_sharded_push (pull the gradients of all ranks, Adam, push the bf16 weights to all
ranks), sf_adam_step_sharded (pull only) and sf_dp_mean take arrays of device pointers; whether
a pointer is local or peer-mapped makes no difference to the arithmetic, so every code path the
multi-GPU runs use (every world-specialised kernel, both vector widths, the scalar fallback, the
tail) can be driven through the C ABI with buffers of one device and compared with the CPU
oracle: fp32 rank-order mean (multi_gpu/shared_data_parallel.py:130-133), then the reference
Adam call.  Tolerance: 0 ulp on p / m / v, bit-exact bf16 in EVERY output copy.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG0 = (1e-5, 0.9, 0.999, 1e-8, 0.01)
REFHP = (0.01, 0.8, 0.95, 1e-6, 0.1)


@pytest.fixture(scope="module")
def lib():
    from slideformer_b200 import _lib
    return _lib.load()


def _bits32(t):
    return t.detach().cpu().numpy().view(np.uint32)


def _bits16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _rows(world, n, dtype, gen, special=False):
    rows = torch.randn(world, n, generator=gen) * 1e-3
    if special and n >= 32:
        rows[0, :8] = torch.tensor([0.0, -0.0, 1e-30, -1e-22, 65504.0, 1e-40, -1e-38, 3.0])
        rows[:, 8:12] = -0.0          # 0 + (-0) + (-0) ... = +0 in the reference's accumulator
    return rows.to(dtype)


def _np(rows):
    if rows.dtype == torch.bfloat16:
        return rows.view(torch.int16).numpy().view(np.uint16)
    return rows.numpy()


class Case:
    """State on the device and its CPU twin; `off` shifts every device buffer by `off` elements
    to reach the scalar (misaligned) kernels."""

    def __init__(self, n, world, dtype, hp, adamw=True, off=0, seed=0, outs=True):
        from slideformer_b200 import _lib
        self.n, self.world, self.dtype, self.hp, self.adamw, self.off = n, world, dtype, hp, adamw, off
        self.gen = torch.Generator().manual_seed(seed)
        p0 = torch.randn(n, generator=self.gen) * 0.02
        self.po, self.mo, self.vo = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        self.oo = np.zeros(n, np.uint16)
        pad = torch.zeros(off)
        self.pd = torch.cat([pad, p0]).to(DEV)
        self.md = torch.zeros(n + off, device=DEV)
        self.vd = torch.zeros(n + off, device=DEV)
        self.outs = [torch.zeros(n + off, device=DEV, dtype=torch.bfloat16) for _ in range(world if outs else 0)]
        self.gcode = _lib.SF_GRAD_BF16 if dtype == torch.bfloat16 else _lib.SF_GRAD_F32
        self.oid = 770000 + seed % 1000
        _lib.check(_lib.load().sf_adam_create(self.oid, *hp, int(adamw), 0))

    def grads(self, special=False):
        rows = _rows(self.world, self.n, self.dtype, self.gen, special)
        dev = [torch.cat([torch.zeros(self.off, dtype=self.dtype), rows[r]]).to(DEV) for r in range(self.world)]
        return rows, dev

    def scalars(self, lib, step, bc=True):
        from slideformer_b200 import _lib
        sc = _lib.SfAdamScalars()
        _lib.check(lib.sf_adam_scalars(self.oid, step, *self.hp, int(bc), C.byref(sc)))
        return sc

    def ptrs(self, tensors, esize):
        return (C.c_void_p * len(tensors))(*[t.data_ptr() + self.off * esize for t in tensors])

    def check(self, what=""):
        o = self.off
        for name, a, b in (("p", self.po, self.pd), ("m", self.mo, self.md), ("v", self.vo, self.vd)):
            got, want = _bits32(b[o:]), a.view(np.uint32)
            bad = np.nonzero(got != want)[0]
            assert bad.size == 0, f"{what} {name}: {bad.size} of {want.size} differ, first at {bad[0]}"
            if o:
                assert not _bits32(b[:o]).any() or name == "p", f"{what} {name}: wrote in front of the slice"
        for r, out in enumerate(self.outs):
            got = _bits16(out[o:])
            bad = np.nonzero(got != self.oo)[0]
            assert bad.size == 0, f"{what} bf16 copy {r}: {bad.size} differ, first at {bad[0]}"
            if o:
                assert not _bits16(out[:o]).any()

    def close(self, lib):
        lib.sf_adam_destroy(self.oid)


def _oracle_step(O, orc, case, step, rows, vec_n=None, bc=True):
    mean = O.rank_mean(np.ascontiguousarray(_np(rows)))
    orc.adam_update(step, *case.hp, bc, case.po, mean, case.mo, case.vo, case.oo, vec_n=vec_n)
    return mean


PUSH_SHAPES = [(8, 1), (4, 1), (4, 0)]   # (elements per thread, world-specialised kernels on/off)


@pytest.mark.parametrize("vec,spec", PUSH_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8, 16])
def test_push_kernel_vs_oracle(world, dtype, vec, spec, oracle, lib):
    """Three steps at a size with a tile remainder and a 13-element scalar tail."""
    from slideformer_b200 import _lib
    n = 2048 * 37 + 8 * 5 + 13
    _lib.check(lib.sf_set_push_tuning(vec, spec))
    case = Case(n, world, dtype, CFG0, seed=world * 7 + vec + spec)
    orc = oracle.OracleAdam(*CFG0, True)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for step in (1, 2, 3):
            rows, dev = case.grads(special=(step == 2))
            _oracle_step(oracle, orc, case, step, rows)
            sc = case.scalars(lib, step)
            _lib.check(lib.sf_adam_step_sharded_push(
                C.byref(sc), case.pd.data_ptr(), case.ptrs(dev, 2 if dtype == torch.bfloat16 else 4),
                case.ptrs(case.outs, 2), world, case.gcode, case.md.data_ptr(), case.vd.data_ptr(), n, n & ~15, stream))
            torch.cuda.synchronize()
            case.check(f"world {world} step {step}")
    finally:
        _lib.check(lib.sf_set_push_tuning(8, 1))
        case.close(lib)


@pytest.mark.parametrize("off", [1, 3])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [2, 8])
def test_push_kernel_misaligned_buffers(world, dtype, off, oracle, lib):
    """Buffers that start at an odd element: the scalar fallback, spread over the grid, writes the
    same bits and nothing outside the slice."""
    from slideformer_b200 import _lib
    n = 300_007
    case = Case(n, world, dtype, REFHP, off=off, seed=off + world)
    orc = oracle.OracleAdam(*REFHP, True)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for step in (1, 2):
            rows, dev = case.grads()
            _oracle_step(oracle, orc, case, step, rows)
            sc = case.scalars(lib, step)
            before = lib.sf_launch_count()
            _lib.check(lib.sf_adam_step_sharded_push(
                C.byref(sc), case.pd.data_ptr() + 4 * off, case.ptrs(dev, 2 if dtype == torch.bfloat16 else 4),
                case.ptrs(case.outs, 2), world, case.gcode, case.md.data_ptr() + 4 * off, case.vd.data_ptr() + 4 * off,
                n, n & ~15, stream))
            assert lib.sf_launch_count() == before + 1
            torch.cuda.synchronize()
            case.check(f"off {off} step {step}")
    finally:
        case.close(lib)


@pytest.mark.parametrize("vec", [4, 8])
@pytest.mark.parametrize("cut", ["head", "middle", "tail", "all_tail"])
def test_push_kernel_vec_n_cut(cut, vec, oracle, lib):
    """One reference call over 16*700+11 elements executed as slices: the slice-relative vec_n says
    where that call's tail arithmetic starts (first slices: everything is body; last: a short
    tail; 'all_tail': vec_n = 0, every element uses the tail's rounding)."""
    from slideformer_b200 import _lib
    from slideformer_b200.shared_data_parallel import slice_vec_n
    total = 16 * 700 + 11
    a, b = {"head": (0, 16 * 300), "middle": (16 * 300, 16 * 650), "tail": (16 * 650, total), "all_tail": (0, 5000)}[cut]
    n = b - a
    vec_local = 0 if cut == "all_tail" else slice_vec_n(0, total, a, b)
    world = 4
    _lib.check(lib.sf_set_push_tuning(vec, 1))
    case = Case(n, world, torch.bfloat16, CFG0, seed=11)
    orc = oracle.OracleAdam(*CFG0, True)
    try:
        rows, dev = case.grads()
        _oracle_step(oracle, orc, case, 1, rows, vec_n=vec_local)
        sc = case.scalars(lib, 1)
        _lib.check(lib.sf_adam_step_sharded_push(
            C.byref(sc), case.pd.data_ptr(), case.ptrs(dev, 2), case.ptrs(case.outs, 2), world, case.gcode,
            case.md.data_ptr(), case.vd.data_ptr(), n, vec_local, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        case.check(cut)
    finally:
        _lib.check(lib.sf_set_push_tuning(8, 1))
        case.close(lib)


@pytest.mark.parametrize("adamw,bc,wd", [(True, True, 0.1), (False, True, 0.1), (True, False, 0.0)])
@pytest.mark.parametrize("world", [2, 8])
def test_push_kernel_modes(world, adamw, bc, wd, oracle, lib):
    from slideformer_b200 import _lib
    hp = REFHP[:4] + (wd,)
    n = 70_001
    case = Case(n, world, torch.bfloat16, hp, adamw=adamw, seed=23)
    orc = oracle.OracleAdam(*hp, adamw)
    try:
        for step in (1, 2, 3):
            rows, dev = case.grads()
            _oracle_step(oracle, orc, case, step, rows, bc=bc)
            sc = case.scalars(lib, step, bc)
            _lib.check(lib.sf_adam_step_sharded_push(
                C.byref(sc), case.pd.data_ptr(), case.ptrs(dev, 2), case.ptrs(case.outs, 2), world, case.gcode,
                case.md.data_ptr(), case.vd.data_ptr(), n, n & ~15, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        case.check(f"adamw={adamw} bc={bc} wd={wd}")
    finally:
        case.close(lib)


@pytest.mark.parametrize("with_out", [True, False])
@pytest.mark.parametrize("off", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_pull_kernel_vs_oracle(world, dtype, off, with_out, oracle, lib):
    """sf_adam_step_sharded: gradients pulled, bf16 written to one local buffer (or not at all)."""
    from slideformer_b200 import _lib
    n = 1024 * 53 + 4 * 3 + 9
    case = Case(n, world, dtype, CFG0, off=off, seed=31 + world, outs=False)
    if with_out:
        case.outs = [torch.zeros(n + off, device=DEV, dtype=torch.bfloat16)]
    orc = oracle.OracleAdam(*CFG0, True)
    try:
        for step in (1, 2):
            rows, dev = case.grads(special=(step == 1))
            _oracle_step(oracle, orc, case, step, rows)
            sc = case.scalars(lib, step)
            _lib.check(lib.sf_adam_step_sharded(
                C.byref(sc), case.pd.data_ptr() + 4 * off, case.ptrs(dev, 2 if dtype == torch.bfloat16 else 4), world,
                case.gcode, case.md.data_ptr() + 4 * off, case.vd.data_ptr() + 4 * off,
                case.outs[0].data_ptr() + 2 * off if with_out else None, n, n & ~15,
                torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            case.check(f"world {world} step {step}")
    finally:
        case.close(lib)


@pytest.mark.parametrize("off", [0, 1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 3, 8, 16])
def test_dp_mean_vs_oracle(world, dtype, off, oracle, lib):
    from slideformer_b200 import _lib
    for n in (1, 5, 4096 + 3, 1_000_003):
        gen = torch.Generator().manual_seed(n + world)
        rows = _rows(world, n, dtype, gen, special=True)
        dev = [torch.cat([torch.zeros(off, dtype=dtype), rows[r]]).to(DEV) for r in range(world)]
        esize = 2 if dtype == torch.bfloat16 else 4
        peers = (C.c_void_p * world)(*[t.data_ptr() + off * esize for t in dev])
        mean = torch.full((n + off + 1,), 7.0, device=DEV)
        _lib.check(lib.sf_dp_mean(peers, world, _lib.SF_GRAD_BF16 if dtype == torch.bfloat16 else _lib.SF_GRAD_F32,
                                  mean.data_ptr() + 4 * off, n, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        want = oracle.rank_mean(np.ascontiguousarray(_np(rows)))
        assert np.array_equal(_bits32(mean[off:off + n]), want.view(np.uint32)), (n, world, off)
        assert (mean[:off] == 7.0).all() and mean[off + n] == 7.0   # nothing outside [0, n) was written


def test_shared_data_parallel_slices_cover_a_layer(oracle, lib):
    """The way SharedDataParallel cuts a layer: each of `world` owners runs the push kernel on its
    16-aligned slice with the slice-relative vec_n; together they reproduce ONE reference call
    over the whole layer, and every rank's bf16 copy is complete."""
    from slideformer_b200 import _lib
    from slideformer_b200.shared_data_parallel import shard_range, slice_vec_n
    world, n = 8, 1_000_003
    case = Case(n, world, torch.bfloat16, CFG0, seed=5)
    orc = oracle.OracleAdam(*CFG0, True)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for step in (1, 2, 3):
            rows, dev = case.grads()
            _oracle_step(oracle, orc, case, step, rows)
            sc = case.scalars(lib, step)     # one reference call per layer: one state-machine advance
            for owner in range(world):
                a, b = shard_range(n, world, owner)
                if b <= a:
                    continue
                peers = (C.c_void_p * world)(*[t.data_ptr() + 2 * a for t in dev])
                outs = (C.c_void_p * world)(*[t.data_ptr() + 2 * a for t in case.outs])
                _lib.check(lib.sf_adam_step_sharded_push(
                    C.byref(sc), case.pd.data_ptr() + 4 * a, peers, outs, world, case.gcode,
                    case.md.data_ptr() + 4 * a, case.vd.data_ptr() + 4 * a, b - a, slice_vec_n(0, n, a, b), stream))
            torch.cuda.synchronize()
            case.check(f"step {step}")
    finally:
        case.close(lib)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("world", [1, 2, 8])
def test_multi_segment_launch_equals_separate_reference_calls(world, dtype, oracle, lib):
    """sf_adam_step_sharded_push_multi: segments of very different sizes (one empty, one misaligned
    by an element, one whose tail arithmetic starts early) in ONE launch.  Each segment is its own
    reference call on a shared optimizer object, so the calls after the first of a step take the
    pow() branch of the scalar state machine; the oracle follows the same sequence."""
    from slideformer_b200 import _lib
    sizes = [70_001, 0, 16 * 9 + 5, 1024 * 300, 7, 2048 * 11 + 1]
    offs = [0, 0, 0, 0, 0, 1]
    gcode = _lib.SF_GRAD_BF16 if dtype == torch.bfloat16 else _lib.SF_GRAD_F32
    esize = 2 if dtype == torch.bfloat16 else 4
    oid = 551000 + world
    _lib.check(lib.sf_adam_create(oid, *CFG0, 1, 0))
    orc = oracle.OracleAdam(*CFG0, True)
    gen = torch.Generator().manual_seed(world)
    cpu, devs = [], []
    for n, off in zip(sizes, offs):
        p0 = torch.randn(n, generator=gen) * 0.02
        cpu.append([p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)])
        devs.append(dict(p=torch.cat([torch.zeros(off), p0]).to(DEV), m=torch.zeros(n + off, device=DEV),
                         v=torch.zeros(n + off, device=DEV),
                         outs=[torch.zeros(n + off, device=DEV, dtype=torch.bfloat16) for _ in range(world)]))
    try:
        for step in (1, 2, 3):
            segs = (_lib.SfPushSegment * len(sizes))()
            keep = []
            for k, (n, off) in enumerate(zip(sizes, offs)):
                rows = _rows(world, n, dtype, gen)
                gd = [torch.cat([torch.zeros(off, dtype=dtype), rows[r]]).to(DEV) for r in range(world)]
                vec_n = 16 if k == 3 else n & ~15
                if n:
                    mean = oracle.rank_mean(np.ascontiguousarray(_np(rows)))
                else:
                    mean = np.zeros(0, np.float32)
                p, m, v, o = cpu[k]
                orc.adam_update(step, *CFG0, True, p, mean, m, v, o, vec_n=vec_n)
                _lib.check(lib.sf_adam_scalars(oid, step, *CFG0, 1, C.byref(segs[k].s)))
                d = devs[k]
                pg = (C.c_void_p * world)(*[t.data_ptr() + off * esize for t in gd])
                po = (C.c_void_p * world)(*[t.data_ptr() + off * 2 for t in d["outs"]])
                keep += [gd, pg, po]
                segs[k].p, segs[k].m, segs[k].v = (d[x].data_ptr() + 4 * off for x in "pmv")
                segs[k].peer_g, segs[k].peer_out = pg, po
                segs[k].n, segs[k].vec_n = n, vec_n
            before = lib.sf_launch_count()
            _lib.check(lib.sf_adam_step_sharded_push_multi(segs, len(sizes), world, gcode, torch.cuda.current_stream().cuda_stream))
            assert lib.sf_launch_count() == before + 1
            torch.cuda.synchronize()
            for k, (n, off) in enumerate(zip(sizes, offs)):
                p, m, v, o = cpu[k]
                d = devs[k]
                assert np.array_equal(_bits32(d["p"][off:]), p.view(np.uint32)), (step, k, "p")
                assert np.array_equal(_bits32(d["m"][off:]), m.view(np.uint32)), (step, k, "m")
                assert np.array_equal(_bits32(d["v"][off:]), v.view(np.uint32)), (step, k, "v")
                for out in d["outs"]:
                    assert np.array_equal(_bits16(out[off:]), o), (step, k, "bf16")
    finally:
        lib.sf_adam_destroy(oid)
