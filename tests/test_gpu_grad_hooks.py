"""Gradient statistics and the gradient multiplier folded into the update pass.

The oracle here is the CPU restatement plus two numpy lines: sum(g*g) in float64 and isfinite
over the gradient the kernel consumes, and g' = fl32(g * scale) handed to the reference
arithmetic as an fp32 gradient.  p / m / v / bf16 must match bit for bit; sumsq is accumulated
with fp32 atomics in no fixed order, so it is compared to 1e-5 relative.  With scale 1 and no
statistics block the element loop must be the plain one (checked against the unhooked call).
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG0 = (1e-5, 0.9, 0.999, 1e-8, 0.01)


def _np_g(g):
    return g.view(torch.int16).numpy().view(np.uint16) if g.dtype == torch.bfloat16 else g.numpy()


def _f32(gnp, oracle):
    return oracle.bf16_to_f32(gnp) if gnp.dtype == np.uint16 else gnp


def _expect(oracle, orc, step, hp, p, gnp, m, v, out, scale, tally):
    gf = _f32(gnp, oracle)
    tally["sumsq"] += float(np.sum(gf.astype(np.float64) ** 2))
    tally["nonfinite"] |= not bool(np.isfinite(gf).all())
    gs = (gf * np.float32(scale)).astype(np.float32)
    orc.adam_update(step, *hp, True, p, gs, m, v, out)


def _same(a_np, t):
    if a_np.dtype == np.float32:
        return np.array_equal(a_np.view(np.uint32), t.cpu().numpy().view(np.uint32))
    return np.array_equal(a_np, t.view(torch.int16).cpu().numpy().view(np.uint16))


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [7, 4096 + 16 + 5, (1 << 20) + 13])
@pytest.mark.parametrize("scale", [1.0, 0.37])
def test_layer_adam_stats_and_scale(n, scale, gdtype, oracle):
    from slideformer_b200 import LayerAdam
    gen = torch.Generator().manual_seed(n)
    p0 = torch.randn(n, generator=gen) * 0.02
    po, mo, vo, oo = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
    pd, md, vd = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    od = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    opt = LayerAdam(lr=CFG0[0], betas=CFG0[1:3], eps=CFG0[3], weight_decay=CFG0[4])
    orc = oracle.OracleAdam(*CFG0, True)
    opt.enable_grad_stats(DEV)
    opt.set_grad_scale(scale)
    tally = {"sumsq": 0.0, "nonfinite": False}
    for step in (1, 2, 3):
        g = (torch.randn(n, generator=gen) * 1e-3).to(gdtype)
        _expect(oracle, orc, step, CFG0, po, _np_g(g), mo, vo, oo, scale, tally)
        opt.step_chunk(pd, g.to(DEV), md, vd, dict(opt.defaults, step=step), od)
    st = opt.read_grad_stats()
    assert st["nonfinite"] is False
    assert st["sumsq"] == pytest.approx(tally["sumsq"], rel=1e-5)
    assert st["norm"] == pytest.approx(tally["sumsq"] ** 0.5, rel=1e-5)
    for a, b in ((po, pd), (mo, md), (vo, vd), (oo, od)):
        assert _same(a, b)
    assert opt.read_grad_stats()["sumsq"] == 0.0      # the read above reset the block


def test_nonfinite_gradient_is_flagged(oracle):
    from slideformer_b200 import LayerAdam
    n = 50_000
    opt = LayerAdam(lr=1e-3)
    opt.enable_grad_stats(DEV)
    z = lambda: torch.zeros(n, device=DEV)  # noqa: E731
    g = torch.zeros(n, dtype=torch.bfloat16)
    opt.step_chunk(z(), g.to(DEV), z(), z(), dict(opt.defaults, step=1))
    assert opt.read_grad_stats()["nonfinite"] is False
    for bad in (float("inf"), float("nan"), -float("inf")):
        g2 = g.clone()
        g2[n - 3] = bad
        opt.step_chunk(z(), g2.to(DEV), z(), z(), dict(opt.defaults, step=2))
        assert opt.read_grad_stats()["nonfinite"] is True


def test_hooks_off_is_the_plain_kernel(oracle):
    """scale 1 and no statistics block after hooks were on: same launch path and bits as an
    optimizer that never had hooks."""
    from slideformer_b200 import LayerAdam, _lib
    n = 200_003
    gen = torch.Generator().manual_seed(1)
    p0 = (torch.randn(n, generator=gen) * 0.02).to(DEV)
    g = (torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16).to(DEV)
    outs = []
    for hooked in (False, True):
        opt = LayerAdam(lr=CFG0[0], betas=CFG0[1:3], eps=CFG0[3], weight_decay=CFG0[4])
        if hooked:
            opt.enable_grad_stats(DEV)
            opt.set_grad_scale(0.5)
            opt.disable_grad_stats()
            opt.set_grad_scale(1.0)
        sc = _lib.SfAdamScalars()
        _lib.check(opt._lib.sf_adam_scalars(opt.optimizer_id, 1, *CFG0, 1, C.byref(sc)))
        assert sc.grad_scale == 1.0 and not sc.grad_stats
        p, m, v = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        o = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
        opt.step_chunk(p, g, m, v, dict(opt.defaults, step=2), o)
        outs.append((p, m, v, o))
    for a, b in zip(*outs):
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                           b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16))


@pytest.mark.parametrize("entry", ["push", "pull"])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_dp_kernels_stats_and_scale(world, entry, oracle):
    """The statistics of the data-parallel kernels are those of the fp32 MEAN gradient."""
    from slideformer_b200 import _lib
    lib = _lib.load()
    n, scale = 300_000 + 11, 0.25
    gen = torch.Generator().manual_seed(world)
    p0 = torch.randn(n, generator=gen) * 0.02
    po, mo, vo, oo = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
    pd, md, vd = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    outs = [torch.zeros(n, device=DEV, dtype=torch.bfloat16) for _ in range(world if entry == "push" else 1)]
    stats = torch.zeros(64, device=DEV)
    oid = 660000 + world
    _lib.check(lib.sf_adam_create(oid, *CFG0, 1, 0))
    _lib.check(lib.sf_adam_set_grad_hooks(oid, scale, stats.data_ptr()))
    orc = oracle.OracleAdam(*CFG0, True)
    tally = {"sumsq": 0.0, "nonfinite": False}
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for step in (1, 2):
            rows = (torch.randn(world, n, generator=gen) * 1e-3).to(torch.bfloat16)
            mean = oracle.rank_mean(np.ascontiguousarray(rows.view(torch.int16).numpy().view(np.uint16)))
            _expect(oracle, orc, step, CFG0, po, mean, mo, vo, oo, scale, tally)
            dev = [rows[r].to(DEV) for r in range(world)]
            peers = (C.c_void_p * world)(*[t.data_ptr() for t in dev])
            sc = _lib.SfAdamScalars()
            _lib.check(lib.sf_adam_scalars(oid, step, *CFG0, 1, C.byref(sc)))
            if entry == "push":
                op = (C.c_void_p * world)(*[t.data_ptr() for t in outs])
                _lib.check(lib.sf_adam_step_sharded_push(C.byref(sc), pd.data_ptr(), peers, op, world, _lib.SF_GRAD_BF16,
                                                         md.data_ptr(), vd.data_ptr(), n, n & ~15, stream))
            else:
                _lib.check(lib.sf_adam_step_sharded(C.byref(sc), pd.data_ptr(), peers, world, _lib.SF_GRAD_BF16,
                                                    md.data_ptr(), vd.data_ptr(), outs[0].data_ptr(), n, n & ~15, stream))
        torch.cuda.synchronize()
        host = stats.cpu()
        assert float(host[:32].double().sum()) == pytest.approx(tally["sumsq"], rel=1e-5)
        assert host[32:33].view(torch.int32).item() == 0
        for a, b in ((po, pd), (mo, md), (vo, vd)):
            assert _same(a, b)
        for o in outs:
            assert _same(oo, o)
    finally:
        lib.sf_adam_destroy(oid)
