"""Index arithmetic beyond 2^31 elements (a flat vector of 2^31 + 4099 parameters, 34-43 GB on
the device): 64-bit offsets in the vector kernel, its scalar remainder and the pull + push kernel.

A CPU pass over everything would take minutes, so the check is by properties that hold for every
element plus oracle windows at the start, across the 2^31 boundary and at the end:
  * the bf16 output is the round-to-nearest-even cast of the updated p everywhere;
  * after one step from m = 0, m is zero exactly where the gradient is zero (no element skipped,
    none visited with a wrong gradient index);
  * the windows match the CPU oracle bit for bit.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG0 = (1e-5, 0.9, 0.999, 1e-8, 0.01)
N_BIG = (1 << 31) + 4099


def _fill(t, std, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    step = 1 << 28
    for lo in range(0, t.numel(), step):
        hi = min(lo + step, t.numel())
        if t.dtype == torch.float32:
            t[lo:hi].normal_(0, std, generator=gen)
        else:
            t[lo:hi].copy_(torch.empty(hi - lo, device=DEV).normal_(0, std, generator=gen))


def _windows(n):
    w = 1 << 16
    return [(0, w), ((1 << 31) - w, (1 << 31) + 2048), (n - w - 3, n)]


def _need_memory(gb):
    free = torch.cuda.mem_get_info()[0] / 2 ** 30
    if free < gb:
        pytest.skip(f"needs {gb} GB of free device memory, {free:.0f} GB available")


def _check_everywhere(p, m, out, grads_zero_mask_fn, n):
    step = 1 << 28
    for lo in range(0, n, step):
        hi = min(lo + step, n)
        assert torch.equal(out[lo:hi].view(torch.int16), p[lo:hi].to(torch.bfloat16).view(torch.int16)), lo
        assert torch.equal(m[lo:hi] == 0, grads_zero_mask_fn(lo, hi)), lo


def test_vector_kernel_beyond_2_31_elements(oracle):
    from slideformer_b200 import LayerAdam
    _need_memory(45)
    n = N_BIG
    p = torch.empty(n, device=DEV)
    _fill(p, 0.02, 1)
    g = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    _fill(g, 1e-3, 2)
    g[(1 << 31) - 5:(1 << 31) + 5] = 0          # zeros straddling the boundary
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    out = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    wins = _windows(n)
    before = [p[lo:hi].cpu().numpy().copy() for lo, hi in wins]
    opt = LayerAdam(lr=CFG0[0], betas=CFG0[1:3], eps=CFG0[3], weight_decay=CFG0[4])
    opt.step_chunk(p, g, m, v, dict(opt.defaults, step=1), out)
    torch.cuda.synchronize()
    _check_everywhere(p, m, out, lambda lo, hi: g[lo:hi] == 0, n)
    c = oracle.OracleAdam(*CFG0, True).scalars(1, *CFG0, True)
    for (lo, hi), p0 in zip(wins, before):
        k = hi - lo
        mo, vo, oo = np.zeros(k, np.float32), np.zeros(k, np.float32), np.zeros(k, np.uint16)
        gnp = g[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16)
        oracle.apply_step(c, p0, gnp, mo, vo, oo, vec_n=min(max((n & ~15) - lo, 0), k))
        assert np.array_equal(p0.view(np.uint32), p[lo:hi].cpu().numpy().view(np.uint32)), (lo, hi)
        assert np.array_equal(mo.view(np.uint32), m[lo:hi].cpu().numpy().view(np.uint32))
        assert np.array_equal(vo.view(np.uint32), v[lo:hi].cpu().numpy().view(np.uint32))
        assert np.array_equal(oo, out[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16))


def test_pull_push_kernel_beyond_2_31_elements(oracle):
    """Two local buffers as the ranks: the world-2 kernel with 16-byte peer accesses."""
    from slideformer_b200 import _lib
    _need_memory(55)
    lib = _lib.load()
    n, world = N_BIG, 2
    p = torch.empty(n, device=DEV)
    _fill(p, 0.02, 3)
    grads = []
    for r in range(world):
        gr = torch.empty(n, device=DEV, dtype=torch.bfloat16)
        _fill(gr, 1e-3, 10 + r)
        gr[(1 << 31) - 5:(1 << 31) + 5] = 0
        grads.append(gr)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    outs = [torch.zeros(n, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    wins = _windows(n)
    before = [p[lo:hi].cpu().numpy().copy() for lo, hi in wins]
    oid = 440044
    _lib.check(lib.sf_adam_create(oid, *CFG0, 1, 0))
    try:
        sc = _lib.SfAdamScalars()
        _lib.check(lib.sf_adam_scalars(oid, 1, *CFG0, 1, C.byref(sc)))
        pg = (C.c_void_p * world)(*[t.data_ptr() for t in grads])
        po = (C.c_void_p * world)(*[t.data_ptr() for t in outs])
        _lib.check(lib.sf_adam_step_sharded_push(C.byref(sc), p.data_ptr(), pg, po, world, _lib.SF_GRAD_BF16, m.data_ptr(),
                                                 v.data_ptr(), n, n & ~15, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
    finally:
        lib.sf_adam_destroy(oid)
    # the mean of two bf16 values is zero iff their fp32 sum is zero
    _check_everywhere(p, m, outs[0], lambda lo, hi: (grads[0][lo:hi].float() + grads[1][lo:hi].float()) == 0, n)
    assert torch.equal(outs[0].view(torch.int16)[-(1 << 20):], outs[1].view(torch.int16)[-(1 << 20):])
    c = oracle.OracleAdam(*CFG0, True).scalars(1, *CFG0, True)
    for (lo, hi), p0 in zip(wins, before):
        k = hi - lo
        rows = np.stack([gr[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16) for gr in grads])
        mo, vo, oo = np.zeros(k, np.float32), np.zeros(k, np.float32), np.zeros(k, np.uint16)
        oracle.apply_step(c, p0, oracle.rank_mean(rows), mo, vo, oo, vec_n=min(max((n & ~15) - lo, 0), k))
        assert np.array_equal(p0.view(np.uint32), p[lo:hi].cpu().numpy().view(np.uint32)), (lo, hi)
        assert np.array_equal(mo.view(np.uint32), m[lo:hi].cpu().numpy().view(np.uint32))
        for out in outs:
            assert np.array_equal(oo, out[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16))
