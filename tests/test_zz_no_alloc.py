"""The entry point that allocates nothing (sf_adam_update_dp_static).

Some callers sit in the steady state of a training step -- the per-chunk gradient reduction on
the optimizer thread while backward is still running -- where all of HBM is already spoken for
and a cudaMalloc would either fail or stall the device.  For them the library stages the fp32
gradient mean in an array that is part of its own image.  This test drives that entry point
through the C ABI and requires the same bits as the existing pair of entry points
(sf_dp_mean into a caller buffer + sf_adam_update), on two calls in a row so that whatever the
first call leaves in the shared array cannot leak into the second.  It lives in a file that
sorts last, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HP = (1e-5, 0.9, 0.999, 1e-8, 0.01)


def _bits(t):
    return t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)


def test_static_scratch_matches_existing_entry_points_twice():
    from slideformer_b200 import _lib
    lib = _lib.load()
    world = 3
    max_elems = _lib.SF_STATIC_SCRATCH_MAX_ELEMS
    assert max_elems == 4 << 20
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(2024)
    id_a, id_b = 880001, 880002
    _lib.check(lib.sf_adam_create(id_a, *HP, 1, 0))
    _lib.check(lib.sf_adam_create(id_b, *HP, 1, 0))
    try:
        # the second call is shorter than the first: stale values beyond its n stay in the array
        for call, n in enumerate(((1 << 20) + 13, 300_007), start=1):
            p0 = (torch.randn(n, generator=gen) * 0.02).to(DEV)
            m0 = (torch.randn(n, generator=gen) * 1e-4).to(DEV)
            v0 = (torch.rand(n, generator=gen) * 1e-6).to(DEV)
            rows = [(torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16).to(DEV) for _ in range(world)]
            peers = (C.c_void_p * world)(*[r.data_ptr() for r in rows])

            # existing entry points, caller-owned fp32 staging buffer
            pa, ma, va = p0.clone(), m0.clone(), v0.clone()
            oa = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
            mean = torch.empty(n, device=DEV)
            _lib.check(lib.sf_dp_mean(peers, world, _lib.SF_GRAD_BF16, mean.data_ptr(), n, stream))
            _lib.check(lib.sf_adam_update(id_a, call, *HP, 1, pa.data_ptr(), mean.data_ptr(), _lib.SF_GRAD_F32,
                                          ma.data_ptr(), va.data_ptr(), oa.data_ptr(), n, stream))

            # the new entry point: no staging buffer passed, nothing allocated
            pb, mb, vb = p0.clone(), m0.clone(), v0.clone()
            ob = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            _lib.check(lib.sf_adam_update_dp_static(id_b, call, *HP, 1, pb.data_ptr(), peers, world, _lib.SF_GRAD_BF16,
                                                    mb.data_ptr(), vb.data_ptr(), ob.data_ptr(), n, stream))
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            for name, a, b in (("p", pa, pb), ("m", ma, mb), ("v", va, vb), ("bf16", oa, ob)):
                assert torch.equal(_bits(a), _bits(b)), f"call {call}: {name} differs"
            assert not torch.equal(pb, p0)  # the step really ran

        # beyond the built-in limit: refused with a clear message, state untouched
        z = torch.zeros(16, device=DEV)
        rc = lib.sf_adam_update_dp_static(id_b, 3, *HP, 1, z.data_ptr(), peers, world, _lib.SF_GRAD_BF16,
                                          z.data_ptr(), z.data_ptr(), None, max_elems + 1, stream)
        assert rc == _lib.SF_ERR_SIZE
        msg = lib.sf_last_error().decode()
        assert str(max_elems) in msg and "exceeds" in msg
        assert not z.any()
    finally:
        lib.sf_adam_destroy(id_a)
        lib.sf_adam_destroy(id_b)
