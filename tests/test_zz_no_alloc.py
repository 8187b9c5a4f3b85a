"""The entry point that allocates nothing (sf_adam_update_dp_static).

Some callers sit in the steady state of a training step -- the per-chunk gradient reduction on
the optimizer thread while backward is still running -- where all of HBM is already spoken for
and a cudaMalloc would either fail or stall the device.  For them the library stages the fp32
gradient mean in an array that is part of its own image.  This test drives that entry point
through the C ABI and requires the same bits as (a) the CPU oracle (fp32 rank-order mean, then
the reference Adam call) and (b) the existing pair of entry points (sf_dp_mean into a caller
buffer + sf_adam_update), on two calls in a row so that whatever the first call leaves in the
shared array cannot leak into the second; it also checks that the device's free memory does not
move across a call.  It lives in a file that sorts last, so a run that stops at the first failure
has already run everything else.
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


def _np_rows(rows):
    stacked = torch.stack([r.cpu() for r in rows])
    if stacked.dtype == torch.bfloat16:
        return stacked.view(torch.int16).numpy().view(np.uint16)
    return stacked.numpy()


@pytest.mark.parametrize("gdtype,off", [(torch.bfloat16, 0), (torch.float32, 0), (torch.bfloat16, 1)])
def test_static_scratch_matches_oracle_and_existing_entry_points_twice(gdtype, off, oracle):
    """off = 1 shifts the peers' gradient buffers by one element, so the mean runs on the
    one-element-at-a-time path."""
    from slideformer_b200 import _lib
    lib = _lib.load()
    world = 3
    max_elems = _lib.SF_STATIC_SCRATCH_MAX_ELEMS
    assert max_elems == 4 << 20
    gcode = _lib.SF_GRAD_BF16 if gdtype == torch.bfloat16 else _lib.SF_GRAD_F32
    esize = 2 if gdtype == torch.bfloat16 else 4
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(2024)
    id_a, id_b = 880001, 880002
    _lib.check(lib.sf_adam_create(id_a, *HP, 1, 0))
    _lib.check(lib.sf_adam_create(id_b, *HP, 1, 0))
    orc = oracle.OracleAdam(*HP, True)
    try:
        # the second call is shorter than the first: stale values beyond its n stay in the array
        for call, n in enumerate(((1 << 20) + 13, 300_007), start=1):
            p0 = torch.randn(n, generator=gen) * 0.02
            m0 = torch.randn(n, generator=gen) * 1e-4
            v0 = torch.rand(n, generator=gen) * 1e-6
            rows = [(torch.randn(n + off, generator=gen) * 1e-3).to(gdtype).to(DEV) for _ in range(world)]
            peers = (C.c_void_p * world)(*[r.data_ptr() + off * esize for r in rows])

            # CPU oracle
            po, mo, vo, oo = p0.numpy().copy(), m0.numpy().copy(), v0.numpy().copy(), np.zeros(n, np.uint16)
            mean_o = oracle.rank_mean(np.ascontiguousarray(_np_rows(rows)[:, off:]))
            orc.adam_update(call, *HP, True, po, mean_o, mo, vo, oo)

            # existing entry points, caller-owned fp32 staging buffer
            pa, ma, va = p0.to(DEV), m0.to(DEV), v0.to(DEV)
            oa = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
            mean = torch.empty(n, device=DEV)
            _lib.check(lib.sf_dp_mean(peers, world, gcode, mean.data_ptr(), n, stream))
            _lib.check(lib.sf_adam_update(id_a, call, *HP, 1, pa.data_ptr(), mean.data_ptr(), _lib.SF_GRAD_F32,
                                          ma.data_ptr(), va.data_ptr(), oa.data_ptr(), n, stream))

            # the new entry point: no staging buffer passed, nothing allocated
            pb, mb, vb = p0.to(DEV), m0.to(DEV), v0.to(DEV)
            ob = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
            torch.cuda.synchronize()
            torch_before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0] if call > 1 else None   # call 1 loads the module / symbol
            _lib.check(lib.sf_adam_update_dp_static(id_b, call, *HP, 1, pb.data_ptr(), peers, world, gcode,
                                                    mb.data_ptr(), vb.data_ptr(), ob.data_ptr(), n, stream))
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == torch_before
            if free_before is not None:
                assert torch.cuda.mem_get_info()[0] == free_before, "device memory moved across the call"
            for name, a, b in (("p", pa, pb), ("m", ma, mb), ("v", va, vb), ("bf16", oa, ob)):
                assert torch.equal(_bits(a), _bits(b)), f"call {call}: {name} differs from sf_dp_mean + sf_adam_update"
            for name, a, b in (("p", po, pb), ("m", mo, mb), ("v", vo, vb)):
                assert np.array_equal(a.view(np.uint32), b.cpu().numpy().view(np.uint32)), f"call {call}: {name} differs from the oracle"
            assert np.array_equal(oo, ob.view(torch.int16).cpu().numpy().view(np.uint16)), f"call {call}: bf16 differs from the oracle"
            assert np.array_equal(mean_o.view(np.uint32), mean.cpu().numpy().view(np.uint32)), f"call {call}: sf_dp_mean differs from the oracle"
            assert not torch.equal(pb.cpu(), p0)  # the step really ran

        # beyond the built-in limit: refused with a clear message, state untouched
        z = torch.zeros(16, device=DEV)
        rc = lib.sf_adam_update_dp_static(id_b, 3, *HP, 1, z.data_ptr(), peers, world, gcode,
                                          z.data_ptr(), z.data_ptr(), None, max_elems + 1, stream)
        assert rc == _lib.SF_ERR_SIZE
        msg = lib.sf_last_error().decode()
        assert str(max_elems) in msg and "exceeds" in msg
        assert not z.any()
    finally:
        lib.sf_adam_destroy(id_a)
        lib.sf_adam_destroy(id_b)
