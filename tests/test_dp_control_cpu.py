"""Host-side logic of the data-parallel wrapper on CPU: slice arithmetic, and the gloo control
plane (consistency checks, error-flag exchange, timeouts) with world_size 2."""
import os
import tempfile
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from slideformer_b200.shared_data_parallel import ControlPlane, shard_numel, shard_range, slice_vec_n


def test_shard_arithmetic():
    assert shard_numel(0, 8) == 0
    assert shard_numel(19, 2) == 16 and shard_numel(3, 4) == 16
    assert shard_numel(218_112_000, 8) == 27_264_000
    for numel in (0, 1, 3, 16, 17, 19, 1000, 218_112_000, 10**9):
        for world in (1, 2, 3, 4, 8):
            s = shard_numel(numel, world)
            assert s % 16 == 0 and s * world >= numel
            covered = 0
            prev_end = 0
            for r in range(world):
                a, b = shard_range(numel, world, r)
                assert a == min(r * s, numel) and a <= b <= numel and a >= prev_end
                assert a % 16 == 0 or a == numel
                covered += b - a
                prev_end = b
            assert covered == numel
    # the reference test's layers on 2 and 4 ranks
    assert [shard_range(19, 2, r) for r in range(2)] == [(0, 16), (16, 19)]
    assert [shard_range(19, 4, r) for r in range(4)] == [(0, 16), (16, 19), (19, 19), (19, 19)]
    assert [shard_range(3, 2, r) for r in range(2)] == [(0, 3), (3, 3)]


def _worker(rank, world, path, scenario, q):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=30))
    try:
        ctl = ControlPlane(timeout_seconds=5 if scenario == "timeout" else 20)
        if scenario == "agree":
            assert ctl.all_same(("layer", 0, 19))
            assert not ctl.all_same(("layer", rank, 19))          # ranks disagree -> detected by all
            assert ctl.gather(rank * 10) == [r * 10 for r in range(world)]
            assert ctl.any_failed(False) is False
            assert ctl.any_failed(rank == 1) is True               # one rank's failure reaches everyone
            ctl.barrier()
            q.put((rank, "ok"))
        elif scenario == "timeout":
            # rank 1 never joins the barrier: rank 0's wait ends with an error instead of hanging
            if rank == 0:
                try:
                    ctl.barrier()
                    q.put((rank, "no error"))
                except Exception as exc:
                    q.put((rank, "raised:" + type(exc).__name__))
            else:
                q.put((rank, "skipped"))
                import time
                time.sleep(8)
        if scenario != "timeout":
            ctl.close()
    finally:
        if scenario != "timeout":
            dist.destroy_process_group()


def _run(scenario, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, world, os.path.join(d, "rdv"), scenario, q)) for r in range(world)]
        for p in procs:
            p.start()
        out = dict(q.get(timeout=120) for _ in range(world))
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
    return out


def test_control_plane_agreement_and_error_flags():
    assert _run("agree") == {0: "ok", 1: "ok"}


def test_control_plane_barrier_times_out_instead_of_hanging():
    out = _run("timeout")
    assert out[1] == "skipped"
    assert out[0].startswith("raised:"), out


def test_needs_cuda():
    from slideformer_b200.shared_data_parallel import SharedDataParallel
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError, match="Initialize torch.distributed"):
        SharedDataParallel()


def _dp_worker(rank, world, path, q):
    """Every rank plays the sharded update on the CPU with the oracle: gradients exchanged over
    gloo, fp32 rank-order mean of the owned slice, Adam on the slice with the slice-relative
    body/tail boundary, bf16 slices gathered.  Must equal the reference's rank-0 update of the
    whole chunk bit for bit."""
    import numpy as np
    from oracle import oracle as O
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=60))
    try:
        hp = (0.01, 0.8, 0.95, 1e-6, 0.1)
        ok = True
        for numel, chunk in ((19, 5), (1000, 160), (4099, 4099), (65, 48)):
            gen = torch.Generator().manual_seed(numel)
            p0 = torch.linspace(-0.5, 0.5, numel)
            a, b = shard_range(numel, world, rank)
            p_ref, m_ref, v_ref = p0.numpy().copy(), np.zeros(numel, np.float32), np.zeros(numel, np.float32)
            p_my, m_my, v_my = p0.numpy().copy()[a:b], np.zeros(b - a, np.float32), np.zeros(b - a, np.float32)
            ref_opt, my_opt = O.OracleAdam(*hp, True), O.OracleAdam(*hp, True)
            for step in (1, 2, 3):
                rows = torch.stack([(torch.randn(numel, generator=gen) * 0.1).to(torch.bfloat16) for _ in range(world)])
                mine = rows[rank].clone()
                gathered = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(gathered, mine)
                rows_np = np.stack([g.view(torch.int16).numpy().view(np.uint16) for g in gathered])
                for cs in range(0, numel, chunk):
                    ce = min(cs + chunk, numel)
                    # the reference: rank 0 averages the whole chunk and updates it in one call
                    ref_opt.adam_update(step, *hp, True, p_ref[cs:ce], O.rank_mean(np.ascontiguousarray(rows_np[:, cs:ce])),
                                        m_ref[cs:ce], v_ref[cs:ce])
                    # this rank: its part of the chunk, one scalar-state advance per chunk on every rank
                    c = my_opt.scalars(step, *hp, True)
                    lo, hi = max(cs, a), min(ce, b)
                    if hi > lo:
                        mean = O.rank_mean(np.ascontiguousarray(rows_np[:, lo:hi]))
                        O.apply_step(c, p_my[lo - a:hi - a], mean, m_my[lo - a:hi - a], v_my[lo - a:hi - a],
                                     vec_n=slice_vec_n(cs, ce, lo, hi))
            ok = ok and np.array_equal(p_my.view(np.uint32), p_ref[a:b].view(np.uint32))
            ok = ok and np.array_equal(m_my.view(np.uint32), m_ref[a:b].view(np.uint32))
            ok = ok and np.array_equal(v_my.view(np.uint32), v_ref[a:b].view(np.uint32))
        q.put((rank, "ok" if ok else "mismatch"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_update_arithmetic_equals_rank0_reference(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_dp_worker, args=(r, world, os.path.join(d, "rdv"), q)) for r in range(world)]
        for p in procs:
            p.start()
        out = dict(q.get(timeout=180) for _ in range(world))
        for p in procs:
            p.join(timeout=60)
    assert out == {r: "ok" for r in range(world)}


def test_slice_vec_n():
    assert slice_vec_n(0, 19, 0, 16) == 16 and slice_vec_n(0, 19, 16, 19) == 0
    assert slice_vec_n(0, 4099, 0, 2064) == 2064 and slice_vec_n(0, 4099, 2064, 4099) == 4096 - 2064
    assert slice_vec_n(160, 320, 160, 320) == 160 and slice_vec_n(0, 5, 0, 5) == 0
