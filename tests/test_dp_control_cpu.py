"""Host-side logic of the data-parallel wrapper on CPU: slice arithmetic, and the gloo control
plane (consistency checks, error-flag exchange, timeouts) with world_size 2."""
import os
import tempfile
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from slideformer_b200.shared_data_parallel import ControlPlane, shard_numel, shard_range


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
