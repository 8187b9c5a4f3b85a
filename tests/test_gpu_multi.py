"""Multi-GPU data-parallel path: one process per GPU over NCCL, peer-mapped gradient reads.

Needs at least two GPUs; with fewer the tests skip (ranks are never stacked on one GPU).
Expected values come from the CPU oracle: fp32 rank-order mean, then the reference Adam with
the reference's call sequence.  Tolerance: bit-exact (fused and callback modes).
"""
import os
import tempfile

import numpy as np
import pytest
import torch

from golden_cases import REFT, REFTEST_CHUNK, REFTEST_SIZES, reftest_lr

pytestmark = pytest.mark.gpu


def _need(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


def _bits(t):
    return t.detach().cpu().numpy().view(np.uint32)


def _grad(size, peer, step, dtype):
    return ((torch.arange(size) * 0.13 + peer + step * 0.2).sin() * 0.1).to(dtype)


def _np_rows(rows):
    if rows.dtype == torch.bfloat16:
        return rows.view(torch.int16).numpy().view(np.uint16)
    return rows.numpy()


def _worker(rank, world, path, scenario):
    import torch.distributed as dist
    from oracle import oracle as O
    from slideformer_b200 import LayerAdam
    from slideformer_b200.shared_data_parallel import SharedDataParallel

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{path}", rank=rank, world_size=world, device_id=dev)
    try:
        if scenario in ("reftest_callback", "reftest_fused"):
            for dtype in (torch.float32, torch.bfloat16):
                dp = SharedDataParallel(chunk_numel=REFTEST_CHUNK, dtype=dtype, timeout_seconds=60)
                adam = LayerAdam(lr=0.01, betas=(REFT["b1"], REFT["b2"]), eps=REFT["eps"], weight_decay=REFT["wd"])
                orc = O.OracleAdam(0.01, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True)
                exp = []
                for layer, size in enumerate(REFTEST_SIZES):
                    st = dp.register_layer(layer, size)
                    init = torch.linspace(-0.5, 0.5, size)
                    dp.load_full_params(layer, init.to(dev))
                    exp.append([init.numpy().copy(), np.zeros(size, np.float32), np.zeros(size, np.float32)])
                    assert st.exp_avg.numel() == st.exp_avg_sq.numel() == st.shard
                total = torch.tensor([sum(s.end - s.start for s in dp.layers.values())], device=dev)
                dist.all_reduce(total)
                assert total.item() == sum(REFTEST_SIZES)  # exactly one global copy of each moment
                for step in range(1, 6):
                    lr = reftest_lr(step)
                    for layer, size in enumerate(REFTEST_SIZES):
                        st = dp.layers[layer]
                        grads = [_grad(size, peer, step, dtype) for peer in range(world)]
                        rows = _np_rows(torch.stack(grads)) if size else None
                        calls = 0

                        def update(params, g, first, second):
                            nonlocal calls
                            calls += 1
                            adam.step_chunk(params, g, first, second, dict(adam.defaults, step=step, lr=lr))

                        for start in range(0, size, dp.chunk_numel):
                            end = min(start + dp.chunk_numel, size)
                            local = grads[rank][start:end].to(dev)
                            if scenario == "reftest_callback":
                                dp.reduce_chunk(layer, start, end, local, update)
                            else:
                                dp.fused_update(layer, adam, dict(adam.defaults, step=step, lr=lr), start, end, local,
                                                gather=False)
                            mean = O.rank_mean(np.ascontiguousarray(rows[:, start:end]))
                            p, m, v = exp[layer]
                            orc.adam_update(step, lr, REFT["b1"], REFT["b2"], REFT["eps"], REFT["wd"], True,
                                            p[start:end], mean, m[start:end], v[start:end])
                        if scenario == "reftest_callback":
                            assert calls == (size + dp.chunk_numel - 1) // dp.chunk_numel
                        else:
                            dp.all_gather_params(layer)
                        torch.cuda.synchronize()
                        k = st.end - st.start
                        p, m, v = exp[layer]
                        assert np.array_equal(_bits(st.params[:k]), p[st.start:st.end].view(np.uint32)), (layer, step)
                        assert np.array_equal(_bits(st.exp_avg[:k]), m[st.start:st.end].view(np.uint32))
                        assert np.array_equal(_bits(st.exp_avg_sq[:k]), v[st.start:st.end].view(np.uint32))
                        if scenario == "reftest_fused" and size:
                            got = st.bf16[:size].view(torch.int16).cpu().numpy().view(np.uint16)
                            assert np.array_equal(got, O.f32_to_bf16(p))
                dp.barrier()
                dp.close()
        elif scenario in ("medium", "medium_allgather"):
            n = 1_000_003
            hp = (1e-5, 0.9, 0.999, 1e-8, 0.01)
            # default: the update kernel pushes the bf16 weights to every rank; otherwise NCCL all-gather
            dp = SharedDataParallel(chunk_numel=n, dtype=torch.bfloat16, timeout_seconds=60,
                                    push_weights=(scenario == "medium"))
            assert (dp.register_layer(7, 64).peer_bf16 is not None) == (scenario == "medium")
            adam = LayerAdam(lr=hp[0], betas=hp[1:3], eps=hp[3], weight_decay=hp[4])
            orc = O.OracleAdam(*hp, True)
            st = dp.register_layer(0, n)
            gen = torch.Generator().manual_seed(5)
            p0 = torch.randn(n, generator=gen) * 0.02
            dp.load_full_params(0, p0.to(dev))
            p, m, v, o = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
            for step in (1, 2, 3):
                rows = torch.stack([(torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16) for _ in range(world)])
                dp.grad_buffer(0)[:n].copy_(rows[rank].to(dev))
                dp.fused_update(0, adam, dict(adam.defaults, step=step))
                mean = O.rank_mean(_np_rows(rows))
                orc.adam_update(step, *hp, True, p, mean, m, v, o)
            torch.cuda.synchronize()
            k = st.end - st.start
            assert np.array_equal(_bits(st.params[:k]), p[st.start:st.end].view(np.uint32))
            assert np.array_equal(_bits(st.exp_avg[:k]), m[st.start:st.end].view(np.uint32))
            assert np.array_equal(_bits(st.exp_avg_sq[:k]), v[st.start:st.end].view(np.uint32))
            assert np.array_equal(st.bf16[:n].view(torch.int16).cpu().numpy().view(np.uint16), o)  # every rank holds the full layer
            # NCCL variant: bf16 reduction, so only close to the fp32-mean result
            dp2_state = dp.register_layer(1, n)
            dp.load_full_params(1, p0.to(dev))
            adam2 = LayerAdam(lr=hp[0], betas=hp[1:3], eps=hp[3], weight_decay=hp[4])
            gen2 = torch.Generator().manual_seed(5)
            torch.randn(n, generator=gen2)
            rows = torch.stack([(torch.randn(n, generator=gen2) * 1e-3).to(torch.bfloat16) for _ in range(world)])
            dp.grad_buffer(1)[:n].copy_(rows[rank].to(dev))
            dp.nccl_update(1, adam2, dict(adam2.defaults, step=1), slot=1)
            torch.cuda.synchronize()
            ref1 = p0.numpy().copy()
            m1, v1 = np.zeros(n, np.float32), np.zeros(n, np.float32)
            O.OracleAdam(*hp, True).adam_update(1, *hp, True, ref1, O.rank_mean(_np_rows(rows)), m1, v1)
            k = dp2_state.end - dp2_state.start
            got = dp2_state.params[:k].cpu().numpy()
            assert np.allclose(got, ref1[dp2_state.start:dp2_state.end], rtol=0, atol=2.5e-5)  # |step| <= lr, sign may flip on tiny means
            dp.barrier()
            dp.close()
        elif scenario == "nvls":
            # in-switch reduction (multimem): not bit-exact by contract.  Expected values: the fp32
            # rank-order sum rounded once to bf16, divided by world, through the reference update;
            # the last n mod 8 elements take the exact peer path.
            from torch._C._distributed_c10d import _SymmetricMemory
            if not _SymmetricMemory.has_multicast_support(torch._C._autograd.DeviceType.CUDA, rank):
                return
            from slideformer_b200.shared_data_parallel import ShardedLayerAdam
            n = 1_000_003
            hp = (1e-5, 0.9, 0.999, 1e-8, 0.01)
            sh = ShardedLayerAdam(numel=n, device=dev, mode="nvls", lr=hp[0], betas=hp[1:3], eps=hp[3], weight_decay=hp[4])
            gen = torch.Generator().manual_seed(17)
            p0 = torch.randn(n, generator=gen) * 0.02
            sh.dp.load_full_params(0, p0.to(dev))
            orc = O.OracleAdam(*hp, True)
            p, m, v, o = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
            st = sh.state
            for step in (1, 2, 3):
                rows = torch.stack([(torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16) for _ in range(world)])
                sh.grad_buffer(0).copy_(rows[rank].to(dev))
                sh.step(0)
                exact = O.rank_mean(_np_rows(rows))
                summed = exact * np.float32(world)            # world is a power of two here: exact
                mean = O.bf16_to_f32(O.f32_to_bf16(summed)) / np.float32(world)
                # per owner the multicast path covers its slice up to the last multiple of 8 below
                # the reference call's 16-lane boundary; beyond that the exact peer path runs
                from slideformer_b200.shared_data_parallel import shard_range, slice_vec_n
                for r in range(world):
                    a, b = shard_range(n, world, r)
                    cut = a + (slice_vec_n(0, n, a, b) & ~7)
                    mean[cut:b] = exact[cut:b]
                orc.adam_update(step, *hp, True, p, mean.astype(np.float32), m, v, o)
            torch.cuda.synchronize()
            k = st.end - st.start
            got_p, got_m = st.params[:k].cpu().numpy(), st.exp_avg[:k].cpu().numpy()
            want_p, want_m = p[st.start:st.end], m[st.start:st.end]
            # tolerance of the mode: the mean may be off by half a bf16 ulp of the sum
            gmax = float(np.max(np.abs(mean)))
            assert np.max(np.abs(got_m - want_m)) <= 3 * 2 ** -8 * gmax, np.max(np.abs(got_m - want_m))
            assert np.max(np.abs(got_p - want_p)) <= 3 * 2 * hp[0]
            # (how the switch rounds is not documented: about half of the fp32 results carry the same
            # bits as this model of it, so only the tolerance above is asserted)
            full = st.bf16[:n].view(torch.int16).cpu().numpy().view(np.uint16)
            assert float(np.mean(full == o)) > 0.99                      # every rank holds the whole layer
            mine = st.bf16[st.start:st.end].view(torch.int16).cpu().numpy().view(np.uint16)
            assert np.array_equal(mine, O.f32_to_bf16(got_p))            # and the pushed copy is the cast of p
            sh.dp.barrier()
            sh.close()
        elif scenario == "host_stepper":
            # gradients in pinned host memory on every rank, bf16 slices back to host, pieces pipelined
            from slideformer_b200.shared_data_parallel import ShardedHostStepper, ShardedLayerAdam
            n = 300_000 + 37
            hp = (1e-5, 0.9, 0.999, 1e-8, 0.01)
            sh = ShardedLayerAdam(numel=n, device=dev, mode="fused", lr=hp[0], betas=hp[1:3], eps=hp[3], weight_decay=hp[4])
            gen = torch.Generator().manual_seed(11)
            p0 = torch.randn(n, generator=gen) * 0.02
            sh.dp.load_full_params(0, p0.to(dev))
            stepper = ShardedHostStepper(sh, chunk_numel=65536, min_chunk_numel=16384)
            assert len(stepper.chunks) > 4
            orc = O.OracleAdam(*hp, True)
            p, m, v, o = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
            st = sh.state
            k = st.end - st.start
            out_host = torch.zeros(max(k, 1), dtype=torch.bfloat16).pin_memory()
            for step in (1, 2, 3, 4):
                rows = torch.stack([(torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16) for _ in range(world)])
                g_host = rows[rank].clone().pin_memory()
                stepper.step(g_host, out_host, join=(step % 2 == 0))   # odd steps overlap with the next one
                mean = O.rank_mean(_np_rows(rows))
                for a, b in stepper.chunks:                              # one reference call per piece
                    orc.adam_update(step, *hp, True, p[a:b], mean[a:b], m[a:b], v[a:b], o[a:b])
                if step % 2 == 1:
                    torch.cuda.synchronize()   # g_host of this step is dropped next: let its uploads finish
            stepper.join()
            torch.cuda.synchronize()
            assert np.array_equal(_bits(st.params[:k]), p[st.start:st.end].view(np.uint32))
            assert np.array_equal(_bits(st.exp_avg[:k]), m[st.start:st.end].view(np.uint32))
            assert np.array_equal(_bits(st.exp_avg_sq[:k]), v[st.start:st.end].view(np.uint32))
            assert np.array_equal(out_host[:k].view(torch.int16).numpy().view(np.uint16), o[st.start:st.end])
            assert np.array_equal(st.bf16[:n].view(torch.int16).cpu().numpy().view(np.uint16), o)
            sh.dp.barrier()
            sh.close()
        elif scenario == "error":
            dp = SharedDataParallel(chunk_numel=64, dtype=torch.bfloat16, timeout_seconds=60)
            dp.register_layer(0, 64)

            def update(params, g, first, second):
                if rank == 1:
                    raise ValueError("injected host-side failure")

            raised = False
            try:
                dp.reduce_chunk(0, 0, 64, torch.zeros(64, dtype=torch.bfloat16, device=dev), update)
            except RuntimeError as exc:
                raised = "distributed update failed" in str(exc)
            assert raised, f"rank {rank} did not see the failure"
            try:
                dp.raise_if_failed()
                raise AssertionError("error slot was cleared")
            except RuntimeError:
                pass
            with pytest.raises(ValueError, match="Invalid gradient chunk"):
                dp.error = None
                dp.reduce_chunk(0, 0, 65, torch.zeros(65, dtype=torch.bfloat16, device=dev), update)
            # bad arguments on ONE rank: that rank gets its ValueError, the other learns of it on the
            # host, and both have enqueued the same number of stream barriers (nothing hangs)
            adam = LayerAdam(lr=1e-3)
            try:
                dp.fused_update(0, adam, dict(adam.defaults, step=1), 0, 65 if rank == 1 else 64, check_errors=True)
                outcome = "ok"
            except ValueError:
                outcome = "value"
            except RuntimeError as exc:
                outcome = "runtime" if "distributed update failed" in str(exc) else "other"
            assert outcome == ("value" if rank == 1 else "runtime"), (rank, outcome)
            dp.error = None
            dp.fused_update(0, adam, dict(adam.defaults, step=2), 0, 64, check_errors=True)   # and the next call works
            torch.cuda.synchronize()
        elif scenario == "mismatch":
            dp = SharedDataParallel(chunk_numel=64, dtype=torch.bfloat16, timeout_seconds=60)
            with pytest.raises(ValueError, match="identical layers"):
                dp.register_layer(0, 64 + rank)
            dp.register_layer(1, 64)
            with pytest.raises(ValueError, match="identical layers"):
                dp.register_layer(1, 64)
            dp.barrier()
            dp.close()
    finally:
        dist.destroy_process_group()


def _run(world, scenario):
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), scenario), nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("scenario", ["reftest_callback", "reftest_fused"])
def test_reference_dp_sequence_sharded(world, scenario):
    _need(world)
    _run(world, scenario)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("scenario", ["medium", "medium_allgather"])
def test_medium_layer_fused_and_nccl(world, scenario):
    _need(world)
    _run(world, scenario)


def test_nvls_mode_two_ranks():
    """Needs NVLink multicast (NVSwitch); returns quietly where the driver reports none."""
    _need(2)
    _run(2, "nvls")


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_host_stepper(world):
    _need(world)
    _run(world, "host_stepper")


def test_host_failure_reaches_every_rank():
    _need(2)
    _run(2, "error")


def test_registration_mismatch_is_detected():
    _need(2)
    _run(2, "mismatch")
