"""The engine with optimizer state sharded over ranks (SlideFormerOffloader(shared_dp=...)).

Two ranks train the same tiny model on different batches.  After every step each rank's bf16
weights must be identical across ranks (all-gather), and equal to a single-process run whose
gradient is the fp32 rank-order mean of the two ranks' gradients fed through the CPU oracle.
Needs two GPUs.
"""
import os
import tempfile

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def _worker(rank, world, path, mode):
    import torch.distributed as dist
    from oracle import oracle as O
    from slideformer_b200.model_compat import build_random_model
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    from slideformer_b200.shared_data_parallel import SharedDataParallel

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{path}", rank=rank, world_size=world, device_id=dev)
    try:
        dp = SharedDataParallel(dtype=torch.bfloat16, exchange_slots=2, timeout_seconds=60)
        if mode == "meta":
            # skeleton on the meta device, weights created per unit inside the engine, window mode
            model = build_random_model("llama-tiny", dev, torch.bfloat16, seed=3, meta=True)
            eng = SlideFormerOffloader(model, dev, torch.bfloat16, enable_timing=False, enable_memory_stats=False,
                                       optimizer_kwargs=dict(HP), auto_backward_in_forward=True, shared_dp=dp,
                                       weight_window=True)
            gen = torch.Generator().manual_seed(100 + rank)
            losses = []
            for step in range(4):
                ids = torch.randint(0, eng.config.vocab_size, (2, 32), generator=torch.Generator().manual_seed(7)).to(dev)
                losses.append(float(eng(ids, labels=ids).loss.detach()))
            assert all(np.isfinite(losses)) and losses[-1] < losses[0], losses   # same batch every step: loss falls
            # save from the slices (collective) and reload on rank 0: same logits as the engine
            import tempfile as _tf
            ids = torch.randint(0, eng.config.vocab_size, (2, 16), generator=torch.Generator().manual_seed(8)).to(dev)
            with torch.no_grad():
                mine = eng(ids).logits.float()
            out_dir = os.path.join(os.path.dirname(path), "saved")
            eng.save_pretrained(out_dir)
            if rank == 0:
                from transformers import AutoModelForCausalLM
                again = AutoModelForCausalLM.from_pretrained(out_dir, dtype=torch.bfloat16).to(dev)
                with torch.no_grad():
                    ref = again(input_ids=ids).logits.float()
                assert torch.allclose(mine, ref, atol=2e-2, rtol=0), (mine - ref).abs().max().item()
            eng.close()          # what the benchmark does between models: every buffer of the engine is dropped
            assert all(u._params_flat is None and u._dp_state is None for u in eng.transformer_layers)
            dp.barrier()
            dp.close()
            return
        model = build_random_model("llama-tiny", dev, torch.bfloat16, seed=3)
        init_full = {}
        eng = SlideFormerOffloader(model, dev, torch.bfloat16, enable_timing=False, enable_memory_stats=False,
                                   optimizer_kwargs=dict(HP), auto_backward_in_forward=False, shared_dp=dp,
                                   weight_window=(mode == "window"), update_chunk=(8192 if mode == "resident_chunked" else None),
                                   batch_small_units=(False if mode == "resident_per_unit" else None))
        assert eng.batch_small_units == (mode in ("resident", "resident_chunked"))
        units = eng.transformer_layers
        # expected state, full layers, kept on every rank
        exp = {}
        for u in units:
            if mode == "window":
                tmp = torch.empty(u._dp_state.shard * world, dtype=torch.bfloat16, device=dev)
                dp.gather_weights(u.layer_idx, tmp)
                full = tmp[: u.total_size].float().cpu().numpy().copy()
            else:
                full = u._bf16_flat.float().cpu().numpy().copy()   # masters were created from the bf16 init
            n = u.total_size
            exp[u.layer_idx] = [full, np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)]
        orc = O.OracleAdam(HP["lr"], *HP["betas"], HP["eps"], HP["weight_decay"], True)
        grabbed = {}
        for u in units:
            orig = u.update_params

            def wrapped(u=u, orig=orig):
                if u._unit is not None:
                    grabbed[u.layer_idx] = u._unit["grad"][: u.total_size].clone()
                return orig()
            u.update_params = wrapped
        gen = torch.Generator().manual_seed(100 + rank)
        for step in (1, 2, 3):
            ids = torch.randint(0, eng.config.vocab_size, (2, 32), generator=gen).to(dev)
            grabbed.clear()
            eng(ids, labels=ids).loss.backward()
            eng.wait_for_completion()
            for idx in range(len(units) - 1, -1, -1):
                u = units[idx]
                n = u.total_size
                mine = grabbed[idx]
                rows = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(rows, mine)
                rows_np = np.stack([r.view(torch.int16).cpu().numpy().view(np.uint16) for r in rows])
                mean = O.rank_mean(rows_np)
                p, m, v, o = exp[idx]
                for cs in range(0, n, u.update_chunk):
                    ce = min(cs + u.update_chunk, n)
                    orc.adam_update(step, HP["lr"], *HP["betas"], HP["eps"], HP["weight_decay"], True,
                                    p[cs:ce], mean[cs:ce], m[cs:ce], v[cs:ce], o[cs:ce])
                st = u._dp_state
                k = st.end - st.start
                assert np.array_equal(st.params[:k].cpu().numpy().view(np.uint32), p[st.start:st.end].view(np.uint32)), (step, idx)
                assert np.array_equal(st.exp_avg[:k].cpu().numpy().view(np.uint32), m[st.start:st.end].view(np.uint32))
                if mode == "window":
                    got = st.bf16_shard[:k].view(torch.int16).cpu().numpy().view(np.uint16)
                    assert np.array_equal(got, o[st.start:st.end]), (step, idx)
                else:
                    assert np.array_equal(u._bf16_flat.view(torch.int16).cpu().numpy().view(np.uint16), o), (step, idx)
        eng.close()
        dp.barrier()
        dp.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["resident", "resident_chunked", "resident_per_unit", "window", "meta"])
def test_sharded_engine_two_ranks(mode):
    """resident: every rank keeps all bf16 layers (weights pushed by the update kernel), all units
    updated by one multi-segment launch after backward; resident_chunked: the same with units cut
    into several reference calls; resident_per_unit: one launch and barrier pair per unit;
    window: only bf16 slices are kept and layers are all-gathered into window units on demand;
    meta: window mode on a model whose weights are created per unit (never whole on one GPU)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, os.path.join(d, "rdv"), mode), nprocs=2, join=True)
