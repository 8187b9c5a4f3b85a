"""Fine-tune throughput of the layer-sliding engine on a random-init model (tokens/s).

    python -m slideformer_b200.finetune_bench --model gpt2-small --batch 8 --seq 1024
    python -m slideformer_b200.finetune_bench --model llama3.1-8b --batch 8 --seq 1024 [--state-device host]
    torchrun --nproc-per-node N -m slideformer_b200.finetune_bench --model gpt2-small --dp     # sharded state

Counterpart of the reference's scripts/main_bench.py measurement loop (warm-up steps, timed
steps, tokens/s and TFLOPS by the Megatron formula of utils/metric.py:4-57) on synthetic data:
token ids uniform in [0, vocab), labels = inputs (the engine shifts them).  Every step uploads
its batch from pinned host memory and downloads the loss, inside the timed region.
Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch


def model_flops_per_step(cfg, batch, seq):
    """Forward + backward FLOPs of one step, dense decoder (utils/metric.py:4-57); 3x forward,
    without the recompute of activation checkpointing."""
    if getattr(cfg, "model_type", "") == "gpt2":
        h, L, V, inter, heads, kv = cfg.n_embd, cfg.n_layer, cfg.vocab_size, 4 * cfg.n_embd, cfg.n_head, cfg.n_head
        gated = 1.0
    else:
        h, L, V, inter = cfg.hidden_size, cfg.num_hidden_layers, cfg.vocab_size, cfg.intermediate_size
        heads, kv = cfg.num_attention_heads, cfg.num_key_value_heads
        gated = 1.5
    return 12 * batch * seq * L * h * h * ((1 + kv / heads + seq / h) + (inter / h) * gated + V / (2 * L * h))


def run_finetune(model_name: str, batch: int, seq: int, steps: int, warmup: int, dev, world: int = 1, rank: int = 0,
                 dp=None, layers=None, state_device: str = "hbm", activation_offload: str = "hbm",
                 activation_checkpoint: bool = True, double_buffer: bool = False, lr: float = 1e-5,
                 weight_window: bool = False, meta: bool = False, hbm_state_budget_gb=None) -> dict:
    """Build the random-init model, run warm-up + timed steps, return the result line as a dict.
    `dp` is a SharedDataParallel (state sharded over the ranks of the default process group) or None."""
    from slideformer_b200 import _lib
    from slideformer_b200.model_compat import build_random_model
    from slideformer_b200.offload_transformer import SlideFormerOffloader

    lib = _lib.load()
    torch.cuda.reset_peak_memory_stats(dev)
    t_build = time.perf_counter()
    model = build_random_model(model_name, dev, torch.bfloat16, seed=0, num_layers=layers, meta=meta)
    engine = SlideFormerOffloader(
        model, dev, torch.bfloat16, double_buffer=double_buffer, enable_timing=True, enable_memory_stats=False,
        optimizer_kwargs=dict(lr=lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01),
        shared_dp=dp, state_device=state_device, activation_offload=activation_offload,
        activation_checkpoint=activation_checkpoint, weight_window=weight_window,
        hbm_state_budget_gb=hbm_state_budget_gb)
    torch.cuda.synchronize()
    placement = engine.state_placement
    build_s = time.perf_counter() - t_build

    vocab = model.config.vocab_size
    gen = torch.Generator().manual_seed(1234 + rank)
    nb = 4
    host_ids = [torch.randint(0, vocab, (batch, seq), generator=gen).pin_memory() for _ in range(nb)]
    loss_host = torch.zeros(1).pin_memory()

    def step(i):
        ids = host_ids[i % nb].to(dev, non_blocking=True)
        out = engine(ids, labels=ids)
        loss_host.copy_(out.loss.detach().float().reshape(1), non_blocking=True)
        return out

    losses = []
    for i in range(warmup):
        step(i)
        torch.cuda.synchronize()
        losses.append(float(loss_host.item()))
    if dp is not None:
        dp.barrier()
    torch.cuda.synchronize()
    l0 = lib.sf_launch_count()
    for u in engine.transformer_layers:
        u.host_update_seconds = 0.0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for i in range(steps):
        step(i)
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    losses.append(float(loss_host.item()))
    ms = max(a.elapsed_time(b), wall * 1e3) / steps
    if dp is not None:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    tokens = batch * seq * world
    upd = engine.parameter_update_ms()
    flops = model_flops_per_step(model.config, batch, seq) * world
    line = {"metric": "fine-tune tokens/s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{model_name} full fine-tune, layer sliding", "global_batch": batch * world,
                       "seq_len": seq, "state_device": state_device, "activation_offload": activation_offload,
                       "activation_checkpoint": activation_checkpoint, "weight_window": weight_window,
                       "hbm_state_budget_gb": hbm_state_budget_gb,
                       "units_with_state_in_hbm": (placement.count("hbm") if placement is not None else None),
                       "units": len(engine.transformer_layers),
                       "parallelism": f"dp{world} sharded state" if dp is not None else "single GPU"},
            "model_tflops": flops / (ms * 1e-3) / 1e12, "params": sum(u.total_size for u in engine.transformer_layers),
            "optimizer_ms_per_step": sum(upd.values()),
            "optimizer_host_enqueue_ms_per_step": 1e3 * sum(u.host_update_seconds for u in engine.transformer_layers) / steps, "optimizer_ms_decoder_layer": upd.get(1),
            "gpu_launches": int(lib.sf_launch_count() - l0), "loss_first": losses[0] if losses else None,
            "loss_last": losses[-1], "build_seconds": build_s,
            "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 2**30,
            "e2e": {"h2d_bytes_per_step": batch * seq * 8 * world, "d2h_bytes_per_step": 4 * world}}
    engine.close()
    del engine, model
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return line


CSV_FIELDS = ["Model", "Sequence_Length", "Batch_Size", "Precision", "GPUs", "State_Device", "Activation_Offload",
              "Activation_Checkpoint", "Avg_Time", "Avg_Tokens_Per_Second", "Avg_TFLOPS", "Max_CUDA_Memory_Allocated_MB"]


def append_result_to_csv(path: str, line: dict) -> None:
    """One row per run, in the spirit of the reference's results file (scripts/main_bench.py:65-95):
    time per step, tokens/s, model TFLOPS and peak CUDA memory next to the run's settings."""
    import csv
    cfg = line["config"]
    new_file = not os.path.isfile(path)
    with open(path, "a", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=CSV_FIELDS)
        if new_file:
            w.writeheader()
        w.writerow({"Model": cfg["workload"].split()[0], "Sequence_Length": cfg["seq_len"],
                    "Batch_Size": cfg["global_batch"] // line["n_gpus"], "Precision": line["dtype"],
                    "GPUs": line["n_gpus"], "State_Device": cfg["state_device"],
                    "Activation_Offload": cfg["activation_offload"], "Activation_Checkpoint": cfg["activation_checkpoint"],
                    "Avg_Time": f"{line['ms_per_step'] / 1e3:.4f}", "Avg_Tokens_Per_Second": f"{line['value']:.1f}",
                    "Avg_TFLOPS": f"{line['model_tflops']:.2f}",
                    "Max_CUDA_Memory_Allocated_MB": f"{line['max_memory_gb'] * 1024:.1f}"})


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-small")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None, help="override the number of decoder layers")
    ap.add_argument("--state-device", default="hbm", choices=["hbm", "host", "auto"])
    ap.add_argument("--hbm-state-budget-gb", type=float, default=None,
                    help="with --state-device auto: HBM the fp32 state may take; units beyond it keep their state in pinned host memory")
    ap.add_argument("--activation-offload", default="hbm", choices=["hbm", "host"])
    ap.add_argument("--no-ckpt", action="store_true", help="keep all activations instead of checkpointing each layer")
    ap.add_argument("--double-buffer", action="store_true")
    ap.add_argument("--dp", action="store_true", help="shard optimizer state over all ranks (launch with torchrun)")
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--weight-window", action="store_true",
                    help="keep only bf16 slices resident and all-gather each layer into a window unit before it runs")
    ap.add_argument("--meta", action="store_true", help="build the model skeleton on the meta device (large models)")
    ap.add_argument("--csv", metavar="FILE", help="also append the result as one CSV row")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dp = None
    if args.dp or world > 1:
        import torch.distributed as dist
        from slideformer_b200.shared_data_parallel import SharedDataParallel
        dist.init_process_group("nccl", device_id=dev)
        dp = SharedDataParallel(dtype=torch.bfloat16, exchange_slots=3 if args.double_buffer else 2)
    line = run_finetune(args.model, args.batch, args.seq, args.steps, args.warmup, dev, world, rank, dp, args.layers,
                        args.state_device, args.activation_offload, not args.no_ckpt, args.double_buffer, args.lr,
                        args.weight_window, args.meta, args.hbm_state_budget_gb)
    if rank == 0:
        print(json.dumps(line))
        if args.csv:
            append_result_to_csv(args.csv, line)
    if dp is not None:
        dp.close()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
