"""Data-parallel fine-tuning launcher: one rank per GPU, optimizer state sharded 1/N in HBM.

    python -m slideformer_b200.main_dp --tiny                        # single GPU smoke run
    torchrun --nproc-per-node N -m slideformer_b200.main_dp --tiny [--tied] [--double-buffer]
    torchrun --nproc-per-node N -m slideformer_b200.main_dp --model CKPT_DIR --tokens ids.pt

The command line follows the reference's multi_gpu/scripts/main_dp.py so existing job scripts
keep working (`--cpu-threads` is accepted and ignored: no CPU thread runs the optimizer here).
`--tiny` reproduces that script's self-check (main_dp.py:55-61,117-124): a random two-layer
Llama is trained for a few steps, after which every unit's fp32 master weights must be finite
and different from their initial values and each unit must have taken exactly one optimizer
step per training step.
"""
from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass
from typing import Iterator, List, Optional

import torch
import torch.distributed as dist

TINY_SHAPE = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2)


@dataclass
class Ranks:
    rank: int
    world: int
    device: torch.device

    @property
    def distributed(self) -> bool:
        return self.world > 1


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(prog="slideformer_b200.main_dp", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    what = ap.add_mutually_exclusive_group(required=True)
    what.add_argument("--tiny", action="store_true", help="train a random two-layer Llama on synthetic tokens and self-check")
    what.add_argument("--model", metavar="DIR", help="Hugging Face checkpoint directory on local disk")
    ap.add_argument("--tokens", metavar="FILE", help="torch.save'd int64 tensor [num_sequences, seq_len] (required with --model)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--batch-size", type=int, default=1, help="sequences per rank and step")
    ap.add_argument("--seq-length", type=int, default=32, help="length of the synthetic sequences of --tiny")
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--warmup-steps", type=int, default=0,
                    help="with --total-steps: linear warm-up then cosine decay of the learning rate")
    ap.add_argument("--total-steps", type=int, default=0, help="length of the cosine schedule (0 = constant lr)")
    ap.add_argument("--clip-norm", type=float, default=0.0,
                    help="clip the global gradient norm to this value, using the norm measured by the previous step's "
                         "update kernels (0 = off)")
    ap.add_argument("--chunk-numel", type=int, default=1 << 25, help="elements per optimizer call")
    ap.add_argument("--double-buffer", action="store_true", help="three gradient units instead of two")
    ap.add_argument("--tied", action="store_true", help="--tiny with tied input/output embeddings")
    ap.add_argument("--attn-implementation", default="sdpa", choices=("eager", "sdpa", "flash_attention_2"))
    ap.add_argument("--save-model", metavar="DIR", help="write the final weights (optimizer state is not saved)")
    ap.add_argument("--cpu-threads", type=int, default=1, help="ignored; kept for command-line compatibility")
    ns = ap.parse_args(argv)
    for name in ("steps", "batch_size", "chunk_numel"):
        if getattr(ns, name) < 1:
            ap.error(f"--{name.replace('_', '-')} must be at least 1")
    if ns.seq_length < 2:
        ap.error("--seq-length must be at least 2")
    if ns.model and not ns.tokens:
        ap.error("--model needs --tokens (synthetic tokens are only generated for --tiny)")
    return ns


def join_ranks() -> Ranks:
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world == 1:
        return Ranks(0, 1, device)
    if int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
        raise ValueError("all ranks must run on one node")
    dist.init_process_group("nccl", device_id=device)
    return Ranks(dist.get_rank(), world, device)


def make_model(ns: argparse.Namespace):
    torch.manual_seed(1234)   # identical initial weights on every rank
    if ns.tiny:
        from transformers import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig(**TINY_SHAPE, max_position_embeddings=max(128, ns.seq_length), attention_dropout=0.0,
                          tie_word_embeddings=ns.tied, attn_implementation=ns.attn_implementation, use_cache=False)
        return LlamaForCausalLM(cfg).to(torch.bfloat16)
    from transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(ns.model, dtype=torch.bfloat16, attn_implementation=ns.attn_implementation)
    model.config.use_cache = False
    return model


def load_sequences(ns: argparse.Namespace, vocab: int, world: int) -> torch.Tensor:
    if not ns.tokens:
        g = torch.Generator().manual_seed(4321)
        return torch.randint(vocab, (ns.steps * world * ns.batch_size, ns.seq_length), generator=g)
    seqs = torch.load(ns.tokens, map_location="cpu", weights_only=True)
    good = isinstance(seqs, torch.Tensor) and seqs.dtype == torch.int64 and seqs.ndim == 2 and seqs.shape[1] >= 2
    if not good:
        raise ValueError("--tokens must hold a 2-D int64 tensor with at least two tokens per sequence")
    if seqs.numel() == 0 or int(seqs.min()) < 0 or int(seqs.max()) >= vocab:
        raise ValueError("token ids must be non-empty and inside the model's vocabulary")
    return seqs


def batches(seqs: torch.Tensor, ranks: Ranks, per_rank: int) -> Iterator[torch.Tensor]:
    """Endless stream of this rank's batches: every epoch draws a fresh permutation (same on all
    ranks) and rank r takes sequences r, r + world, ... of it, dropping the ragged end."""
    group = per_rank * ranks.world
    usable = (seqs.shape[0] // group) * group
    if usable == 0:
        raise ValueError("the token file is too small for one full batch on every rank")
    epoch = 0
    while True:
        order = torch.randperm(seqs.shape[0], generator=torch.Generator().manual_seed(epoch))[:usable]
        mine = order[ranks.rank::ranks.world]
        for lo in range(0, mine.numel(), per_rank):
            yield seqs[mine[lo:lo + per_rank]]
        epoch += 1


def all_ranks_finite(x: torch.Tensor, ranks: Ranks) -> bool:
    flag = torch.isfinite(x.detach()).all().to(torch.int32)
    if ranks.distributed:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def mean_over_ranks(x: torch.Tensor, ranks: Ranks) -> float:
    y = x.detach().float().clone()
    if ranks.distributed:
        dist.all_reduce(y)
        y /= ranks.world
    return float(y.item())


def owned_master_weights(engine) -> List[torch.Tensor]:
    """The fp32 master weights this rank owns, one flat tensor per unit."""
    out = []
    for unit in engine.transformer_layers:
        st = unit._dp_state
        out.append(unit._params_flat[: (st.end - st.start) if st is not None else unit.total_size])
    return out


def self_check(engine, before: List[torch.Tensor], steps_done: int, dp) -> None:
    for unit, old, new in zip(engine.transformer_layers, before, owned_master_weights(engine)):
        if new.numel() and (torch.equal(old, new) or not bool(torch.isfinite(new).all())):
            raise RuntimeError(f"unit {unit.layer_idx}: master weights unchanged or not finite after training")
        taken = unit._dp_state.step if dp is not None else engine.layer_optimizer.param_groups[unit.layer_idx]["step"]
        if taken != steps_done:
            raise RuntimeError(f"unit {unit.layer_idx}: {taken} optimizer steps for {steps_done} training steps")


def main(argv=None) -> int:
    ns = parse_args(argv)
    ranks = join_ranks()
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    from slideformer_b200.shared_data_parallel import SharedDataParallel

    model = make_model(ns)
    stream = batches(load_sequences(ns, model.config.vocab_size, ranks.world), ranks, ns.batch_size)
    dp: Optional[SharedDataParallel] = None
    if ranks.distributed:
        dp = SharedDataParallel(chunk_numel=ns.chunk_numel, dtype=torch.bfloat16,
                                exchange_slots=3 if ns.double_buffer else 2)
    engine = SlideFormerOffloader(model, ranks.device, torch.bfloat16, double_buffer=ns.double_buffer,
                                  enable_timing=False, enable_memory_stats=False, auto_backward_in_forward=False,
                                  shared_dp=dp, update_chunk=ns.chunk_numel,
                                  optimizer_kwargs={"lr": ns.lr, "weight_decay": 0.01, "fp32_optimizer_state": True})
    engine.train()
    before = [w.clone() for w in owned_master_weights(engine)] if ns.tiny else []
    torch.manual_seed(1234 + ranks.rank)   # anything stochastic from here on differs per rank

    sched = None
    if ns.total_steps > 0:
        from slideformer_b200.lr_schedule import WarmupCosine
        sched = WarmupCosine(engine, ns.lr, ns.warmup_steps, ns.total_steps)
    if ns.clip_norm > 0:
        engine.enable_grad_stats()

    done = 0
    for done in range(1, ns.steps + 1):
        if sched is not None:
            sched.step()
        ids = next(stream).to(ranks.device)
        loss = engine(ids, labels=ids).loss
        if not all_ranks_finite(loss, ranks):
            raise RuntimeError("Nonfinite loss on at least one rank")
        loss.backward()
        engine.wait_for_completion()
        shown = mean_over_ranks(loss, ranks)
        extra = ""
        if ns.clip_norm > 0:
            stats = engine.read_grad_stats()
            if stats["nonfinite"]:
                raise RuntimeError("Nonfinite gradient on at least one rank")
            scale = engine.clip_scale_for_next_step(ns.clip_norm, stats)
            extra = f" grad_norm={stats['norm']:.6f} next_clip={scale:.4f}"
        if ranks.rank == 0:
            print(f"step={done} global_loss={shown:.6f} ranks={ranks.world}{extra}", flush=True)

    if ns.tiny:
        self_check(engine, before, done, dp)
        print(f"rank={ranks.rank} tiny_weight_checks=passed", flush=True)
    if ns.save_model:
        engine.save_pretrained(ns.save_model)   # collective: every rank calls it, rank 0 writes
    engine.wait_for_completion()
    if dp is not None:
        dp.barrier()
        dp.close()
    print(f"rank={ranks.rank} completed={done}", flush=True)
    if ranks.distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
