"""Single-node data-parallel fine-tuning entry point (one rank per GPU, state sharded 1/N).

    python -m slideformer_b200.main_dp --tiny                                   # one GPU smoke check
    torchrun --nproc-per-node N -m slideformer_b200.main_dp --tiny [--tied] [--double-buffer]
    torchrun --nproc-per-node N -m slideformer_b200.main_dp --model /path/to/checkpoint --tokens ids.pt

Counterpart of the reference's multi_gpu/scripts/main_dp.py (same flags where they still mean
something; --cpu-threads is accepted and ignored because no CPU thread runs the optimizer).
With --tiny it repeats the reference's smoke checks (main_dp.py:55-61,117-124): a random
two-layer Llama, a few steps, then every unit's fp32 weights must be finite and changed and
the optimizer step count must equal the number of completed steps.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler, TensorDataset


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="local Hugging Face checkpoint directory")
    source.add_argument("--tiny", action="store_true", help="random tiny Llama with synthetic tokens, for smoke checks")
    parser.add_argument("--tokens", help="torch.save file containing a 2-D int64 input_ids tensor")
    parser.add_argument("--batch-size", type=int, default=1, help="sequences per rank")
    parser.add_argument("--seq-length", type=int, default=32, help="synthetic sequence length for --tiny")
    parser.add_argument("--steps", type=int, default=3)
    parser.add_argument("--lr", type=float, default=1e-4)
    parser.add_argument("--cpu-threads", type=int, default=1, help="accepted for compatibility; unused")
    parser.add_argument("--chunk-numel", type=int, default=32 * 1024 * 1024)
    parser.add_argument("--double-buffer", action="store_true")
    parser.add_argument("--attn-implementation", choices=("eager", "sdpa", "flash_attention_2"), default="sdpa")
    parser.add_argument("--tied", action="store_true", help="use tied embeddings with --tiny")
    parser.add_argument("--save-model", help="save final model weights; optimizer resume is not supported")
    args = parser.parse_args(argv)
    if min(args.steps, args.batch_size, args.chunk_numel) < 1 or args.seq_length < 2:
        parser.error("steps, batch-size and chunk-numel must be positive; seq-length must be >= 2")
    if args.model and not args.tokens:
        parser.error("--model requires --tokens; synthetic data is only used with --tiny")

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
        if int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
            raise ValueError("This entry point supports a single node only")
    rank = dist.get_rank() if distributed else 0

    from transformers import AutoModelForCausalLM, LlamaConfig, LlamaForCausalLM
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    from slideformer_b200.shared_data_parallel import SharedDataParallel

    torch.manual_seed(1234)
    dtype = torch.bfloat16
    if args.tiny:
        config = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2,
                             max_position_embeddings=max(128, args.seq_length), tie_word_embeddings=args.tied,
                             attention_dropout=0.0, attn_implementation=args.attn_implementation)
        base_model = LlamaForCausalLM(config).to(dtype=dtype)
    else:
        base_model = AutoModelForCausalLM.from_pretrained(args.model, dtype=dtype,
                                                          attn_implementation=args.attn_implementation)
    base_model.config.use_cache = False
    vocab = base_model.config.vocab_size
    if args.tokens:
        tokens = torch.load(args.tokens, map_location="cpu", weights_only=True)
        if not isinstance(tokens, torch.Tensor) or tokens.dtype != torch.int64 or tokens.ndim != 2 or tokens.shape[1] < 2:
            raise ValueError("--tokens must contain a 2-D int64 tensor with sequence length >= 2")
        if tokens.numel() == 0 or tokens.min() < 0 or tokens.max() >= vocab:
            raise ValueError("Token IDs must be nonempty and within the model vocabulary")
    else:
        generator = torch.Generator().manual_seed(4321)
        tokens = torch.randint(vocab, (args.steps * world * args.batch_size, args.seq_length), generator=generator)
    dataset = TensorDataset(tokens)
    sampler = DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=True, drop_last=True)
    loader = DataLoader(dataset, batch_size=args.batch_size, sampler=sampler, drop_last=True)
    if not len(loader):
        raise ValueError("Dataset must provide at least one full batch per rank")

    dp = None
    if distributed:
        dp = SharedDataParallel(chunk_numel=args.chunk_numel, dtype=dtype, exchange_slots=3 if args.double_buffer else 2)
    model = SlideFormerOffloader(
        base_model, device=device, dtype=dtype, double_buffer=args.double_buffer, enable_timing=False,
        enable_memory_stats=False, auto_backward_in_forward=False, shared_dp=dp,
        optimizer_kwargs=dict(lr=args.lr, weight_decay=0.01, fp32_optimizer_state=True),
        update_chunk=args.chunk_numel)
    model.train()
    initial = [layer._params_flat.clone() for layer in model.transformer_layers] if args.tiny else None
    torch.manual_seed(1234 + rank)
    completed, epoch = 0, 0
    while completed < args.steps:
        sampler.set_epoch(epoch)
        for (input_ids,) in loader:
            input_ids = input_ids.to(device)
            loss = model(input_ids, labels=input_ids).loss
            health = torch.isfinite(loss.detach()).to(torch.int64)
            if distributed:
                dist.all_reduce(health, op=dist.ReduceOp.MIN)
            if not health.item():
                raise RuntimeError("Nonfinite loss on at least one rank")
            loss.backward()
            model.wait_for_completion()
            mean_loss = loss.detach().float()
            if distributed:
                dist.all_reduce(mean_loss)
                mean_loss /= world
            completed += 1
            if rank == 0:
                print(f"step={completed} global_loss={mean_loss.item():.6f} ranks={world}", flush=True)
            if completed == args.steps:
                break
        epoch += 1
    if args.tiny:
        for before, layer in zip(initial, model.transformer_layers):
            owned = layer._dp_state.end - layer._dp_state.start if dp is not None else layer.total_size
            after, before = layer._params_flat[:owned], before[:owned]
            if owned and (not torch.isfinite(after).all() or torch.equal(before, after)):
                raise RuntimeError(f"Layer {layer.layer_idx} has invalid or unchanged weights")
            steps_done = layer._dp_state.step if dp is not None else model.layer_optimizer.param_groups[layer.layer_idx]["step"]
            if steps_done != completed:
                raise RuntimeError("Incorrect optimizer step count")
        print(f"rank={rank} tiny_weight_checks=passed", flush=True)
    if args.save_model and rank == 0:
        model.save_pretrained(args.save_model)
    model.wait_for_completion()
    if dp is not None:
        dp.barrier()
        dp.close()
    print(f"rank={rank} completed={completed}", flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
