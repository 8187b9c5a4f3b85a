"""Chunked host <-> device plumbing around the fused step when the gradient arrives in host
memory and the bf16 weights are wanted back in host memory.

This is the boundary the reference crosses on every layer: its gradient chunks travel
device -> host before the CPU Adam (transformer_layer.py:384-389) and the bf16 weights travel
host -> device afterwards (transformer_layer.py:296-305).  With the optimizer state resident
in HBM the directions flip: bf16 gradient in, bf16 weights out, 2 bytes per parameter each
way, and the three phases of neighbouring chunks overlap on three CUDA streams.
"""
from __future__ import annotations

from typing import Optional

import torch

from .layer_adam import LayerAdam
from .numa import numa_local, pinned_empty  # noqa: F401  (re-exported: host buffers belong on the GPU's NUMA node)


def chunk_schedule(numel: int, chunk: int, min_chunk: int):
    """Cut [0, numel) into pieces that ramp up from `min_chunk` to `chunk` by doubling, stay at
    `chunk`, and ramp down again.  The first upload and the last download are the only copies
    that nothing overlaps, so short pieces at both ends shrink the pipeline's fill and drain time.
    Every boundary is a multiple of 16 elements (each piece keeps the vector body / scalar tail
    split of one reference call), except the end of the last piece."""
    if chunk % 16 or min_chunk % 16 or min_chunk <= 0 or chunk < min_chunk:
        raise ValueError("chunk sizes must be positive multiples of 16 with min_chunk <= chunk")
    up, c = [], min_chunk
    while c < chunk:
        up.append(c)
        c *= 2
    pieces, pos = [], 0
    ramp = sum(up)
    if numel <= 2 * ramp + chunk:          # too small to ramp: plain equal chunks
        while pos < numel:
            pieces.append((pos, min(pos + chunk, numel)))
            pos += chunk
        return pieces
    for c in up:
        pieces.append((pos, pos + c))
        pos += c
    while numel - pos > ramp + chunk:
        pieces.append((pos, pos + chunk))
        pos += chunk
    tail = numel - pos - ramp               # in (0, chunk]
    pieces.append((pos, pos + tail - (tail % 16 if numel - (pos + tail) > 0 else 0)))
    pos = pieces[-1][1]
    for c in reversed(up):
        end = min(pos + c, numel)
        if end > pos:
            pieces.append((pos, end))
        pos = end
    if pos < numel:
        pieces.append((pos, numel))
    return pieces


class HostGradStepper:
    """Runs `LayerAdam.step_chunk` over a flat HBM-resident layer whose gradient is in pinned
    host memory, optionally returning the bf16 copy of the updated weights to pinned host
    memory.  Chunk k+1's upload, chunk k's kernel and chunk k-1's download run concurrently."""

    def __init__(self, opt: LayerAdam, numel: int, device, chunk_numel: int = 32 * 1024 * 1024,
                 grad_dtype=torch.bfloat16, min_chunk_numel: int = None):
        if chunk_numel % 16:
            raise ValueError("chunk_numel must be a multiple of 16 so every chunk but the last stays on the vector body")
        self.opt = opt
        self.numel = int(numel)
        self.device = torch.device(device)
        self.chunk = int(chunk_numel)
        self.chunks = chunk_schedule(self.numel, self.chunk, int(min_chunk_numel or chunk_numel))
        with torch.cuda.device(self.device):
            self.s_in = torch.cuda.Stream()
            self.s_k = torch.cuda.Stream()
            self.s_out = torch.cuda.Stream()
            self.g_dev = [torch.empty(min(self.chunk, max(self.numel, 1)), dtype=grad_dtype, device=self.device)
                          for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_k = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in self.chunks]   # download of piece k finished

    @torch.no_grad()
    def step(self, p: torch.Tensor, g_host: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
             bf16_dev: Optional[torch.Tensor], bf16_host: Optional[torch.Tensor], param_group: dict,
             join: bool = True):
        """One optimizer step.  p, m, v, bf16_dev: flat CUDA tensors; g_host, bf16_host: flat pinned
        host tensors.  Returns after enqueueing.  join=True makes the caller's current stream wait
        for the end of the step.  With join=False the next step's uploads may start while this
        step's downloads drain (every hazard between the two steps is covered by an event); call
        `join()` before reading `bf16_host` or touching p, m, v from another stream."""
        n = self.numel
        if not g_host.is_pinned() or (bf16_host is not None and not bf16_host.is_pinned()):
            raise RuntimeError("host buffers must be pinned")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_k, self.s_out):
            s.wait_stream(cur)
        for k, (a, b) in enumerate(self.chunks):
            slot = k & 1
            with torch.cuda.stream(self.s_in):
                # the kernel that last read this staging slot (piece k-2, or a piece of the previous
                # step) has finished; waiting on a never-recorded event is a no-op
                self.s_in.wait_event(self.ev_k[slot])
                self.g_dev[slot][: b - a].copy_(g_host[a:b], non_blocking=True)
                self.ev_in[slot].record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(self.ev_in[slot])
                self.s_k.wait_event(self.ev_out[k])   # the previous step's download of this piece is done
                self.opt.step_chunk(p[a:b], self.g_dev[slot][: b - a], m[a:b], v[a:b], param_group,
                                    bf16_dev[a:b] if bf16_dev is not None else None)
                self.ev_k[slot].record(self.s_k)
            if bf16_host is not None and bf16_dev is not None:
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_k[slot])
                    bf16_host[a:b].copy_(bf16_dev[a:b], non_blocking=True)
                    self.ev_out[k].record(self.s_out)
        if join:
            self.join()

    def join(self):
        """Make the current stream wait for everything this stepper has enqueued."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_k)
        cur.wait_stream(self.s_out)
