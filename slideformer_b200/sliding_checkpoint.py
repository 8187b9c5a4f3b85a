"""Activation checkpoint storage for the layer-sliding runtime.

Counterpart of the reference's sliding_checkpoint.py:57-280.  Each decoder layer keeps exactly
one saved tensor across forward/backward: its [B, S, H] input (everything else is recomputed
by torch's non-reentrant checkpoint).  Two placements:

  "hbm"   the tensor stays where it is.  One Llama-3.1-8B step at batch 8 x 1024 tokens keeps
          32 x 64 MiB = 2 GiB, which a 180 GB part holds without noticing; nothing crosses PCIe.
  "host"  the reference's scheme: in forward the tensor is copied to a pre-allocated pinned host
          tensor on a side stream; in backward, while layer k recomputes, layer k-1's tensor is
          prefetched into one of two device buffers; the last layer's tensor never leaves the
          GPU (sliding_checkpoint.py:110-111,171-173).  All ordering is by CUDA events.
"""
from __future__ import annotations

from collections import deque
from typing import List, Optional

import torch
from torch.autograd.graph import saved_tensors_hooks

from .numa import pinned_empty


class ActivationStore:
    """Pinned host tensors for every decoder layer plus the 2-deep device prefetch pool.
    Owned by the engine; re-created when (batch, seq, hidden) changes
    (offload_transformer.py:413-437)."""

    def __init__(self, num_layers: int, shape, dtype, device, pool_size: int = 2):
        self.device = torch.device(device)
        self.shape = tuple(shape)
        numel = torch.Size(self.shape).numel()
        self.host: List[torch.Tensor] = [pinned_empty(numel, dtype, device).view(self.shape) for _ in range(num_layers)]
        self.pool = [torch.empty(self.shape, dtype=dtype, device=self.device) for _ in range(pool_size)]
        self.pool_idx = 0
        self.stream = torch.cuda.Stream(device=self.device)
        self.saved = [torch.cuda.Event() for _ in range(num_layers)]      # forward copy of layer i landed
        self.fifo = deque()                                               # (layer, buffer, event) prefetched, in order
        self.pool_free = [torch.cuda.Event() for _ in range(pool_size)]   # compute finished reading the buffer
        self.bytes_d2h = 0
        self.bytes_h2d = 0
        # CUDA-event pairs around the copies, filled only when `timing` is set by the engine:
        # the reference's "ac fwd d2h" / "ac bwd h2d" timer labels (utils/timer.py:19-20)
        self.timing = False
        self.spans_d2h: List[tuple] = []
        self.spans_h2d: List[tuple] = []

    def _span(self, bucket, name):
        """Start an optional timing span + NVTX range on the store's stream; returns a closer."""
        if not self.timing:
            return lambda: None
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record(self.stream)
        rid = torch.cuda.nvtx.range_start(name)

        def close():
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(self.stream)
            bucket.append((t0, t1))
            if len(bucket) > 4096:
                del bucket[:2048]
            torch.cuda.nvtx.range_end(rid)
        return close

    def next_buffer(self):
        i = self.pool_idx % len(self.pool)
        self.pool_idx += 1
        return i, self.pool[i]

    def reset(self):
        self.fifo.clear()


class SlidingCheckpoint(saved_tensors_hooks):
    """Context manager around one decoder layer's `checkpoint(...)` call."""

    def __init__(self, layer_idx: int, store: Optional[ActivationStore], is_last_layer: bool = False):
        self.i = layer_idx - 1  # decoder layers are engine units 1..L
        self.store = store
        self.is_last = is_last_layer
        self.packed = 0
        self.unpacked = 0

        def pack(t: torch.Tensor):
            if store is None or self.is_last or t.numel() == 0 or tuple(t.shape) != store.shape or self.packed > 0:
                return ("keep", t)
            host = store.host[self.i]
            cur = torch.cuda.current_stream(store.device)
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(store.stream):
                store.stream.wait_event(ready)
                close = store._span(store.spans_d2h, f"AC_D2H_Layer_{layer_idx}")
                host.copy_(t, non_blocking=True)
                close()
                store.saved[self.i].record(store.stream)
            t.record_stream(store.stream)
            store.bytes_d2h += host.numel() * host.element_size()
            self.packed += 1
            return ("host", t.device)

        def prefetch(layer: int):
            """Start the host->device copy of `layer`'s tensor (called while layer+1 recomputes)."""
            if layer < 0 or store is None:
                return
            k, buf = store.next_buffer()
            done = torch.cuda.Event()
            with torch.cuda.stream(store.stream):
                store.stream.wait_event(store.pool_free[k])   # previous reader of this buffer is done
                store.stream.wait_event(store.saved[layer])
                close = store._span(store.spans_h2d, f"AC_H2D_Layer_{layer + 1}")
                buf.copy_(store.host[layer], non_blocking=True)
                close()
                done.record(store.stream)
            store.bytes_h2d += buf.numel() * buf.element_size()
            store.fifo.append((layer, k, buf, done))

        def unpack(packed):
            kind, payload = packed
            if kind == "keep":
                if self.is_last and self.unpacked == 0 and store is not None:
                    prefetch(self.i - 1)   # the last layer starts the chain
                self.unpacked += 1
                return payload
            cur = torch.cuda.current_stream(store.device)
            if not store.fifo or store.fifo[0][0] != self.i:
                # nothing prefetched for this layer (e.g. backward did not start at the last layer)
                store.fifo.clear()
                prefetch(self.i)
            layer, k, buf, done = store.fifo.popleft()
            prefetch(self.i - 1)
            cur.wait_event(done)
            out = buf.clone()             # recompute may outlive the pool slot
            store.pool_free[k].record(cur)
            self.unpacked += 1
            return out

        super().__init__(pack, unpack)
