"""Single-node data parallelism with the optimizer state sharded 1/N across the GPUs.

Mirror of the reference's `SharedDataParallel` (multi_gpu/shared_data_parallel.py:21-148):
same constructor keywords, `register_layer`, `reduce_chunk(layer, start, end, local_grad,
update)`, `barrier`, `raise_if_failed`, `close`, and the attributes `rank`, `world_size`,
`chunk_numel`, `dtype`, `layers`, `error`, `directory`.

What changes.  The reference funnels every rank's gradient chunk through a /dev/shm slab,
lets rank 0 average them in fp32 and run the CPU Adam, and shares one fp32 weight mapping.
Here every rank owns a contiguous 1/N slice of each layer's fp32 weights and Adam moments in
its own HBM.  Gradients stay on the GPUs in an exchange buffer that every rank maps from
every other rank (CUDA IPC over NVLink); the owner of a slice reads the N per-rank gradients
with plain loads, adds them to a zero fp32 accumulator in rank order and divides by N, which
is the reference's arithmetic (shared_data_parallel.py:130-133) bit for bit, either into an
fp32 buffer handed to the caller's `update` callback or directly inside the fused Adam
kernel (`fused_update`).  The bf16 weights of all slices are then all-gathered with NCCL.

Ordering between ranks uses stream-ordered NCCL operations only (a one-element all-reduce as
a barrier, the all-gather itself); no kernel of this package ever waits on another GPU.
A gloo group carries the host-side control plane: consistency checks and error flags.

Exactness: results equal the reference's rank-0 update bit for bit when chunk starts are
multiples of 16 elements (slice boundaries always are), because a chunk cut at a slice
boundary then keeps the reference's 16-lane body / scalar tail split.
"""
from __future__ import annotations

import ctypes as C
import socket
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from . import _lib

SHARD_ALIGN = 16  # elements; keeps every slice on the vector body and 32-byte aligned in fp32


def shard_numel(numel: int, world: int, align: int = SHARD_ALIGN) -> int:
    """Elements per rank: ceil(numel / world) rounded up to `align` (0 for an empty layer)."""
    if numel <= 0:
        return 0
    per = -(-numel // world)
    return -(-per // align) * align


def shard_range(numel: int, world: int, rank: int, align: int = SHARD_ALIGN):
    """Global [start, end) of the slice `rank` owns, clipped to the layer (may be empty)."""
    s = shard_numel(numel, world, align)
    a = min(rank * s, numel)
    b = min((rank + 1) * s, numel)
    return a, b


def slice_vec_n(call_start: int, call_end: int, a: int, b: int) -> int:
    """Where the reference call over [call_start, call_end) switches from its 16-lane body to its
    scalar tail (cpu_adam_impl.cpp:23-68), expressed relative to the slice [a, b) of that call:
    the `vec_n` to pass to the kernel so that a call executed in pieces keeps the reference's bits."""
    vec_ref = call_start + ((call_end - call_start) & ~15)
    return min(max(vec_ref - a, 0), b - a)


@dataclass
class LayerState:
    """Per-layer state.  `params`, `exp_avg`, `exp_avg_sq` keep the reference's names but hold
    THIS RANK's slice (every rank has one; the reference gives the moments to rank 0 only)."""
    params: torch.Tensor
    exp_avg: Optional[torch.Tensor]
    exp_avg_sq: Optional[torch.Tensor]
    step: int = 0
    numel: int = 0
    shard: int = 0           # slice length including padding (same on every rank)
    start: int = 0           # global range of the slice, clipped to numel
    end: int = 0
    bf16: Optional[torch.Tensor] = None  # full layer, bf16, padded to shard * world: all-gather target
    peer_bf16: Optional[list] = None     # base pointer of every rank's `bf16` (push mode only)
    mc_bf16: int = 0                     # multicast address aliasing every rank's `bf16` (NVLS mode only)
    bf16_shard: Optional[torch.Tensor] = None  # window mode: only this rank's bf16 slice is kept; the full
                                               # layer is all-gathered into a window unit when it is needed


class _RawCuda:
    """Wraps a raw device pointer for torch.as_tensor (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class ControlPlane:
    """Host-side agreement between ranks over gloo: identical-spec checks and error flags.
    Works on CPU-only hosts (it is what the world_size-2 CPU tests exercise)."""

    def __init__(self, timeout_seconds: float = 120):
        if not dist.is_initialized():
            raise RuntimeError("Initialize torch.distributed before SharedDataParallel")
        self.rank = dist.get_rank()
        self.world_size = dist.get_world_size()
        self.group = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_seconds))

    def all_same(self, spec) -> bool:
        specs = [None] * self.world_size
        dist.all_gather_object(specs, spec, group=self.group)
        return len(set(specs)) == 1

    def gather(self, obj) -> list:
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def any_failed(self, failed: bool) -> bool:
        t = torch.tensor([1 if failed else 0], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return bool(t.item())

    def barrier(self):
        dist.barrier(group=self.group)

    def close(self):
        dist.destroy_process_group(self.group)


class SharedDataParallel:
    """Collectively construct on all local ranks (after `init_process_group("nccl")` and
    `torch.cuda.set_device`).  Call `reduce_chunk` / `fused_update` in identical layer and
    chunk order on every rank."""

    def __init__(self, chunk_numel=32 * 1024 * 1024, dtype=torch.bfloat16, shm_dir=None, timeout_seconds=120,
                 *, device=None, exchange_slots: int = 2, push_weights: bool = True, nvls: bool = False):
        if not dist.is_initialized():
            raise RuntimeError("Initialize torch.distributed before SharedDataParallel")
        if chunk_numel < 1:
            raise ValueError("chunk_numel must be positive")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("gradient dtype must be bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("SharedDataParallel needs CUDA devices; there is no CPU data path")
        self.ctl = ControlPlane(timeout_seconds)
        self.rank, self.world_size = self.ctl.rank, self.ctl.world_size
        if self.world_size > 16:
            raise ValueError("at most 16 ranks")
        self.chunk_numel = int(chunk_numel)
        self.dtype = dtype
        self.layers: Dict[int, LayerState] = {}
        self.error = None
        self._closed = False
        self.directory = None  # the reference's /dev/shm directory has no counterpart
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._lib = _lib.load()
        self._gcode = _lib.SF_GRAD_BF16 if dtype == torch.bfloat16 else _lib.SF_GRAD_F32
        self._esize = 2 if dtype == torch.bfloat16 else 4
        if nvls and (dtype != torch.bfloat16 or not push_weights):
            raise ValueError("nvls needs bfloat16 gradients and push_weights")
        if not self.ctl.all_same((socket.gethostname(), self.chunk_numel, str(dtype), exchange_slots, bool(push_weights),
                                  bool(nvls))):
            raise ValueError("SharedDataParallel requires one host and matching chunk size/dtype")
        self.exchange_slots = int(exchange_slots)
        # True: the update kernel stores the bf16 weights into every rank's layer buffer itself
        # (peer-mapped stores); False: NCCL all-gather after the kernel.
        self.push_weights = bool(push_weights)
        # True: exchange and bf16 layer buffers are symmetric-memory allocations with an NVSwitch
        # multicast address, and fused_update reduces gradients / replicates weights inside the
        # switch (multimem).  Faster, not bit-exact (see sf_adam_step_sharded_nvls).  Keep it off in
        # any run where a rank may leave early: its memory stays bound to the multicast object.
        self.nvls = bool(nvls)
        self._symm_keep = []                # symmetric-memory tensors and handles kept alive
        self._mc_base = 0                   # multicast address of the exchange allocation
        self._weight_allocs = []            # (base, peers) of the IPC-visible bf16 layer buffers
        self._views_out = False             # grad_buffer() views exist: the slots must not move any more
        self._cap = 0                       # elements per exchange slot
        self._base = None                   # local exchange allocation (raw pointer)
        self._peer_base: List[int] = []     # every rank's exchange base mapped here (own = local pointer)
        self._exchange: List[torch.Tensor] = []
        self._mean: Optional[torch.Tensor] = None
        self._token = torch.zeros(1, device=self.device)
        self.group = self.ctl.group

    # ---- memory every rank can address (CUDA IPC) --------------------------------------------------
    def _shared_alloc(self, nbytes: int):
        """Collective: allocate `nbytes` on every rank, exchange IPC handles, map the peers'.
        Returns (local base pointer, [base pointer of rank r as seen from this process])."""
        with torch.cuda.device(self.device):
            ptr = C.c_void_p()
            _lib.check(self._lib.sf_dev_alloc(nbytes, C.byref(ptr)))
            base = ptr.value
            handle = (C.c_ubyte * _lib.SF_IPC_HANDLE_BYTES)()
            _lib.check(self._lib.sf_ipc_export(base, handle))
            handles = self.ctl.gather(bytes(handle))
            peers = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    peers.append(base)
                    continue
                buf = (C.c_ubyte * _lib.SF_IPC_HANDLE_BYTES).from_buffer_copy(h)
                out = C.c_void_p()
                _lib.check(self._lib.sf_ipc_open(buf, C.byref(out)))
                peers.append(out.value)
        return base, peers

    def _symm_alloc(self, nbytes: int):
        """Collective: a symmetric-memory allocation of `nbytes` on every rank.  Returns (local
        base pointer, [every rank's base as seen from here], multicast address)."""
        import torch.distributed._symmetric_memory as symm_mem
        with torch.cuda.device(self.device):
            t = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(t, dist.group.WORLD)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        ok = self.ctl.gather(mc != 0)
        if not all(ok):
            raise RuntimeError("NVLS multicast is not available on every rank (driver / fabric without multicast support)")
        self._symm_keep.append((t, hdl))
        return t.data_ptr(), [int(x) for x in hdl.buffer_ptrs], mc

    def _shared_free(self, base, peers):
        if self.nvls:
            return   # symmetric-memory tensors are released when close() drops them
        for r, ptr in enumerate(peers):
            if r != self.rank and ptr:
                self._lib.sf_ipc_close(ptr)
        if base:
            with torch.cuda.device(self.device):
                _lib.check(self._lib.sf_dev_free(base))

    # ---- exchange buffers ------------------------------------------------------------------
    def _free_exchange(self):
        self._exchange = []
        self._shared_free(self._base, self._peer_base)
        self._peer_base = []
        self._base = None

    def ensure_exchange_slots(self, slots: int):
        """Collective: have at least `slots` exchange slots.  Only before any slot exists."""
        if slots <= self.exchange_slots:
            return
        if self._cap or self._views_out:
            raise RuntimeError("the number of exchange slots can only grow before the first layer is registered")
        self.exchange_slots = int(slots)

    def reserve_exchange(self, elems: int):
        """Collective: make every exchange slot at least `elems` elements long.  Call it with the
        largest layer size before handing out `grad_buffer()` views: growing the slots later
        re-allocates them, which would leave such views dangling (and is refused)."""
        self._grow_exchange(-(-int(elems) // (SHARD_ALIGN * self.world_size)) * SHARD_ALIGN * self.world_size)

    def _grow_exchange(self, elems: int):
        """Collective: (re)allocate the exchange slots for `elems` elements and map the peers'."""
        if elems <= self._cap:
            return
        if self._views_out:
            raise RuntimeError("a layer larger than the exchange slots was registered after grad_buffer() views "
                               "were handed out; call reserve_exchange(largest_layer_numel) first")
        torch.cuda.synchronize(self.device)
        self.ctl.barrier()
        self._free_exchange()
        elems = -(-elems // 128) * 128
        nbytes = elems * self._esize * self.exchange_slots
        if self.nvls:
            self._base, self._peer_base, self._mc_base = self._symm_alloc(nbytes)
        else:
            self._base, self._peer_base = self._shared_alloc(nbytes)
        with torch.cuda.device(self.device):
            flat = torch.as_tensor(_RawCuda(self._base, nbytes), device=self.device)
            flat.zero_()
            self._exchange = [flat[k * elems * self._esize:(k + 1) * elems * self._esize].view(self.dtype)
                              for k in range(self.exchange_slots)]
        self._cap = elems
        torch.cuda.synchronize(self.device)
        self.ctl.barrier()

    def grad_buffer(self, slot: int = 0) -> torch.Tensor:
        """This rank's exchange slot (dtype = self.dtype, capacity >= the largest registered layer).
        Writing gradients straight into it saves the copy `reduce_chunk` would make."""
        self._views_out = True
        return self._exchange[slot]

    def _peer_ptrs(self, slot: int, offset_elems: int):
        arr = (C.c_void_p * self.world_size)()
        for r in range(self.world_size):
            arr[r] = self._peer_base[r] + (slot * self._cap + offset_elems) * self._esize
        return arr

    def _push_ptrs(self, state, offset_elems: int):
        """Every rank's bf16 layer buffer at `offset_elems`, starting with the next rank: the order
        of the destinations does not change the result, and each rank starting at a different
        peer keeps the ranks from storing to the same destination in the same order."""
        w = self.world_size
        return (C.c_void_p * w)(*[state.peer_bf16[(self.rank + 1 + j) % w] + 2 * offset_elems for j in range(w)])

    # ---- registration ----------------------------------------------------------------------
    def register_layer(self, layer_idx, numel, resident_bf16: bool = True) -> LayerState:
        if not self.ctl.all_same((layer_idx, int(numel))) or layer_idx in self.layers:
            raise ValueError("Ranks must register identical layers exactly once")
        numel = int(numel)
        s = shard_numel(numel, self.world_size)
        a, b = shard_range(numel, self.world_size, self.rank)
        dev = self.device
        peer_bf16 = None
        bf16_shard = None
        mc_bf16 = 0
        if not resident_bf16:
            bf16 = None
            bf16_shard = torch.zeros(s, dtype=torch.bfloat16, device=dev)
        elif self.push_weights and s > 0:
            nbytes = s * self.world_size * 2
            if self.nvls:
                base, peer_bf16, mc_bf16 = self._symm_alloc(nbytes)
            else:
                base, peer_bf16 = self._shared_alloc(nbytes)
            self._weight_allocs.append((base, peer_bf16))
            with torch.cuda.device(dev):
                bf16 = torch.as_tensor(_RawCuda(base, nbytes), device=dev).view(torch.bfloat16)
                bf16.zero_()
        else:
            bf16 = torch.zeros(s * self.world_size, dtype=torch.bfloat16, device=dev)
        state = LayerState(
            params=torch.zeros(s, dtype=torch.float32, device=dev),
            exp_avg=torch.zeros(s, dtype=torch.float32, device=dev),
            exp_avg_sq=torch.zeros(s, dtype=torch.float32, device=dev),
            numel=numel, shard=s, start=a, end=b, bf16=bf16, peer_bf16=peer_bf16, bf16_shard=bf16_shard,
            mc_bf16=mc_bf16)
        self._grow_exchange(s * self.world_size)
        self.layers[layer_idx] = state
        return state

    def load_full_params(self, layer_idx, full_fp32: torch.Tensor):
        """Initialise this rank's slice (and the bf16 copy) from a full flat fp32 layer."""
        st = self.layers[layer_idx]
        st.params[: st.end - st.start].copy_(full_fp32[st.start:st.end])
        if st.bf16 is not None:
            st.bf16[: st.numel].copy_(full_fp32[: st.numel])
        else:
            st.bf16_shard[: st.end - st.start].copy_(full_fp32[st.start:st.end])

    @torch.no_grad()
    def gather_weights(self, layer_idx, dst: torch.Tensor):
        """Window mode: all-gather the bf16 slices of a layer into `dst` (>= shard * world elements)
        on the current stream."""
        st = self.layers[layer_idx]
        if st.shard == 0:
            return None
        return dist.all_gather_into_tensor(dst[: st.shard * self.world_size], st.bf16_shard)

    # ---- synchronisation ---------------------------------------------------------------------
    def barrier(self):
        """Host barrier over the control plane, like the reference's gloo barrier."""
        self.ctl.barrier()

    def stream_barrier(self):
        """Orders the current CUDA stream after every rank's stream has reached this point."""
        dist.all_reduce(self._token)

    def raise_if_failed(self):
        if self.error is not None:
            raise RuntimeError("A distributed update failed") from self.error

    def _validate(self, state, start, end, local_grad):
        count = end - start
        if not 0 <= start < end <= state.numel or count > self.chunk_numel:
            raise ValueError("Invalid gradient chunk")
        if local_grad is not None and (local_grad.device.type != "cuda" or local_grad.numel() != count
                                       or local_grad.dtype != self.dtype):
            raise ValueError("Gradient chunk must match the configured CUDA dtype and size")
        return count

    def _stage(self, slot, start, end, local_grad):
        if local_grad is None:
            return
        dst = self._exchange[slot][start:end]
        if local_grad.data_ptr() != dst.data_ptr():
            dst.copy_(local_grad.view(-1))

    # ---- the reference-shaped call -------------------------------------------------------------
    @torch.no_grad()
    def reduce_chunk(self, layer_idx, start, end, local_grad, update: Callable, slot: int = 0,
                     check_errors: bool = True):
        """Average a chunk over all ranks in fp32 (rank order) and hand each slice owner its part:
        `update(params, mean_grad, exp_avg, exp_avg_sq)` receives fp32 device views of the
        intersection of [start, end) with this rank's slice.  EVERY rank is called once per chunk,
        with empty views when it owns nothing of the chunk: an optimizer whose scalars depend on
        the call history (the reference's beta^t state machine does) then sees the same history
        on every rank as the reference's rank 0.  On return the exchange slot region may be
        overwritten (stream-ordered)."""
        self.raise_if_failed()
        state = self.layers[layer_idx]
        failure = None
        try:
            self._validate(state, start, end, local_grad)
            self._stage(slot, start, end, local_grad)
        except Exception as exc:   # reported to every rank below, after the barrier this rank still owes
            failure = exc
        invalid = failure
        self.stream_barrier()
        a, b = max(start, state.start), min(end, state.end)
        try:
            if failure is not None:
                raise failure
            k = max(b - a, 0)
            if self._mean is None or self._mean.numel() < k:
                self._mean = torch.empty(max(k, min(self.chunk_numel, state.shard)), dtype=torch.float32,
                                         device=self.device)
            mean = self._mean[:k]
            if k > 0:
                with torch.cuda.device(self.device):
                    _lib.check(self._lib.sf_dp_mean(self._peer_ptrs(slot, a), self.world_size, self._gcode,
                                                    mean.data_ptr(), k, torch.cuda.current_stream().cuda_stream))
            lo = max(a - state.start, 0) if k > 0 else 0
            update(state.params[lo:lo + k], mean, state.exp_avg[lo:lo + k], state.exp_avg_sq[lo:lo + k])
        except Exception as exc:  # propagate to every rank below
            failure = exc
        if check_errors and self.ctl.any_failed(failure is not None):
            self.stream_barrier()
            if invalid is not None:
                raise invalid      # this rank's own bad arguments keep their type (ValueError), as in the reference
            self.error = failure if failure is not None else RuntimeError("a peer rank failed")
            self.raise_if_failed()
        elif failure is not None:
            self.stream_barrier()
            if invalid is not None:
                raise invalid
            self.error = failure
            self.raise_if_failed()
        self.stream_barrier()

    # ---- the fused call --------------------------------------------------------------------------
    @torch.no_grad()
    def fused_update(self, layer_idx, adam, param_group: dict, start: int = 0, end: Optional[int] = None,
                     local_grad: Optional[torch.Tensor] = None, slot: int = 0, gather: bool = True,
                     barrier: bool = True, check_errors: bool = False):
        """Mean + Adam + bf16 cast in one kernel on this rank's part of [start, end), then (by
        default) the all-gather of the layer's bf16 weights.  `adam` is a LayerAdam (its scalar
        state machine advances once per call, like one reference adam_update).  barrier=False
        skips the leading cross-rank stream barrier: correct for the second and later chunks of
        a layer whose whole gradient was complete on every rank before the first chunk's barrier.

        A host-side failure on this rank between the two barriers (a rejected argument, a CUDA
        error at launch) still enqueues the trailing barrier before it is raised, so the peers'
        streams are not left waiting for this rank inside the current unit.  check_errors=True
        additionally exchanges a failure flag over the host control plane (one gloo all-reduce
        per call, which synchronises the hosts) and raises on EVERY rank, like `reduce_chunk`."""
        self.raise_if_failed()
        state = self.layers[layer_idx]
        end = state.numel if end is None else end
        if state.numel == 0:
            return
        failure = None
        try:
            if not 0 <= start < end <= state.numel:
                raise ValueError("Invalid gradient chunk")
            if local_grad is not None:
                self._validate(state, start, end, local_grad)
                self._stage(slot, start, end, local_grad)
        except Exception as exc:
            failure = exc
        invalid = failure
        if barrier:
            self.stream_barrier()
        if failure is None:
            try:
                self._launch_fused(state, adam, param_group, start, end, slot)
            except Exception as exc:
                failure = exc
        if (check_errors and self.ctl.any_failed(failure is not None)) or failure is not None:
            self.all_gather_params(layer_idx)      # keep the barrier count of this unit balanced
            if invalid is not None:
                raise invalid      # this rank's own bad arguments keep their type (ValueError)
            self.error = failure if failure is not None else RuntimeError("a peer rank failed")
            self.raise_if_failed()
        if gather:
            self.all_gather_params(layer_idx)

    @torch.no_grad()
    def fused_update_multi(self, items, adam):
        """`fused_update` for many (layer, chunk) pieces with ONE barrier before, one or a few kernel
        launches (up to 32 pieces each) and ONE barrier after, instead of a launch and two barriers
        per piece: what a model made of small units needs.  items: sequence of
        (layer_idx, param_group, start, end, slot) in the order the reference would update them;
        every piece is still one reference adam_update (the scalar state machine advances once per
        piece on every rank), so the bits equal those of separate `fused_update` calls.  The
        whole gradient of every listed layer must be complete in its exchange slot on every rank
        before this call is enqueued.  Push mode only (resident bf16 layers, at most 8 ranks)."""
        self.raise_if_failed()
        if self.world_size > 8:
            raise ValueError("fused_update_multi supports at most 8 ranks")
        segs, keep = [], []
        for layer_idx, param_group, start, end, slot in items:
            state = self.layers[layer_idx]
            if state.numel == 0:
                continue
            if state.peer_bf16 is None or state.mc_bf16:
                raise ValueError("fused_update_multi needs push-mode layers (resident, peer-mapped bf16 weights)")
            end = state.numel if end is None else end
            if not 0 <= start < end <= state.numel:
                raise ValueError("Invalid gradient chunk")
            sg = _lib.SfPushSegment()
            _lib.check(self._lib.sf_adam_scalars(adam.optimizer_id, int(param_group["step"]), param_group["lr"],
                                                 param_group["betas"][0], param_group["betas"][1], param_group["eps"],
                                                 param_group["weight_decay"], int(param_group["bias_correction"] == 1),
                                                 C.byref(sg.s)))
            a, b = max(start, state.start), min(end, state.end)
            if b <= a:
                continue                        # nothing of this piece is ours; the state machine still advanced
            k, lo = b - a, a - state.start
            pg, po = self._peer_ptrs(slot, a), self._push_ptrs(state, a)
            keep += [pg, po]
            sg.p = state.params[lo:lo + k].data_ptr()
            sg.m = state.exp_avg[lo:lo + k].data_ptr()
            sg.v = state.exp_avg_sq[lo:lo + k].data_ptr()
            sg.peer_g, sg.peer_out = pg, po
            sg.n, sg.vec_n = k, slice_vec_n(start, end, a, b)
            segs.append(sg)
        self.stream_barrier()
        failure = None
        try:
            with torch.cuda.device(self.device):
                stream = torch.cuda.current_stream().cuda_stream
                for i in range(0, len(segs), _lib.SF_MAX_SEGMENTS):
                    part = segs[i:i + _lib.SF_MAX_SEGMENTS]
                    arr = (_lib.SfPushSegment * len(part))(*part)
                    _lib.check(self._lib.sf_adam_step_sharded_push_multi(arr, len(part), self.world_size, self._gcode, stream))
        except Exception as exc:
            failure = exc
        self.stream_barrier()                   # all pushes landed everywhere; gradients may be overwritten
        if failure is not None:
            self.error = failure
            self.raise_if_failed()

    def _launch_fused(self, state, adam, param_group, start, end, slot):
        sc = _lib.SfAdamScalars()
        _lib.check(self._lib.sf_adam_scalars(adam.optimizer_id, int(param_group["step"]), param_group["lr"],
                                             param_group["betas"][0], param_group["betas"][1], param_group["eps"],
                                             param_group["weight_decay"], int(param_group["bias_correction"] == 1),
                                             C.byref(sc)))
        a, b = max(start, state.start), min(end, state.end)
        if b > a:
            k, lo = b - a, a - state.start
            vec_local = slice_vec_n(start, end, a, b)
            with torch.cuda.device(self.device):
                stream = torch.cuda.current_stream().cuda_stream
                if state.bf16 is None:
                    _lib.check(self._lib.sf_adam_step_sharded(
                        C.byref(sc), state.params[lo:lo + k].data_ptr(), self._peer_ptrs(slot, a), self.world_size,
                        self._gcode, state.exp_avg[lo:lo + k].data_ptr(), state.exp_avg_sq[lo:lo + k].data_ptr(),
                        state.bf16_shard[lo:lo + k].data_ptr(), k, vec_local, stream))
                elif state.mc_bf16:
                    outs = self._push_ptrs(state, a)
                    _lib.check(self._lib.sf_adam_step_sharded_nvls(
                        C.byref(sc), state.params[lo:lo + k].data_ptr(),
                        self._mc_base + (slot * self._cap + a) * self._esize, state.mc_bf16 + 2 * a,
                        self._peer_ptrs(slot, a), outs, self.world_size, state.exp_avg[lo:lo + k].data_ptr(),
                        state.exp_avg_sq[lo:lo + k].data_ptr(), k, vec_local, stream))
                elif state.peer_bf16 is not None:
                    outs = self._push_ptrs(state, a)
                    _lib.check(self._lib.sf_adam_step_sharded_push(
                        C.byref(sc), state.params[lo:lo + k].data_ptr(), self._peer_ptrs(slot, a), outs,
                        self.world_size, self._gcode, state.exp_avg[lo:lo + k].data_ptr(),
                        state.exp_avg_sq[lo:lo + k].data_ptr(), k, vec_local, stream))
                else:
                    _lib.check(self._lib.sf_adam_step_sharded(
                        C.byref(sc), state.params[lo:lo + k].data_ptr(), self._peer_ptrs(slot, a), self.world_size,
                        self._gcode, state.exp_avg[lo:lo + k].data_ptr(), state.exp_avg_sq[lo:lo + k].data_ptr(),
                        state.bf16[a:b].data_ptr(), k, vec_local, stream))

    @torch.no_grad()
    def all_gather_params(self, layer_idx, async_op: bool = False, force_nccl: bool = False):
        """All-gather the bf16 slices into every rank's full-layer buffer (in place).  Its
        completion on a rank also means every rank has finished reading that rank's gradients."""
        state = self.layers[layer_idx]
        if state.shard == 0:
            return None
        if state.bf16 is None:
            # window mode: nothing to publish now, but the gradients of this layer may only be
            # overwritten once every rank has finished reading them
            self.stream_barrier()
            return None
        if state.peer_bf16 is not None and not force_nccl:
            # the update kernels already stored every slice everywhere; once every rank's stream
            # has passed this point all of those stores have completed
            self.stream_barrier()
            return None
        mine = state.bf16[self.rank * state.shard:(self.rank + 1) * state.shard]
        return dist.all_gather_into_tensor(state.bf16, mine, async_op=async_op)

    # ---- NCCL-only variant (bf16 reduction, not bit-identical to the fp32 rank-order mean) --------
    @torch.no_grad()
    def nccl_update(self, layer_idx, adam, param_group: dict, slot: int = 0, gather: bool = True):
        state = self.layers[layer_idx]
        if state.numel == 0:
            return
        full = self._exchange[slot][: state.shard * self.world_size]
        mine = full[self.rank * state.shard:(self.rank + 1) * state.shard]
        dist.reduce_scatter_tensor(mine, full, op=dist.ReduceOp.AVG)
        k = state.end - state.start
        if k > 0:
            adam.step_chunk(state.params[:k], mine[:k], state.exp_avg[:k], state.exp_avg_sq[:k], param_group,
                            state.bf16[state.start:state.end])
        if gather:
            self.all_gather_params(layer_idx, force_nccl=True)

    def close(self):
        """Release local resources after all ranks have drained their work."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        self.ctl.barrier()
        self.layers.clear()
        self._free_exchange()
        for base, peers in self._weight_allocs:
            self._shared_free(base, peers)
        self._weight_allocs = []
        self._cap = 0
        if self._symm_keep:
            self._exchange = []
            self._symm_keep = []
            self.ctl.barrier()
        self.ctl.close()


class ShardedLayerAdam:
    """One flat layer sharded over all ranks; the multi-GPU benchmark and the sweep drive this.

    step(k): every rank's gradient buffer k -> fp32 rank-order mean + Adam on the owned slice
    (mode "fused": one kernel reading the peers' buffers; mode "nccl": NCCL bf16 reduce-scatter,
    then the single-GPU kernel) -> all-gather of the bf16 weights."""

    def __init__(self, numel: int, device, mode: str = "fused", grad_slots: int = 3, **hp):
        from .layer_adam import LayerAdam
        if mode not in ("fused", "fused_ag", "nccl", "nvls"):
            raise ValueError("mode must be 'fused', 'fused_ag', 'nccl' or 'nvls'")
        self.mode = mode
        self.dp = SharedDataParallel(chunk_numel=max(int(numel), 1), dtype=torch.bfloat16, device=device,
                                     exchange_slots=grad_slots, push_weights=(mode in ("fused", "nvls")),
                                     nvls=(mode == "nvls"))
        self.adam = LayerAdam(**hp)
        self.state = self.dp.register_layer(0, numel)
        self.numel = int(numel)
        self.shard_numel = self.state.end - self.state.start
        self.params_shard = self.state.params
        self.group = dict(self.adam.defaults, step=0)

    def grad_buffer(self, k: int) -> torch.Tensor:
        return self.dp.grad_buffer(k)[: self.numel]

    def describe(self) -> str:
        if self.mode == "fused":
            return ("one kernel: peer-read fp32 rank-order gradient mean + Adam + bf16 weights pushed to every rank "
                    "over NVLink, stream barriers before and after")
        if self.mode == "nvls":
            return ("one kernel: gradient sum reduced inside the NVSwitch (multimem.ld_reduce, bf16 result) + Adam + bf16 "
                    "weights replicated by the switch (multimem.st), stream barriers before and after; not bit-exact")
        if self.mode == "fused_ag":
            return "fused peer-read fp32 rank-order mean + Adam kernel over NVLink, NCCL bf16 all-gather"
        return "NCCL bf16 reduce-scatter (avg), Adam kernel, NCCL bf16 all-gather"

    def step(self, k: int = 0):
        self.group["step"] += 1
        if self.mode in ("fused", "fused_ag", "nvls"):
            self.dp.fused_update(0, self.adam, self.group, slot=k)
        else:
            self.dp.nccl_update(0, self.adam, self.group, slot=k)

    # ---- measurement helpers (device-timed with CUDA events on the launching stream) -------------
    def _timed(self, fn, reps: int) -> float:
        fn()
        torch.cuda.synchronize(self.dp.device)
        self.dp.ctl.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize(self.dp.device)
        t = torch.tensor([a.elapsed_time(b) / reps], device=self.dp.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_kernel_only(self, reps: int) -> float:
        """Average duration (ms, max over ranks) of the Adam kernel alone on the owned slice: in
        fused mode it includes the peer gradient reads over NVLink, but no barrier or all-gather."""
        st, dp = self.state, self.dp
        k = st.end - st.start

        def fused():
            self.group["step"] += 1
            sc = _lib.SfAdamScalars()
            g = self.group
            _lib.check(dp._lib.sf_adam_scalars(self.adam.optimizer_id, g["step"], g["lr"], g["betas"][0], g["betas"][1],
                                               g["eps"], g["weight_decay"], int(g["bias_correction"] == 1), C.byref(sc)))
            if k > 0 and st.mc_bf16:
                outs = dp._push_ptrs(st, st.start)
                _lib.check(dp._lib.sf_adam_step_sharded_nvls(
                    C.byref(sc), st.params.data_ptr(), dp._mc_base + st.start * 2, st.mc_bf16 + 2 * st.start,
                    dp._peer_ptrs(0, st.start), outs, dp.world_size, st.exp_avg.data_ptr(), st.exp_avg_sq.data_ptr(),
                    k, k, torch.cuda.current_stream().cuda_stream))
            elif k > 0 and st.peer_bf16 is not None:
                outs = dp._push_ptrs(st, st.start)
                _lib.check(dp._lib.sf_adam_step_sharded_push(
                    C.byref(sc), st.params.data_ptr(), dp._peer_ptrs(0, st.start), outs, dp.world_size, dp._gcode,
                    st.exp_avg.data_ptr(), st.exp_avg_sq.data_ptr(), k, k, torch.cuda.current_stream().cuda_stream))
            elif k > 0:
                _lib.check(dp._lib.sf_adam_step_sharded(
                    C.byref(sc), st.params.data_ptr(), dp._peer_ptrs(0, st.start), dp.world_size, dp._gcode,
                    st.exp_avg.data_ptr(), st.exp_avg_sq.data_ptr(), st.bf16[st.start:st.end].data_ptr(), k, k,
                    torch.cuda.current_stream().cuda_stream))

        def local():
            self.group["step"] += 1
            mine = dp._exchange[0][dp.rank * st.shard: dp.rank * st.shard + k]
            self.adam.step_chunk(st.params[:k], mine, st.exp_avg[:k], st.exp_avg_sq[:k], self.group,
                                 st.bf16[st.start:st.end])

        return self._timed(fused if self.mode in ("fused", "fused_ag", "nvls") else local, reps)

    def breakdown(self, reps: int) -> dict:
        """Separate device times (ms, max over ranks) of the collectives around the kernel."""
        st, dp = self.state, self.dp
        out = {"stream_barrier_ms": self._timed(dp.stream_barrier, reps),
               "all_gather_bf16_ms": self._timed(lambda: dp.all_gather_params(0, force_nccl=True), reps)}
        if self.mode == "nccl":
            full = dp._exchange[0][: st.shard * dp.world_size]
            mine = full[dp.rank * st.shard:(dp.rank + 1) * st.shard]
            out["reduce_scatter_bf16_ms"] = self._timed(
                lambda: dist.reduce_scatter_tensor(mine, full, op=dist.ReduceOp.AVG), reps)
        sent = 2 * st.shard * (dp.world_size - 1)
        out["all_gather_bus_gbs_per_gpu"] = sent / (out["all_gather_bf16_ms"] * 1e-3) / 1e9
        return {"dp_breakdown": out}

    def e2e(self, steps: int, chunk_numel: int = 16 * 1024 * 1024, min_chunk_numel: int = 4 * 1024 * 1024) -> dict:
        """The same step with host buffers: every rank uploads its pinned bf16 gradient into the
        exchange slot and downloads the bf16 copy of its updated slice, inside the timed region,
        pipelined chunk by chunk (`ShardedHostStepper`)."""
        st, dp = self.state, self.dp
        n, k = self.numel, st.end - st.start
        from .host_io import pinned_empty
        g_host = pinned_empty(n, torch.bfloat16, dp.device)
        g_host.copy_(dp.grad_buffer(0)[:n])
        out_host = pinned_empty(max(k, 1), torch.bfloat16, dp.device)
        stepper = ShardedHostStepper(self, chunk_numel, min_chunk_numel)

        def one():
            stepper.step(g_host, out_host, join=False)

        for _ in range(2):
            one()
        stepper.join()
        reps = max(3, min(steps, 20))
        torch.cuda.synchronize(dp.device)
        dp.ctl.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            one()
        stepper.join()
        b.record()
        torch.cuda.synchronize(dp.device)
        t = torch.tensor([a.elapsed_time(b) / reps], device=dp.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        return {"value": n / (ms * 1e-3) / 1e9, "unit": "Gparams/s", "ms_per_step": ms, "steps": reps,
                "h2d_bytes_per_step": 2 * n * dp.world_size, "d2h_bytes_per_step": 2 * n,
                "h2d_gbs_per_gpu": 2 * n / (ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": 2 * k / (ms * 1e-3) / 1e9,
                "path": f"every rank: pinned bf16 gradient -> exchange slot, fused update, bf16 slice -> pinned host; "
                        f"{len(stepper.chunks)} pieces of {min_chunk_numel}..{chunk_numel} elements, upload / update / "
                        "download of neighbouring pieces overlapped on three streams"}

    def close(self):
        self.dp.close()


class ShardedHostStepper:
    """`ShardedLayerAdam.step` for gradients that arrive in pinned HOST memory on every rank and
    bf16 weights that are wanted back in host memory (each rank: the slice it owns): the
    data-parallel counterpart of `host_io.HostGradStepper`.  The layer is cut into pieces; piece
    k+1's upload, piece k's fused update (with its two cross-rank stream barriers) and piece
    k-1's download run concurrently on three streams.  Every piece is one reference call
    (`fused_update` advances the scalar state machine once per piece on every rank).  All ranks
    must call `step` the same number of times."""

    def __init__(self, sharded: ShardedLayerAdam, chunk_numel: int = 16 * 1024 * 1024,
                 min_chunk_numel: Optional[int] = None, slots: int = 2):
        from .host_io import chunk_schedule
        self.sh, self.dp = sharded, sharded.dp
        if self.dp.exchange_slots < slots:
            raise ValueError(f"needs at least {slots} exchange slots")
        self.slots = slots
        self.chunks = chunk_schedule(sharded.numel, int(chunk_numel), int(min_chunk_numel or chunk_numel))
        dev = self.dp.device
        with torch.cuda.device(dev):
            self.s_in, self.s_k, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        nk = len(self.chunks)
        self.ev_in = [torch.cuda.Event() for _ in range(nk)]
        self.ev_k = [torch.cuda.Event() for _ in range(nk)]
        self.ev_out = [torch.cuda.Event() for _ in range(nk)]
        # every rank has finished reading piece k of exchange slot s (recorded behind the trailing barrier)
        self.ev_free = [[torch.cuda.Event() for _ in range(nk)] for _ in range(slots)]
        self._t = 0

    @torch.no_grad()
    def step(self, g_host: torch.Tensor, out_host: Optional[torch.Tensor], join: bool = True):
        sh, dp, st = self.sh, self.dp, self.sh.state
        if not g_host.is_pinned() or (out_host is not None and not out_host.is_pinned()):
            raise RuntimeError("host buffers must be pinned")
        dev = dp.device
        slot = self._t % self.slots
        self._t += 1
        sh.group["step"] += 1
        cur = torch.cuda.current_stream(dev)
        for s in (self.s_in, self.s_k, self.s_out):
            s.wait_stream(cur)
        gbuf = dp.grad_buffer(slot)
        for k, (a, b) in enumerate(self.chunks):
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(self.ev_free[slot][k])
                gbuf[a:b].copy_(g_host[a:b], non_blocking=True)
                self.ev_in[k].record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(self.ev_in[k])
                self.s_k.wait_event(self.ev_out[k])      # last step's download of this piece is done
                dp.fused_update(0, sh.adam, sh.group, a, b, slot=slot, gather=True, barrier=True)
                self.ev_k[k].record(self.s_k)
                self.ev_free[slot][k].record(self.s_k)
            lo, hi = max(a, st.start), min(b, st.end)
            if out_host is not None and hi > lo and st.bf16 is not None:
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_k[k])
                    out_host[lo - st.start:hi - st.start].copy_(st.bf16[lo:hi], non_blocking=True)
                    self.ev_out[k].record(self.s_out)
        if join:
            self.join()

    def join(self):
        cur = torch.cuda.current_stream(self.dp.device)
        cur.wait_stream(self.s_k)
        cur.wait_stream(self.s_out)
