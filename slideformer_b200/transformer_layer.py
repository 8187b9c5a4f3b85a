"""Layer units of the sliding runtime, rescheduled around the fused GPU optimizer step.

Counterpart of the reference's transformer_layer.py (`OffloadLayerWrapper`, `DecoderWrapper`,
`EmbeddingWrapper`, `OutputWrapper`, `split_transformer_model`).  Public methods keep their
names; what they do changes because the optimizer now runs on the GPU:

  reference (CPU optimizer)                              here (B200)
  ----------------------------------------------------   -----------------------------------------
  fp32 master weights in CPU RAM, transformer_layer.py   fp32 master weights + Adam moments in HBM
    :192-196; moments in CPU RAM, layer_adam.py:163-173    (or pinned host memory, streamed)
  to_device_async: CPU fp32->bf16 cast + H2D into a      bf16 weights are permanent in HBM, written by
    window unit on a worker thread, :273-335               the Adam kernel's epilogue; to_device_async
                                                           only takes a gradient unit for backward
  to_offload_async(is_bwd): chunked gradient D2H with    nothing to copy; the gradient unit is handed to
    one event per chunk, :343-422                          the optimizer stream by an event
  update_params: CPU thread consuming chunks, :453-499   one kernel launch per chunk on the optimizer
                                                           stream (or the data-parallel fused update)
  wait_for_update: threading.Event                       a CUDA event the compute stream waits on

No Python worker threads are involved; every dependency is a CUDA event, so the host never
blocks inside a step.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .model_compat import TextModelParts, call_decoder_layer
from .numa import pinned_empty
from .sliding_checkpoint import SlidingCheckpoint

# Optimizer chunk, in elements: the reference's D2H chunk (transformer_layer.py:26-27).
UPDATE_CHUNK_SIZE = 32 * 1024 * 1024

# Operations timed per unit and how they are printed (utils/timer.py:11-21).  There is no
# gradient or weight D2H on this path, so the reference's two "d2h transfer" labels never get a
# sample here; "h2d transfer fw / bw" time the weight-window fill (all-gather or host copy).
TIMING_LABELS = {
    "h2d_transfer_fw": "h2d transfer fw",
    "h2d_transfer_bw": "h2d transfer bw",
    "d2h_transfer_fw": "d2h transfer fw",
    "d2h_transfer_bw": "d2h transfer bw",
    "forward": "forward",
    "backward": "backward",
    "parameter_update": "parameter update",
    "ac_fwd_d2h": "ac fwd d2h",
    "ac_bwd_h2d": "ac bwd h2d",
}


def format_timing_label(operation: str) -> str:
    return TIMING_LABELS.get(operation, operation.replace("_", " "))


class _Span:
    """A CUDA-event pair on one stream plus an NVTX range on the host thread, both optional."""

    def __init__(self, unit, op: str, nvtx_name: Optional[str], stream):
        self.unit, self.op, self.stream = unit, op, stream
        # start/end ranges rather than push/pop: the phases of neighbouring units overlap in time
        self.nvtx = torch.cuda.nvtx.range_start(nvtx_name) if (unit.enable_nvtx and nvtx_name) else None
        self.t0 = None
        if unit.enable_timing:
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t0.record(stream)

    def close(self):
        if self.t0 is not None:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(self.stream)
            spans = self.unit.timings.setdefault(self.op, [])
            spans.append((self.t0, t1))
            if len(spans) > 4096:
                del spans[:2048]
            self.t0 = None
        if self.nvtx is not None:
            torch.cuda.nvtx.range_end(self.nvtx)
            self.nvtx = None


class GradUnitPool:
    """The gradient side of the reference's GPU cache units (offload_transformer.py:205-219):
    a small ring of flat bf16 buffers, each guarded by a `reuse_ready` event recorded when the
    optimizer has consumed it."""

    def __init__(self, num_units: int, numel: int, dtype, device, buffers: Optional[List[torch.Tensor]] = None):
        self.units = []
        for k in range(num_units):
            grad = buffers[k] if buffers is not None else torch.empty(numel, dtype=dtype, device=device)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(device))
            self.units.append({"grad": grad, "reuse_ready": ev, "slot": k})
        self._next = 0

    def get(self):
        u = self.units[self._next % len(self.units)]
        self._next += 1
        return u


class WeightUnitPool:
    """The parameter side of the reference's GPU cache units, used when a model's bf16 weights do
    not fit next to the sharded optimizer state (70B on 8 GPUs): a ring of full-layer bf16
    buffers that a layer's slices are all-gathered into shortly before the layer runs.  `free`
    is recorded on the compute stream after the last kernel that read the unit."""

    def __init__(self, num_units: int, numel: int, dtype, device, with_stage: bool = False):
        self.units = []
        for _ in range(num_units):
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(device))
            self.units.append({"param": torch.empty(numel, dtype=dtype, device=device), "free": ev})
        self._next = 0
        # one-GPU window: the optimizer writes a unit's new bf16 weights here before they go to the
        # unit's pinned host store; every use is on the optimizer stream, so one buffer serves all units
        self.stage = torch.empty(numel, dtype=dtype, device=device) if with_stage else None

    def get(self):
        u = self.units[self._next % len(self.units)]
        self._next += 1
        return u


def _init_like_hf(name: str, shape, device, generator) -> torch.Tensor:
    """Random init for a parameter that exists only on the meta device: N(0, 0.02) weights, unit
    norm scales, zero biases (the Hugging Face defaults for the families handled here)."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "bias":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if len(shape) == 1:
        return torch.ones(shape, dtype=torch.float32, device=device)
    return torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=generator)


class OffloadLayerWrapper(nn.Module):
    """Base class: owns one unit's flat fp32 master weights, its permanent bf16 weights and the
    scheduling of its optimizer step."""

    def __init__(self, layer: nn.Module, device: torch.device, layer_idx: int,
                 offload_device: torch.device = torch.device("cpu"), grad_pool: Optional[GradUnitPool] = None,
                 opt_stream: Optional[torch.cuda.Stream] = None, skip_params: Optional[set] = None,
                 tied_param: Optional[nn.Parameter] = None, enable_timing: bool = False, is_last_layer: bool = False,
                 layer_optimizer=None, dtype: torch.dtype = torch.bfloat16, state_device: str = "hbm",
                 shared_dp=None, update_chunk: int = UPDATE_CHUNK_SIZE, weight_pool: Optional[WeightUnitPool] = None,
                 comm_stream: Optional[torch.cuda.Stream] = None, init_seed: int = 0, enable_nvtx: bool = True,
                 opt_stream_alt: Optional[torch.cuda.Stream] = None):
        super().__init__()
        if layer_optimizer is None:
            raise RuntimeError("a shared LayerAdam must be provided")
        if state_device not in ("hbm", "host"):
            raise ValueError("state_device must be 'hbm' or 'host'")
        self.device, self.layer_idx, self.is_last_layer, self.dtype = device, layer_idx, is_last_layer, dtype
        self.layer = layer
        self.grad_pool = grad_pool
        self.opt_stream = opt_stream
        # Units whose state streams from host memory alternate between two optimizer streams: the
        # library's copies of two calls issued from different streams overlap (the uploads of one
        # unit start while the downloads of the previous one drain)
        # (not with the one-GPU weight window, whose single bf16 staging buffer relies on one stream)
        if (state_device == "host" and shared_dp is None and opt_stream_alt is not None and weight_pool is None
                and (layer_idx & 1)):
            self.opt_stream = opt_stream_alt
        self.layer_optimizer = layer_optimizer
        self.state_device = state_device
        self.shared_dp = shared_dp
        self.update_chunk = int(update_chunk)
        self.enable_timing = enable_timing
        self.enable_nvtx = enable_nvtx
        self._fw_span = self._bw_span = None
        self.skip_params = skip_params or set()
        self.tied_param = tied_param
        self._is_tied_output = tied_param is not None and tied_param in self.skip_params

        self.compute_ready = torch.cuda.Event()
        self.compute_ready_bw = torch.cuda.Event()
        self.update_done = torch.cuda.Event()
        self._update_recorded = False
        self._unit = None
        self._pending = 0          # parameters whose gradient has not been accumulated yet
        self._in_backward = False
        self.timings: Dict[str, List] = {"parameter_update": []}
        self.host_update_seconds = 0.0   # host time spent enqueueing optimizer steps (not device time)

        self.own_grad_unit = None    # batched small-unit mode: this unit's private exchange slot
        self.defer_to = None         # batched small-unit mode: list the engine drains after backward
        self.weight_pool = weight_pool
        self.comm_stream = comm_stream
        self.weights_ready = torch.cuda.Event()
        self._wunit = None
        if weight_pool is not None and tied_param is not None:
            raise ValueError("the weight window needs untied embeddings")
        self._bf16_host = None   # one-GPU window mode: the permanent bf16 weights, in pinned host memory

        # parameters that exist only on the meta device are created here, directly in their final place
        gen = torch.Generator(device=device).manual_seed(1000003 * init_seed + layer_idx)
        meta_init = {}
        for n_, p_ in list(self.layer.named_parameters()):
            if p_.is_meta and p_ not in self.skip_params:
                owner_name, _, leaf = n_.rpartition(".")
                owner = self.layer.get_submodule(owner_name) if owner_name else self.layer
                newp = nn.Parameter(torch.empty(0, dtype=dtype, device=device), requires_grad=p_.requires_grad)
                meta_init[id(newp)] = (n_, tuple(p_.shape))
                owner._parameters[leaf] = newp
        self._managed_named_params = [(n, p) for n, p in self.layer.named_parameters() if p not in self.skip_params]
        shapes = {n_: (meta_init[id(p_)][1] if id(p_) in meta_init else tuple(p_.shape)) for n_, p_ in self._managed_named_params}
        self.total_size = sum(int(torch.Size(sh).numel()) for sh in shapes.values())
        n = self.total_size

        # ---- storage: fp32 masters (+ moments in the optimizer) and permanent bf16 weights ----
        if shared_dp is not None:
            st = shared_dp.register_layer(layer_idx, n, resident_bf16=weight_pool is None)
            self._dp_state = st
            self._params_flat = st.params                      # this rank's fp32 slice
            self._bf16_flat = st.bf16[:n] if st.bf16 is not None else None   # full layer, or None in window mode
            self._dp_group = None
        else:
            self._dp_state = None
            if state_device == "hbm":
                self._params_flat = torch.empty(n, dtype=torch.float32, device=device)
            else:
                self._params_flat = pinned_empty(n, torch.float32, device)
            if weight_pool is None:
                self._bf16_flat = torch.empty(n, dtype=dtype, device=device)
            else:
                # one-GPU weight window (the reference's headline mode, offload_transformer.py:75-79,
                # transformer_layer.py:273-335): the bf16 weights wait in pinned host memory and are
                # copied into a window unit one unit ahead of the compute stream
                self._bf16_flat = None
                self._bf16_host = pinned_empty(n, dtype, device)

        self._param_maps = OrderedDict()
        self._master_views = []
        self._bf16_views = []
        with torch.no_grad():
            off = 0
            full_fp32 = torch.empty(n, dtype=torch.float32, device=device) if shared_dp is not None else None
            for name, p in self._managed_named_params:
                shape = torch.Size(shapes[name])
                k = shape.numel()
                self._param_maps[name] = (off, shape, k)
                if id(p) in meta_init:
                    src = _init_like_hf(name, shape, device, gen).to(dtype).float().reshape(-1)
                else:
                    src = p.data.detach().to(device=device, dtype=torch.float32).reshape(-1)
                if shared_dp is not None:
                    full_fp32[off:off + k].copy_(src)
                else:
                    self._params_flat[off:off + k].copy_(src, non_blocking=True)
                if self._bf16_flat is not None:
                    self._bf16_flat[off:off + k].copy_(src)
                    p.data = self._bf16_flat[off:off + k].view(shape)   # the weights the layer computes with
                else:
                    if self._bf16_host is not None:
                        self._bf16_host[off:off + k].copy_(src.to(dtype))
                    p.data = torch.empty(0, dtype=dtype, device=device)  # pointed into a window unit on demand
                p.grad = None
                off += k
                del src
            if shared_dp is not None:
                shared_dp.load_full_params(layer_idx, full_fp32)
                del full_fp32
            else:
                off = 0
                for name, p in self._managed_named_params:
                    _, shape, k = self._param_maps[name]
                    self._master_views.append(nn.Parameter(self._params_flat[off:off + k].view(shape), requires_grad=False))
                    if self._bf16_flat is not None:
                        self._bf16_views.append(self._bf16_flat[off:off + k].view(shape))
                    off += k
                self.layer_optimizer.add_layer_params(layer_idx, self._master_views,
                                                      self._bf16_views if self._bf16_flat is not None else None)
        for module in layer.modules():   # constants stay on the compute device (transformer_layer.py:148-152)
            for bname, buf in module.named_buffers(recurse=False):
                if buf is not None and not buf.is_meta and buf.device != device:
                    module._buffers[bname] = buf.to(device)
        # autograd keeps these callables on the C++ side, where Python's cycle collector cannot see
        # them: close() removes them, otherwise the unit (and its HBM) outlives its last reference
        self._hook_handles = []
        for _, p in self._managed_named_params:
            if p.requires_grad:
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._on_param_grad))

    # ---- window management (names of transformer_layer.py:273-343) ------------------------------
    def to_device_async(self, is_bwd: bool = False, bwd_phase: Optional[bool] = None):
        """Forward needs nothing (the bf16 weights are resident).  For backward: take the next
        gradient unit, wait until the optimizer has released it, zero it and point every
        parameter's .grad into it, so autograd accumulates straight into the flat buffer."""
        if self.weight_pool is not None and self._wunit is None and not (is_bwd and isinstance(self, EmbeddingWrapper)):
            self._acquire_weights(is_bwd if bwd_phase is None else bwd_phase)
        if not is_bwd or self._unit is not None:
            return
        unit = self.own_grad_unit if self.own_grad_unit is not None else self.grad_pool.get()
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(unit["reuse_ready"])
        g = unit["grad"]
        g[: self.total_size].zero_()
        self._pending = 0
        for name, p in self._managed_named_params:
            off, shape, k = self._param_maps[name]
            if p.requires_grad:
                p.grad = g[off:off + k].view(shape)
                self._pending += 1
        self._unit = unit

    def _acquire_weights(self, is_bwd: bool = False):
        """Window mode: all-gather this unit's bf16 slices into the next window unit on the
        communication stream (behind the unit's last optimizer step and the unit's previous
        reader) and point the parameters into it (the counterpart of the reference's H2D task,
        transformer_layer.py:273-335)."""
        unit = self.weight_pool.get()
        cs = self.comm_stream
        with torch.cuda.stream(cs):
            cs.wait_event(unit["free"])
            span = _Span(self, "h2d_transfer_bw" if is_bwd else "h2d_transfer_fw", f"H2D_Layer_{self.layer_idx}", cs)
            if self._update_recorded:
                cs.wait_event(self.update_done)
            if self.shared_dp is not None:
                self.shared_dp.gather_weights(self.layer_idx, unit["param"])
            else:
                unit["param"][: self.total_size].copy_(self._bf16_host, non_blocking=True)
            span.close()
            self.weights_ready.record(cs)
        for name, p in self._managed_named_params:
            off, shape, k = self._param_maps[name]
            p.data = unit["param"][off:off + k].view(shape)
        self._wunit = unit

    def wait_for_h2d(self):
        if self._wunit is not None:
            torch.cuda.current_stream(self.device).wait_event(self.weights_ready)

    def release_weights(self):
        """The compute stream is done with this unit's window buffer."""
        if self._wunit is not None:
            self._wunit["free"].record(torch.cuda.current_stream(self.device))
            self._wunit = None

    def to_offload_async(self, is_bwd: bool = False, prev_update=None):
        """Backward: mark the gradients complete on the compute stream (the counterpart of the
        reference handing the unit to its D2H worker)."""
        if is_bwd:
            self.compute_ready_bw.record(torch.cuda.current_stream(self.device))
            self.end_backward_span()

    def wait_for_d2h(self):
        return None

    # ---- timing / NVTX ranges of the compute phases (names of transformer_layer.py:524, offload_transformer.py:262)
    def begin_forward_span(self):
        if self.enable_timing or self.enable_nvtx:
            self._fw_span = _Span(self, "forward", f"Forward_Layer_{self.layer_idx}", torch.cuda.current_stream(self.device))

    def end_forward_span(self):
        if self._fw_span is not None:
            self._fw_span.close()
            self._fw_span = None

    def begin_backward_span(self):
        self._in_backward = True
        if (self.enable_timing or self.enable_nvtx) and self._bw_span is None:
            self._bw_span = _Span(self, "backward", f"Backward_Compute_Layer_{self.layer_idx}",
                                  torch.cuda.current_stream(self.device))

    def end_backward_span(self):
        self._in_backward = False
        if self._bw_span is not None:
            self._bw_span.close()
            self._bw_span = None

    def _on_param_grad(self, _param):
        if self._unit is None:
            return
        self._pending -= 1
        if self._pending == 0:
            self.to_offload_async(is_bwd=True)
            self.release_weights()
            self.update_params()

    def flush(self):
        """Run the update for a unit whose backward finished without touching every parameter."""
        self.release_weights()
        if self._unit is not None:
            self.to_offload_async(is_bwd=True)
            self.update_params()

    # ---- the optimizer step ----------------------------------------------------------------------
    def update_params(self):
        """Enqueue this unit's Adam step on the optimizer stream, behind `compute_ready_bw`."""
        if self._unit is not None and self.defer_to is not None:
            # batched small-unit mode: the engine updates all units in one launch after backward
            self.defer_to.append((self, self._unit))
            self._unit = None
            return None
        unit, self._unit = self._unit, None
        if unit is None:
            return None
        _h0 = time.perf_counter()
        n = self.total_size
        g = unit["grad"]
        opt = self.layer_optimizer
        s = self.opt_stream
        with torch.cuda.stream(s):
            s.wait_event(self.compute_ready_bw)
            span = _Span(self, "parameter_update", f"Update_Layer_{self.layer_idx}", s)
            if self.shared_dp is not None:
                if self._dp_group is None:
                    self._dp_group = dict(opt.defaults, step=0)
                self._dp_group["step"] += 1
                self._dp_group["lr"] = opt.defaults["lr"]
                self._dp_state.step = self._dp_group["step"]
                for cs in range(0, n, self.update_chunk):
                    ce = min(cs + self.update_chunk, n)
                    # the unit's whole gradient is complete here on every rank once the first
                    # chunk's barrier has passed, so later chunks need none
                    self.shared_dp.fused_update(self.layer_idx, opt, self._dp_group, cs, ce, slot=unit["slot"],
                                                gather=False, barrier=(cs == 0))
                self.shared_dp.all_gather_params(self.layer_idx)
            else:
                group = opt.begin_chunk_step(self.layer_idx)
                m, v = opt.exp_avg_flat[self.layer_idx], opt.exp_avg_sq_flat[self.layer_idx]
                bf16_out = self._bf16_flat if self._bf16_flat is not None else self.weight_pool.stage[:n]
                if self.state_device == "hbm":
                    for cs in range(0, n, self.update_chunk):
                        ce = min(cs + self.update_chunk, n)
                        opt.step_chunk(self._params_flat[cs:ce], g[cs:ce], m[cs:ce], v[cs:ce], group, bf16_out[cs:ce])
                else:
                    # host-resident state: chunked and double-buffered inside the library, one
                    # reference call per chunk like the reference's chunk consumer
                    opt.step_chunk(self._params_flat, g[:n], m, v, group, bf16_out,
                                   host_chunk_calls=True, host_chunk_numel=self.update_chunk)
                opt.end_chunk_step(self.layer_idx)
                if self._bf16_host is not None:
                    self._bf16_host.copy_(bf16_out, non_blocking=True)   # the next prefetch reads it from here
            span.close()
            self.update_done.record(s)
            unit["reuse_ready"].record(s)
        self._update_recorded = True
        for _, p in self._managed_named_params:
            p.grad = None
        self.host_update_seconds += time.perf_counter() - _h0
        return self.update_done

    def close(self):
        """Release the unit: remove the gradient hooks and drop every large buffer it owns.  The
        module is unusable afterwards."""
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []
        for _, p in self._managed_named_params:
            p.grad = None
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        self._params_flat = self._bf16_flat = self._bf16_host = None
        self._master_views, self._bf16_views = [], []
        self._unit = self._wunit = self.own_grad_unit = None
        self.grad_pool = self.weight_pool = self.defer_to = None
        self._dp_state = None
        self.timings = {}

    def wait_for_update(self):
        """Order the compute stream after this unit's last optimizer step."""
        if self._update_recorded:
            torch.cuda.current_stream(self.device).wait_event(self.update_done)

    def master_params_full(self) -> torch.Tensor:
        """Flat fp32 master weights on the device (for saving); sharded state is gathered from bf16."""
        if self.shared_dp is not None:
            if self._bf16_flat is None:
                raise NotImplementedError("gathering fp32 masters from window-mode shards is not implemented")
            return self._bf16_flat.float()
        return self._params_flat.to(self.device)

    def bf16_weights_flat(self) -> torch.Tensor:
        """This unit's current bf16 weights as one flat tensor (device-resident, or the pinned host
        store in one-GPU window mode).  Sharded window mode keeps only slices: gather them instead."""
        if self._bf16_flat is not None:
            return self._bf16_flat
        if self._bf16_host is not None:
            return self._bf16_host
        raise RuntimeError("only slices of this unit's bf16 weights are resident; all-gather them")

    def forward(self, *args, **kwargs):
        raise NotImplementedError


class DecoderWrapper(OffloadLayerWrapper):
    """One decoder layer under torch's non-reentrant checkpoint (transformer_layer.py:510-566)."""

    def __init__(self, *args, activation_checkpoint: bool = True, **kwargs):
        super().__init__(*args, **kwargs)
        self.activation_checkpoint = activation_checkpoint
        self.activation_store = None   # set by the engine when activations go to pinned host memory

    def forward(self, hidden_states, **layer_kwargs):
        def _forward(h):
            return call_decoder_layer(self.layer, h, layer_kwargs)

        if not self.activation_checkpoint or not torch.is_grad_enabled():
            out = _forward(hidden_states)
        else:
            with SlidingCheckpoint(self.layer_idx, self.activation_store, self.is_last_layer):
                out = checkpoint(_forward, hidden_states, use_reentrant=False)
        self.compute_ready.record(torch.cuda.current_stream(self.device))
        return out


class EmbeddingWrapper(OffloadLayerWrapper):
    def forward(self, input_ids, **kwargs):
        out = self.layer(input_ids, **kwargs)
        self.compute_ready.record(torch.cuda.current_stream(self.device))
        return out


class OutputWrapper(OffloadLayerWrapper):
    """Final norm + LM head + shifted cross entropy (transformer_layer.py:584-630).  The loss is
    plain torch (`F.linear` + `F.cross_entropy` in fp32 over token chunks); the reference's
    Triton fused loss is not used."""

    def __init__(self, norm_layer: nn.Module, lm_head: nn.Module, *args, softcap=None, loss_chunk_tokens: int = 4096,
                 **kwargs):
        combined = nn.Sequential(norm_layer, lm_head)
        super().__init__(combined, *args, **kwargs)
        self.norm_layer, self.lm_head, self.softcap = norm_layer, lm_head, softcap
        self.loss_chunk_tokens = int(loss_chunk_tokens)

    VOCAB_ALIGN = 64

    def _logits(self, h, mask_padding: bool = False):
        """LM-head logits.  A vocabulary that is not a multiple of 64 (GPT-2: 50257) would give the
        GEMM an odd leading dimension and send cuBLAS to a legacy unaligned kernel (measured: 43 %
        of a GPT-2 small step), so the weight is zero-padded to the next multiple of 64 rows and
        the extra logits are either dropped (view) or set to -inf for the loss."""
        w, b = self.lm_head.weight, self.lm_head.bias
        vocab = w.shape[0]
        pad = (-vocab) % self.VOCAB_ALIGN
        if pad:
            w = F.pad(w, (0, 0, 0, pad))
            b = F.pad(b, (0, pad)) if b is not None else None
        out = F.linear(h, w, b)
        if self.softcap is not None:
            out = torch.tanh(out / self.softcap) * self.softcap
        if pad:
            if not mask_padding:
                return out[..., :vocab]
            out = out.float()
            out[..., vocab:] = float("-inf")
        return out

    def forward(self, hidden_states, labels=None):
        h = self.norm_layer(hidden_states)
        if labels is None:
            out = self._logits(h)
        else:
            h = h[..., :-1, :].contiguous().view(-1, h.size(-1))
            y = labels[..., 1:].contiguous().view(-1)
            valid = (y != -100).sum().clamp(min=1)

            def chunk_loss(hc, yc):
                return F.cross_entropy(self._logits(hc, mask_padding=True).float(), yc, ignore_index=-100,
                                       reduction="sum")

            total = None
            for cs in range(0, h.shape[0], self.loss_chunk_tokens):
                hc, yc = h[cs:cs + self.loss_chunk_tokens], y[cs:cs + self.loss_chunk_tokens]
                part = checkpoint(chunk_loss, hc, yc, use_reentrant=False) if torch.is_grad_enabled() else chunk_loss(hc, yc)
                total = part if total is None else total + part
            out = total / valid
        self.compute_ready.record(torch.cuda.current_stream(self.device))
        return out


def split_transformer_model(parts: TextModelParts, device: torch.device, dtype: torch.dtype = torch.bfloat16,
                            **kwargs) -> Dict[str, Any]:
    """Wrap embedding (idx 0), decoder layers (1..L) and norm + head (L+1) as streamed units
    (transformer_layer.py:29-111).  A tied head weight is owned by the embedding unit and skipped
    by the output unit; autograd sums both uses before the owner's gradient hook fires."""
    activation_checkpoint = kwargs.pop("activation_checkpoint", True)
    loss_chunk_tokens = kwargs.pop("loss_chunk_tokens", 4096)
    placement = kwargs.pop("state_devices", None)   # optional per-unit "hbm" / "host", overrides state_device
    tied = parts.tied_param
    L = len(parts.layers)

    def kw(idx):
        return dict(kwargs, state_device=placement[idx]) if placement is not None else kwargs

    units = nn.ModuleList([])
    units.append(EmbeddingWrapper(parts.embed, device, 0, dtype=dtype, tied_param=tied, **kw(0)))
    for idx, layer in enumerate(parts.layers, start=1):
        units.append(DecoderWrapper(layer, device, idx, dtype=dtype, is_last_layer=(idx == L),
                                    activation_checkpoint=activation_checkpoint, **kw(idx)))
    units.append(OutputWrapper(parts.norm, parts.lm_head, device, L + 1, dtype=dtype,
                               softcap=getattr(parts.config, "final_logit_softcapping", None),
                               skip_params={tied} if tied is not None else None, tied_param=tied,
                               loss_chunk_tokens=loss_chunk_tokens, **kw(L + 1)))
    return {"transformer_layers": units, "rotary_emb": parts.rotary_emb}
