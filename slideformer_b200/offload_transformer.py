"""SlideFormerOffloader: the layer-sliding fine-tuning engine around the GPU LayerAdam.

Counterpart of the reference's offload_transformer.py:28-597 (and of its data-parallel copy,
multi_gpu/offload_transformer.py): same constructor keywords, `forward(input_ids,
attention_mask, labels, position_ids, return_dict)`, `wait_for_completion()`,
`update_learning_rate()`, `save_pretrained()`.

Schedule of one step (all ordering by CUDA events, no worker threads):

  forward   unit i: compute stream waits for unit i's last optimizer step (`update_done`), runs
            the layer on the permanent bf16 weights; decoder layers keep one checkpoint tensor
            (in HBM, or in pinned host memory through `SlidingCheckpoint`).
  backward  unit i, pre-hook: take a gradient unit from the ring (wait for its `reuse_ready`),
            zero it, point .grad views into it.  When the last parameter of the unit has
            accumulated its gradient, `compute_ready_bw` is recorded and the optimizer stream
            runs the fused Adam kernel over the unit (fp32 p/m/v in place, bf16 weights out),
            overlapping with the backward of unit i-1 on the compute stream.

The reference's `double_buffer` selects 2 instead of 1 spare window units
(offload_transformer.py:75-79); here it selects 3 instead of 2 gradient units.
"""
from __future__ import annotations

import time
from typing import Optional

import torch
import torch.nn as nn

from .layer_adam import LayerAdam
from .model_compat import parameter_sizes, prepare_layer_inputs, validate_model
from .sliding_checkpoint import ActivationStore
from .shared_data_parallel import shard_numel
from .transformer_layer import GradUnitPool, WeightUnitPool, split_transformer_model


def unit_numels(parts) -> list:
    """Parameters per streamed unit, in unit order: embedding, decoder layers, norm + head (a tied
    head weight counts once, in the embedding unit)."""
    def count(mods, skip=()):
        seen, total = set(id(s) for s in skip), 0
        for mod in mods:
            for p in mod.parameters():
                if id(p) not in seen:
                    seen.add(id(p))
                    total += p.numel()
        return total
    tied = [parts.tied_param] if parts.tied_param is not None else []
    return [count([parts.embed])] + [count([layer]) for layer in parts.layers] + [count([parts.norm, parts.lm_head], tied)]


def plan_state_placement(unit_sizes, budget_bytes: int) -> list:
    """'hbm' or 'host' per unit: units keep their fp32 master weights and both Adam moments
    (12 bytes per parameter) in HBM, in unit order, while the budget lasts; the rest live in
    pinned host memory and are streamed through the GPU by the update."""
    placement, used = [], 0
    for n in unit_sizes:
        need = 12 * int(n)
        if used + need <= budget_bytes:
            placement.append("hbm")
            used += need
        else:
            placement.append("host")
    return placement


class CausalLMOutput(dict):
    """Minimal stand-in for transformers' CausalLMOutputWithPast (attribute and key access)."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e


class SlideFormerOffloader(nn.Module):
    def __init__(self, model, device: torch.device, dtype: torch.dtype = torch.bfloat16, ac_offload_nvme: bool = False,
                 offload_dir: str = "/RAID0", double_buffer: bool = False, enable_timing: bool = True,
                 enable_memory_stats: bool = True, optimizer_kwargs: Optional[dict] = None,
                 auto_backward_in_forward: bool = True, shared_dp=None, *, state_device: str = "hbm",
                 activation_offload: str = "hbm", activation_checkpoint: bool = True, loss_chunk_tokens: int = 4096,
                 update_chunk: Optional[int] = None, weight_window: bool = False,
                 hbm_state_budget_gb: Optional[float] = None, enable_nvtx: bool = True,
                 batch_small_units: Optional[bool] = None):
        super().__init__()
        if not isinstance(device, torch.device):
            raise TypeError("device must be torch.device")
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("dtype must be float16 or bfloat16")
        if dtype != torch.bfloat16:
            raise NotImplementedError("the fused optimizer emits bfloat16 weights; float16 is not supported")
        if ac_offload_nvme:
            raise NotImplementedError("NVMe activation offload is not part of this build; use activation_offload='host'")
        if activation_offload not in ("hbm", "host"):
            raise ValueError("activation_offload must be 'hbm' or 'host'")
        if state_device not in ("hbm", "host", "auto"):
            raise ValueError("state_device must be 'hbm', 'host' or 'auto'")
        if state_device == "auto" and shared_dp is not None:
            raise ValueError("state_device='auto' applies to one GPU; sharded state is always HBM-resident")
        self.device, self.dtype = device, dtype
        self.double_buffer = double_buffer
        self.auto_backward_in_forward = auto_backward_in_forward
        self.enable_timing = enable_timing
        self.enable_memory_stats = enable_memory_stats
        self.shared_dp = shared_dp
        self.state_device = state_device
        self.activation_offload = activation_offload
        self.base_model = model
        self.parts = validate_model(model)
        self.config = self.parts.config
        self.decoder_layers = self.parts.layers
        self.max_param_size, self.total_param = parameter_sizes(model)
        self.is_tied = self.parts.tied_param is not None
        self.tied_param = self.parts.tied_param

        defaults = {"lr": 1e-5, "bias_correction": True, "weight_decay": 0.01, "eps": 1e-8,
                    "fp32_optimizer_state": True, "num_layer": len(self.decoder_layers) + 2}
        self.layer_optimizer = LayerAdam(**(optimizer_kwargs or defaults))

        with torch.cuda.device(device):
            self.opt_stream = torch.cuda.Stream()
            self.opt_stream_alt = torch.cuda.Stream()
        n_units = min(3 if double_buffer else 2, len(self.decoder_layers) + 2)
        self.gpu_unit_size = n_units
        # Small models under data parallelism: every unit keeps its own exchange slot and all units
        # are updated by ONE multi-segment launch (one barrier pair) after backward, instead of one
        # launch and two cross-rank barriers per unit, which cost more than the update itself when
        # a unit has a few million parameters.  Default: on when the per-unit slots fit in 2 GiB.
        all_units = len(self.decoder_layers) + 2
        slots_bytes = all_units * self.max_param_size * 2
        can_batch = (shared_dp is not None and not weight_window and shared_dp.push_weights and not shared_dp.nvls
                     and shared_dp.world_size <= 8 and shared_dp.dtype == torch.bfloat16)
        if batch_small_units is None:
            batch_small_units = can_batch and slots_bytes <= (2 << 30) and shared_dp._cap == 0
        elif batch_small_units and not can_batch:
            raise ValueError("batch_small_units needs shared_dp in push mode with resident bf16 weights and at most 8 ranks")
        self.batch_small_units = bool(batch_small_units)
        self._deferred = []
        if shared_dp is not None:
            if self.batch_small_units:
                shared_dp.ensure_exchange_slots(all_units)
            if shared_dp.exchange_slots < n_units:
                raise ValueError(f"shared_dp needs at least {n_units} exchange slots")
            shared_dp.reserve_exchange(self.max_param_size)
        self._grad_pool = None  # built after the layers registered (the exchange buffers may grow)

        self.weight_window = bool(weight_window)
        self.weight_pool = self.comm_stream = None
        if self.weight_window:
            # with shared_dp: bf16 slices stay resident and a unit is all-gathered into the window;
            # on one GPU: the bf16 weights wait in pinned host memory and are copied into the window
            with torch.cuda.device(device):
                self.comm_stream = torch.cuda.Stream()
            if shared_dp is not None:
                unit_elems = shard_numel(self.max_param_size, shared_dp.world_size) * shared_dp.world_size
            else:
                unit_elems = -(-self.max_param_size // 128) * 128
            self.weight_pool = WeightUnitPool(3 if double_buffer else 2, unit_elems, dtype, device,
                                              with_stage=shared_dp is None)
        # where each unit's fp32 state lives: everywhere the same, or planned against an HBM budget
        self.state_placement = None
        if state_device == "auto":
            sizes = unit_numels(self.parts)
            if hbm_state_budget_gb is None:
                free = torch.cuda.mem_get_info(device)[0]
                resident_weights = 0 if self.weight_window else 2 * sum(sizes)
                reserve = resident_weights + n_units * 2 * max(sizes) + (24 << 30)   # weights, gradient ring, activations
                budget = max(0, int(0.9 * (free - reserve)))
            else:
                budget = int(hbm_state_budget_gb * (1 << 30))
            self.state_placement = plan_state_placement(sizes, budget)
            self.hbm_state_budget_bytes = budget
        kwargs = dict(weight_pool=self.weight_pool, comm_stream=self.comm_stream,
                      opt_stream=self.opt_stream, opt_stream_alt=self.opt_stream_alt, enable_timing=enable_timing,
                      layer_optimizer=self.layer_optimizer,
                      state_device=("hbm" if state_device == "auto" else state_device), shared_dp=shared_dp,
                      activation_checkpoint=activation_checkpoint, loss_chunk_tokens=loss_chunk_tokens,
                      enable_nvtx=enable_nvtx)
        if self.state_placement is not None:
            kwargs["state_devices"] = self.state_placement
        if update_chunk is not None:
            kwargs["update_chunk"] = update_chunk
        comps = split_transformer_model(self.parts, device, dtype, **kwargs)
        self.transformer_layers = comps["transformer_layers"]
        self.rotary_emb = comps["rotary_emb"]
        self.embed_layer = self.transformer_layers[0]
        self.output_layer = self.transformer_layers[-1]

        buffers = None
        if shared_dp is not None:
            buffers = [shared_dp.grad_buffer(k) for k in range(n_units)]
        self._grad_pool = GradUnitPool(n_units, self.max_param_size, dtype, device, buffers)
        for u in self.transformer_layers:
            u.grad_pool = self._grad_pool
        if self.batch_small_units:
            for j, u in enumerate(self.transformer_layers):
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(device))
                u.own_grad_unit = {"grad": shared_dp.grad_buffer(j), "reuse_ready": ev, "slot": j}
                u.defer_to = self._deferred

        self.activation_store = None
        self._activation_layout_signature = None
        self._register_layer_hooks()
        self.last_step_seconds = None

    # ---- hooks (offload_transformer.py:221-308) ---------------------------------------------------
    def _register_layer_hooks(self):
        units = self.transformer_layers
        last = len(units) - 1

        def pre_forward(module, args):
            module.begin_forward_span()
            if self.weight_window:
                module.to_device_async()                       # no-op if the prefetch already took a unit
                if module.layer_idx < last:
                    units[module.layer_idx + 1].to_device_async()   # prefetch the next unit's weights
                module.wait_for_h2d()
            module.wait_for_update()
            return None

        def post_forward(module, args, output):
            module.end_forward_span()
            # the output unit keeps its weights: its backward starts right away
            if self.weight_window and (module.layer_idx < last or not torch.is_grad_enabled()):
                module.release_weights()
            return None

        def pre_backward(module, grad_output):
            module.begin_backward_span()
            module.to_device_async(is_bwd=True)
            if self.weight_window:
                if module.layer_idx > 1:
                    units[module.layer_idx - 1].to_device_async(bwd_phase=True)   # prefetch the previous unit's weights
                module.wait_for_h2d()
            return None

        self._hook_handles = []
        for unit in units:
            self._hook_handles += [unit.register_forward_pre_hook(pre_forward), unit.register_forward_hook(post_forward),
                                   unit.register_full_backward_pre_hook(pre_backward)]

    def close(self):
        """Drain the last step and release everything the engine holds on the GPU and in pinned host
        memory: hooks, units, optimizer state, gradient and window rings, the activation store.
        Autograd keeps hook callables where Python's cycle collector cannot see them, so an engine
        that is merely dropped stays alive; call this before building another one."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        self.wait_for_completion()
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []
        for unit in self.transformer_layers:
            unit.close()
        opt = self.layer_optimizer
        opt.exp_avg_flat.clear()
        opt.exp_avg_sq_flat.clear()
        opt.state.clear()
        opt.param_groups.clear()
        opt._scratch = {}
        self._grad_pool = self.weight_pool = self.activation_store = None
        self._deferred = []

    def wait_for_completion(self) -> None:
        """Drain the step: flush units whose backward left parameters untouched, make the compute
        stream wait for the optimizer stream, and synchronise (offload_transformer.py:326-335)."""
        for unit in self.transformer_layers:
            unit.flush()
        self._update_deferred_units()
        torch.cuda.current_stream(self.device).wait_stream(self.opt_stream)
        torch.cuda.current_stream(self.device).wait_stream(self.opt_stream_alt)
        torch.cuda.synchronize(self.device)

    def _update_deferred_units(self):
        """Batched small-unit mode: one multi-segment update of every unit whose backward finished,
        in the order they finished (the order the reference updates them), on the optimizer stream."""
        if not self._deferred:
            return
        import time as _time
        h0 = _time.perf_counter()
        opt, dp, s = self.layer_optimizer, self.shared_dp, self.opt_stream
        pending, self._deferred[:] = list(self._deferred), []
        items = []
        with torch.cuda.stream(s):
            for u, unit in pending:
                s.wait_event(u.compute_ready_bw)
                if u._dp_group is None:
                    u._dp_group = dict(opt.defaults, step=0)
                u._dp_group["step"] += 1
                u._dp_group["lr"] = opt.defaults["lr"]
                u._dp_state.step = u._dp_group["step"]
                for cs in range(0, u.total_size, u.update_chunk):
                    items.append((u.layer_idx, u._dp_group, cs, min(cs + u.update_chunk, u.total_size), unit["slot"]))
            from .transformer_layer import _Span
            span = _Span(pending[0][0], "parameter_update", "Update_All_Layers", s)
            dp.fused_update_multi(items, opt)
            span.close()
            for u, unit in pending:
                u.update_done.record(s)
                unit["reuse_ready"].record(s)
                u._update_recorded = True
                for _, p in u._managed_named_params:
                    p.grad = None
        pending[0][0].host_update_seconds += _time.perf_counter() - h0

    def _ensure_activation_storage(self, batch_size, seq_length, hidden_size):
        if self.activation_offload != "host":
            return
        sig = (batch_size, seq_length, hidden_size)
        if self._activation_layout_signature == sig:
            self.activation_store.reset()
            return
        self.activation_store = ActivationStore(len(self.decoder_layers), sig, self.dtype, self.device)
        self.activation_store.timing = bool(self.enable_timing)
        for unit in self.transformer_layers[1:-1]:
            unit.activation_store = self.activation_store
        self._activation_layout_signature = sig

    def forward(self, input_ids, attention_mask=None, labels=None, position_ids=None, return_dict=None):
        return_dict = True if return_dict is None else return_dict
        t0 = time.perf_counter()
        if self.parts.kind == "gpt2":
            hidden = self.embed_layer(input_ids, position_ids=position_ids)
        else:
            hidden = self.embed_layer(input_ids)
        layer_inputs = prepare_layer_inputs(self.parts, hidden, attention_mask, position_ids)
        self._ensure_activation_storage(hidden.shape[0], hidden.shape[1], hidden.shape[2])
        for idx in range(1, len(self.transformer_layers) - 1):
            hidden = self.transformer_layers[idx](hidden, **layer_inputs[idx - 1])
        loss = logits = None
        if labels is not None:
            loss = self.output_layer(hidden, labels=labels)
            if self.auto_backward_in_forward:
                loss.backward()
                self.wait_for_completion()
                self.last_step_seconds = time.perf_counter() - t0
        else:
            logits = self.output_layer(hidden, labels=None)
        if not return_dict:
            return tuple(v for v in (loss, logits) if v is not None)
        return CausalLMOutput(loss=loss, logits=logits, past_key_values=None)

    def update_learning_rate(self, new_lr):
        self.layer_optimizer.update_learning_rate(new_lr)

    # ---- gradient-side work folded into the update kernels ------------------------------------------
    def enable_grad_stats(self):
        """Every update of the coming steps also accumulates sum(g*g) and a non-finite flag of the
        gradients it consumes (no extra pass over HBM); read them with `read_grad_stats`."""
        self.layer_optimizer.enable_grad_stats(self.device)

    def set_grad_scale(self, scale: float):
        """Multiply every gradient by `scale` inside the update kernels of the coming steps."""
        self.layer_optimizer.set_grad_scale(scale)

    def read_grad_stats(self, reset: bool = True) -> dict:
        """Global gradient statistics of the step(s) since the last reset: {"sumsq", "norm",
        "nonfinite"}.  Under `shared_dp` every rank measured the slices it owns of the MEAN
        gradient; the parts are summed over the ranks here (a collective: call it on every rank)."""
        self.wait_for_completion()
        st = self.layer_optimizer.read_grad_stats(reset)
        if self.shared_dp is not None:
            import torch.distributed as dist
            t = torch.tensor([st["sumsq"], 1.0 if st["nonfinite"] else 0.0], dtype=torch.float64, device=self.device)
            dist.all_reduce(t)
            st = {"sumsq": float(t[0]), "norm": float(t[0]) ** 0.5, "nonfinite": bool(t[1] > 0)}
        return st

    def clip_scale_for_next_step(self, max_norm: float, stats: Optional[dict] = None) -> float:
        """Delayed global-norm clipping: derive the multiplier for the NEXT step from the norm the
        last step measured (a layer-wise optimizer has already applied the first layers' updates
        when the last layer's gradient, and with it the step's own norm, exists)."""
        stats = stats if stats is not None else self.read_grad_stats()
        norm = stats["norm"]      # taken before the multiplier is applied: the raw gradient's norm
        new = 1.0 if (stats["nonfinite"] or norm <= max_norm or norm == 0.0) else max_norm / norm
        self.set_grad_scale(new)
        return new

    def parameter_update_ms(self):
        """Per-unit mean device time of the optimizer step (needs enable_timing)."""
        out = {}
        for u in self.transformer_layers:
            spans = u.timings["parameter_update"]
            if spans:
                out[u.layer_idx] = sum(a.elapsed_time(b) for a, b in spans) / len(spans)
        return out

    def _save_from_slices(self, output_dir):
        """Window mode: every rank takes part in gathering each unit's bf16 slices; rank 0 collects
        the full tensors in host memory and writes them.  Collective: call it on all ranks."""
        dp = self.shared_dp
        names = {id(p): n for n, p in self.base_model.named_parameters()}
        state = {}
        for unit in self.transformer_layers:
            st = unit._dp_state
            if st.shard == 0:
                continue
            full = torch.empty(st.shard * dp.world_size, dtype=self.dtype, device=self.device)
            dp.gather_weights(unit.layer_idx, full)
            if dp.rank == 0:
                for local, p in unit._managed_named_params:
                    off, shape, k = unit._param_maps[local]
                    state[names[id(p)]] = full[off:off + k].view(shape).cpu()
            del full
        torch.cuda.synchronize(self.device)
        if dp.rank == 0:
            missing = [n for n, _ in self.base_model.named_parameters() if n not in state]
            if missing:
                raise RuntimeError(f"parameters without a unit: {missing[:5]}")
            for n, b in self.base_model.named_buffers():   # persistent buffers, if a model has any
                if n in self.base_model.state_dict(keep_vars=True) and not b.is_meta:
                    state[n] = b.detach().cpu()
            self.base_model.save_pretrained(output_dir, state_dict=state)
        dp.barrier()
        return output_dir

    def layer_timings_ms(self, show_history: bool = False):
        """{operation: [ms per unit]} from the recorded CUDA-event spans (needs enable_timing): the
        most recent step's span of every unit, or with show_history each unit's mean over all steps.
        Activation-copy spans come from the activation store when activations go to host memory."""
        torch.cuda.synchronize(self.device)
        out = {}
        for u in self.transformer_layers:
            for op, spans in u.timings.items():
                if spans:
                    used = spans if show_history else spans[-1:]
                    out.setdefault(op, []).append((u.layer_idx, sum(a.elapsed_time(b) for a, b in used) / len(used), len(used)))
        store = self.activation_store
        if store is not None:
            for op, spans in (("ac_fwd_d2h", store.spans_d2h), ("ac_bwd_h2d", store.spans_h2d)):
                done = [(a, b) for a, b in spans if b.query()]
                if done:
                    used = done if show_history else done[-len(self.decoder_layers):]
                    out[op] = [(None, sum(a.elapsed_time(b) for a, b in used) / len(used), len(used))]
        return out

    def print_layer_stats(self, layer_idx=None, show_history: bool = False):
        """Per-unit device times under the reference's labels (offload_transformer.py:337-377,
        utils/timer.py:11-21): forward, backward, parameter update, the weight-window fill as
        "h2d transfer fw / bw", and the activation copies as "ac fwd d2h" / "ac bwd h2d".
        show_history averages over all recorded steps, otherwise the most recent step is shown."""
        if not self.enable_timing:
            return
        from .transformer_layer import format_timing_label
        stats = self.layer_timings_ms(show_history)
        if not stats:
            return
        if layer_idx is not None:
            print(f"\nLayer {layer_idx} Statistics:")
            for op, rows in stats.items():
                for idx, ms, calls in rows:
                    if idx == layer_idx:
                        print(f"  {format_timing_label(op)}: {ms:.2f}ms ({calls} calls)")
            return
        print("\nHistorical Average Layer Statistics:" if show_history else "\nCurrent Step Layer Statistics:")
        for op, rows in stats.items():
            mean = sum(r[1] for r in rows) / len(rows)
            if show_history:
                print(f"  {format_timing_label(op)}: {mean:.2f}ms (avg over {sum(r[2] for r in rows)} calls)")
            else:
                print(f"  {format_timing_label(op)}: {mean:.2f}ms (avg across {len(rows)} layers)")

    def save_pretrained(self, output_dir):
        """Write HF-format weights cast to the compute dtype (offload_transformer.py:593-597).  The
        live parameters already are the bf16 weights, so the model saves itself.

        With `shared_dp` this is COLLECTIVE, like the reference's data-parallel engine
        (multi_gpu/offload_transformer.py:581-590): every rank calls it, the ranks meet at a
        barrier, rank 0 alone serialises (every rank holds the full bf16 weights; in window mode
        the slices are all-gathered first, which needs every rank), and a second barrier releases
        them."""
        self.wait_for_completion()
        if self.weight_window and self.shared_dp is None:
            # one-GPU window: the weights live in each unit's pinned host store
            names = {id(p): n for n, p in self.base_model.named_parameters()}
            state = {}
            for unit in self.transformer_layers:
                flat = unit.bf16_weights_flat()
                for local, p in unit._managed_named_params:
                    off, shape, k = unit._param_maps[local]
                    state[names[id(p)]] = flat[off:off + k].view(shape).clone()
            self.base_model.save_pretrained(output_dir, state_dict=state)
            return output_dir
        if self.weight_window:
            self.shared_dp.barrier()
            return self._save_from_slices(output_dir)
        if self.shared_dp is not None:
            self.shared_dp.barrier()
            if self.shared_dp.rank != 0:
                self.shared_dp.barrier()
                return output_dir
        # every parameter is a view into its unit's flat buffer; hand the serializer independent copies
        state, seen = {}, {}
        for name, value in self.base_model.state_dict(keep_vars=True).items():
            if id(value) not in seen:
                seen[id(value)] = value.detach().clone()
            state[name] = seen[id(value)]
        self.base_model.save_pretrained(output_dir, state_dict=state)
        if self.shared_dp is not None:
            self.shared_dp.barrier()
        return output_dir
