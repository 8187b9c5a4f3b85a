"""LayerAdam: one optimizer object for all layers, stepped one layer at a time, on the GPU.

Mirror of the reference front end (optimizer/layer_adam/layer_adam.py:12-484): same
constructor keywords, same methods (`add_layer_params`, `step`, `step_with_grad_views`,
`begin_chunk_step` / `step_chunk` / `end_chunk_step`, `update_learning_rate`) and the same
public attributes (`defaults`, `param_groups`, `state`, `exp_avg_flat`, `exp_avg_sq_flat`,
`fp32_optimizer_state`, `nvme_offload_fraction`).  What changes is where the arithmetic
runs: every update is one launch of the fused sm_100a kernel through the C ABI
(`sf_adam_update`), the fp32 master weights and the Adam moments stay resident in HBM, and
the kernel can also emit the bf16 copy of the new weights that the reference produces later
with a separate CPU cast (transformer_layer.py:296-305).

Placement rules
  * parameter on a CUDA device  -> moments are allocated on that device, HBM-resident step;
  * parameter in PINNED host memory -> moments are pinned too and the step streams chunks
    through the GPU (`sf_adam_update_host`);
  * parameter in pageable host memory -> RuntimeError.  There is no CPU arithmetic here.

Each call to the C ABI on device tensors corresponds to exactly one `adam_update` call of the
reference, so the host scalar state machine (running beta^t product vs pow(), cpu_adam.h:57-76)
sees the same call history and the results stay bit-identical to the reference kernel.  A call
on host-resident tensors is one reference call too, unless `step_chunk(..., host_chunk_calls=True)`
asks for one reference call per streamed chunk (the reference engine's history).
"""
from __future__ import annotations

import itertools
from collections import OrderedDict, defaultdict
from typing import Any, DefaultDict, Dict, Iterable, Optional

import torch

from . import _lib

_ids = itertools.count()
DEFAULT_STREAM_CHUNK = 32 * 1024 * 1024  # elements; the reference's H2D/D2H chunk, transformer_layer.py:26-27


def _grad_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.SF_GRAD_BF16
    if t.dtype == torch.float32:
        return _lib.SF_GRAD_F32
    if t.dtype == torch.float16:
        return _lib.SF_GRAD_F16
    # the reference raises std::runtime_error -> RuntimeError for an unregistered dtype triple
    raise RuntimeError(f"Adam optimizer with param type Float, grads type {t.dtype} and state type Float "
                       "is not supported on current hardware")


def _check_flat(name: str, t: torch.Tensor, dtype=None):
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")  # TORCH_CHECK of cpu_adam_impl.cpp:234-237
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")


class LayerAdam:
    """Layer-wise Adam / AdamW whose element loop is the fused B200 kernel."""

    def __init__(self, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=0,
                 adamw_mode=True, fp32_optimizer_state=True, num_layer: int = 0,
                 nvme_offload_fraction: float = 0.0, offload_dir: str = "/NVME1", prefetch: bool = True,
                 *, stream_chunk_numel: int = DEFAULT_STREAM_CHUNK, should_log: bool = False):
        self.defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                             weight_decay=weight_decay, adamw_mode=adamw_mode)
        self.param_groups = []
        self._lib = _lib.load()
        # The reference always uses id 0 (layer_adam.py:62), so two of its LayerAdam objects
        # share one scalar block and the first __del__ breaks the other.  Ids are unique here.
        self.optimizer_id = next(_ids)
        _lib.check(self._lib.sf_adam_create(self.optimizer_id, lr, betas[0], betas[1], eps, weight_decay,
                                            int(bool(adamw_mode)), int(bool(should_log))))
        # The reference allocates the moments in fp32, or with fp32_optimizer_state=False in the
        # parameters' dtype (layer_adam.py:161).  Master parameters are fp32 here (add_layer_params
        # refuses anything else), so both settings give fp32 moments.
        self.fp32_optimizer_state = fp32_optimizer_state
        self.num_layer = num_layer
        self.state: DefaultDict[torch.Tensor, Any] = defaultdict(dict)
        assert 0.0 <= nvme_offload_fraction <= 1.0
        if nvme_offload_fraction > 0.0:
            raise NotImplementedError("NVMe spill of the Adam moments is not part of this build; "
                                      "keep them in HBM or in pinned host memory")
        self.nvme_offload_fraction = nvme_offload_fraction
        self.prefetch = prefetch
        self.pin_memory = False
        self.offload_dir = None
        self.offloader = None
        self.exp_avg_flat = OrderedDict()
        self.exp_avg_sq_flat = OrderedDict()
        self.bf16_flat: Dict[int, Optional[torch.Tensor]] = {}
        self.stream_chunk_numel = int(stream_chunk_numel)
        self._scratch: Dict[Any, torch.Tensor] = {}
        self.grad_scale = 1.0
        self._grad_stats: Optional[torch.Tensor] = None

    def __del__(self):
        lib = getattr(self, "_lib", None)
        if lib is not None and hasattr(self, "optimizer_id"):
            try:
                lib.sf_adam_destroy(self.optimizer_id)
            except Exception:
                pass

    # ---- registration ---------------------------------------------------------------------
    def _get_layer_numel(self, layer_idx: int) -> int:
        return sum(p.numel() for p in self.param_groups[layer_idx]["params"])

    def add_layer_params(self, layer_idx: int, params: Iterable[torch.nn.Parameter],
                         bf16_params: Optional[Iterable[torch.Tensor]] = None) -> int:
        """Register a layer (layer_adam.py:134-198).  Layers must be added in index order.

        bf16_params (an addition): one bf16 tensor per parameter, same numel, that receives the
        rounded copy of the updated weights in the same kernel launch.
        """
        params = list(params)
        bf16_params = list(bf16_params) if bf16_params is not None else None
        if not params:
            return -1
        for p in params:
            if p.dtype != torch.float32:
                raise RuntimeError(f"master parameters must be float32, got {p.dtype}")
        param_group = {"params": params, "layer_idx": layer_idx, "step": 0, **self.defaults}
        self.param_groups.append(param_group)
        layer_numel = sum(p.numel() for p in params)
        dev = params[0].device
        if dev.type == "cuda":
            kw = dict(device=dev)
        elif dev.type == "cpu":
            if not all(p.is_pinned() for p in params):
                raise RuntimeError("host-resident parameters must be in pinned memory; there is no CPU update path")
            kw = None
        else:
            raise RuntimeError(f"unsupported device type: {dev.type}")
        if kw is not None:
            self.exp_avg_flat[layer_idx] = torch.zeros(layer_numel, dtype=torch.float32, **kw)
            self.exp_avg_sq_flat[layer_idx] = torch.zeros(layer_numel, dtype=torch.float32, **kw)
        else:
            # pinned moments next to the GPU that will stream them (the device of the bf16 outputs,
            # else the current device)
            from .numa import pinned_empty
            near = next((b.device for b in (bf16_params or []) if b is not None), None) if bf16_params is not None else None
            near = near if near is not None else (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
            self.exp_avg_flat[layer_idx] = pinned_empty(layer_numel, torch.float32, near).zero_()
            self.exp_avg_sq_flat[layer_idx] = pinned_empty(layer_numel, torch.float32, near).zero_()
        bf16_list = list(bf16_params) if bf16_params is not None else [None] * len(params)
        if len(bf16_list) != len(params):
            raise ValueError("bf16_params must have one entry per parameter")
        offset = 0
        for p, b in zip(params, bf16_list):
            size = p.numel()
            st = self.state[p]
            st["exp_avg"] = self.exp_avg_flat[layer_idx][offset:offset + size].view(p.shape)
            st["exp_avg_sq"] = self.exp_avg_sq_flat[layer_idx][offset:offset + size].view(p.shape)
            if b is not None:
                if b.dtype != torch.bfloat16 or b.numel() != size or b.device.type != "cuda":
                    raise ValueError("each bf16 output must be a CUDA bfloat16 tensor with the parameter's numel")
                st["bf16"] = b
            offset += size
        return layer_idx

    # ---- the one place that calls the C ABI ---------------------------------------------------
    def _adam_update(self, step, lr, beta1, beta2, eps, weight_decay, bias_correction,
                     p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                     bf16: Optional[torch.Tensor] = None, host_chunk_calls: bool = False,
                     host_chunk_numel: Optional[int] = None):
        _check_flat("params", p, torch.float32)
        _check_flat("grads", g)
        _check_flat("exp_avg", m, torch.float32)
        _check_flat("exp_avg_sq", v, torch.float32)
        gcode = _grad_code(g)
        n = p.numel()
        if not (g.numel() == n and m.numel() == n and v.numel() == n):
            raise RuntimeError("params, grads, exp_avg and exp_avg_sq must have the same number of elements")
        if bf16 is not None:
            _check_flat("bf16 output", bf16, torch.bfloat16)
            if bf16.numel() != n or bf16.device.type != "cuda":
                raise RuntimeError("bf16 output must be a CUDA tensor with the parameter's numel")
        if p.device.type == "cuda":
            if not (g.device == p.device and m.device == p.device and v.device == p.device):
                raise RuntimeError("params, grads and moments must be on the same CUDA device")
            if bf16 is not None and bf16.device != p.device:
                raise RuntimeError("bf16 output must be on the parameter's device")
            args = (self.optimizer_id, int(step), lr, beta1, beta2, eps, weight_decay, int(bias_correction == 1),
                    p.data_ptr(), g.data_ptr(), gcode, m.data_ptr(), v.data_ptr(),
                    bf16.data_ptr() if bf16 is not None else None, n)
            if p.device.index == torch.cuda.current_device():   # the usual case: no device switch to pay for
                rc = self._lib.sf_adam_update(*args, torch.cuda.current_stream().cuda_stream)
            else:
                with torch.cuda.device(p.device):
                    rc = self._lib.sf_adam_update(*args, torch.cuda.current_stream().cuda_stream)
            if rc:
                _lib.check(rc)
            return
        if p.device.type != "cpu":
            raise RuntimeError(f"unsupported device type: {p.device.type}")
        # host-resident state: stream through the GPU
        if not (p.is_pinned() and m.is_pinned() and v.is_pinned()):
            raise RuntimeError("host-resident params and moments must be pinned; there is no CPU update path")
        g_on_host = g.device.type == "cpu"
        if g_on_host and not g.is_pinned():
            raise RuntimeError("a host-resident gradient must be pinned")
        dev = bf16.device if bf16 is not None else (g.device if not g_on_host else torch.device("cuda", torch.cuda.current_device()))
        chunk = max(16, min(int(host_chunk_numel or self.stream_chunk_numel), (n + 15) // 16 * 16)) // 16 * 16
        with torch.cuda.device(dev):
            need = self._lib.sf_adam_host_scratch_bytes(chunk, gcode, int(g_on_host))
            key = (dev.index, need)
            scratch = self._scratch.get(key)
            if scratch is None:
                scratch = torch.empty(need, dtype=torch.uint8, device=dev)
                self._scratch = {key: scratch}  # keep only the newest size
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(self._lib.sf_adam_update_host(
                self.optimizer_id, int(step), lr, beta1, beta2, eps, weight_decay, int(bias_correction == 1),
                p.data_ptr(), g.data_ptr(), gcode, int(g_on_host), m.data_ptr(), v.data_ptr(),
                bf16.data_ptr() if bf16 is not None else None, n, chunk, int(bool(host_chunk_calls)),
                scratch.data_ptr(), need, stream))

    # ---- whole-layer steps (layer_adam.py:271-428) ----------------------------------------------
    def _groups(self, layer_idx):
        return [self.param_groups[layer_idx]] if layer_idx is not None else self.param_groups

    @torch.no_grad()
    def step(self, layer_idx: int = None, closure=None):
        """Update one layer (or all) from `p.grad`; one kernel launch per parameter."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self._groups(layer_idx):
            beta1, beta2 = group["betas"]
            group["step"] += 1
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                assert p.data.numel() == p.grad.data.numel()
                self._adam_update(group["step"], group["lr"], beta1, beta2, group["eps"], group["weight_decay"],
                                  group["bias_correction"], p.data.view(-1), p.grad.data.view(-1),
                                  st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                                  st["bf16"].view(-1) if "bf16" in st else None)
        return loss

    @torch.no_grad()
    def step_with_grad_views(self, layer_idx: int = None, grad_views: Dict[torch.nn.Parameter, torch.Tensor] = None,
                             closure=None):
        """Like `step`, with gradients supplied as {parameter: tensor} (layer_adam.py:362-428)."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self._groups(layer_idx):
            beta1, beta2 = group["betas"]
            group["step"] += 1
            for p in group["params"]:
                grad = grad_views.get(p) if grad_views else None
                if grad is None:
                    print(f"Warning: no gradient view for a parameter of shape {tuple(p.shape)}; skipped")
                    continue
                st = self.state[p]
                assert p.data.numel() == grad.numel()
                self._adam_update(group["step"], group["lr"], beta1, beta2, group["eps"], group["weight_decay"],
                                  group["bias_correction"], p.data.view(-1), grad.view(-1),
                                  st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                                  st["bf16"].view(-1) if "bf16" in st else None)
        return loss

    # ---- chunk API (layer_adam.py:431-468) ---------------------------------------------------
    @torch.no_grad()
    def begin_chunk_step(self, layer_idx: int):
        group = self.param_groups[layer_idx]
        group["step"] += 1
        return group

    @torch.no_grad()
    def step_chunk(self, param_flat, grad_flat, exp_avg_flat, exp_avg_sq_flat, param_group, bf16_flat=None,
                   host_chunk_calls: bool = False, host_chunk_numel: Optional[int] = None):
        """One update on caller-sliced flat tensors; `param_group` may be a plain dict with
        step, lr, betas, eps, weight_decay, bias_correction.  bf16_flat (an addition) receives
        the rounded copy of the updated slice.

        For HOST-resident tensors the library cuts the range into chunks of `host_chunk_numel`
        (default: the optimizer's stream_chunk_numel) and streams them through the GPU.  By
        default that is ONE reference adam_update over the whole range (the scalar state machine
        advances once).  host_chunk_calls=True makes it one reference call PER CHUNK, which is
        what the reference engine does with its 32 Mi-element chunks
        (transformer_layer.py:453-499): from the second chunk on beta^t comes from pow() instead
        of the running product, which can differ in the last bit."""
        self._adam_update(param_group["step"], param_group["lr"], param_group["betas"][0], param_group["betas"][1],
                          param_group["eps"], param_group["weight_decay"], param_group["bias_correction"],
                          param_flat, grad_flat, exp_avg_flat, exp_avg_sq_flat, bf16_flat,
                          host_chunk_calls=host_chunk_calls, host_chunk_numel=host_chunk_numel)

    @torch.no_grad()
    def end_chunk_step(self, layer_idx: int):
        return None

    def update_learning_rate(self, new_lr):
        self.defaults["lr"] = new_lr
        for group in self.param_groups:
            group["lr"] = new_lr

    # ---- gradient-side work folded into the same pass (no counterpart in the reference's kernel) ----
    def set_grad_scale(self, scale: float):
        """Multiply every incoming gradient by `scale` (one rounded fp32 product per element) inside
        the update kernel: a clip factor derived from the norm the previous step measured, or the
        inverse of a loss scale.  1.0 restores the reference's element loop bit for bit."""
        self.grad_scale = float(scale)
        self._push_grad_hooks()

    def enable_grad_stats(self, device=None):
        """Have every update launch add sum(g*g) and a non-finite flag of the gradients it consumed
        (before `grad_scale`) to a 256-byte block on `device`; read it with `read_grad_stats()`.
        The reference's scripts get the equivalent signal from separate passes
        (isfinite(loss), multi_gpu/scripts/main_dp.py:102-105)."""
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._grad_stats = torch.zeros(64, dtype=torch.float32, device=dev)
        self._push_grad_hooks()
        return self._grad_stats

    def disable_grad_stats(self):
        self._grad_stats = None
        self._push_grad_hooks()

    def read_grad_stats(self, reset: bool = True) -> dict:
        """Synchronises with the device.  Returns sum of squares, its square root and the non-finite
        flag over every gradient element consumed since the last reset (this rank's slices only,
        when the state is sharded)."""
        if getattr(self, "_grad_stats", None) is None:
            raise RuntimeError("call enable_grad_stats() first")
        host = self._grad_stats.cpu()
        if reset:
            self._grad_stats.zero_()
        sumsq = float(host[:_lib.SF_STATS_LANES].double().sum())
        nonfinite = bool(host[_lib.SF_STATS_LANES:_lib.SF_STATS_LANES + 1].view(torch.int32).item() != 0)
        return {"sumsq": sumsq, "norm": sumsq ** 0.5, "nonfinite": nonfinite}

    def _push_grad_hooks(self):
        stats = getattr(self, "_grad_stats", None)
        _lib.check(self._lib.sf_adam_set_grad_hooks(self.optimizer_id, getattr(self, "grad_scale", 1.0),
                                                    stats.data_ptr() if stats is not None else None))
