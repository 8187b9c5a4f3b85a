"""numpy front end of the C restatement in layer_adam_oracle.c.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module; the
shipped package never does.  bf16 values travel as uint16 bit patterns.

`OracleAdam` mirrors the reference's process-global Adam_Optimizer object
(optimizer/layer_adam/csrc/cpu_adam.h:24-106) and `adam_update` mirrors ds_adam_step
(optimizer/layer_adam/csrc/cpu_adam_impl.cpp:220-270): advance the scalar state machine,
then run the element loop.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None


class _Adam(C.Structure):
    _fields_ = [("alpha", C.c_float), ("betta1", C.c_float), ("betta2", C.c_float),
                ("eps", C.c_float), ("weight_decay", C.c_float),
                ("betta1_t", C.c_float), ("betta2_t", C.c_float),
                ("step", C.c_uint64),
                ("bias_correction1", C.c_float), ("bias_correction2", C.c_float),
                ("adamw_mode", C.c_int)]


class Consts(C.Structure):
    _fields_ = [("betta1", C.c_float), ("betta2", C.c_float), ("omb1", C.c_float),
                ("omb2", C.c_float), ("bc2", C.c_float), ("eps", C.c_float),
                ("step_size", C.c_float), ("w_decay", C.c_float), ("weight_decay", C.c_float),
                ("adamw_mode", C.c_int)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


def build(force: bool = False) -> Path:
    so = HERE / "liblayer_adam_oracle.so"
    src = HERE / "layer_adam_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["make", "-C", str(HERE), "-s"] + (["-B"] if force else []))
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = build()
        L = C.CDLL(str(so))
        assert L.oracle_sizeof_adam() == C.sizeof(_Adam)
        assert L.oracle_sizeof_consts() == C.sizeof(Consts)
        L.oracle_adam_init.argtypes = [C.POINTER(_Adam)] + [C.c_float] * 5 + [C.c_int]
        L.oracle_increment_step.argtypes = [C.POINTER(_Adam), C.c_uint64, C.c_float, C.c_float]
        L.oracle_update_state.argtypes = [C.POINTER(_Adam), C.c_float, C.c_float, C.c_float, C.c_int]
        L.oracle_consts.argtypes = [C.POINTER(_Adam), C.POINTER(Consts)]
        for name in ("oracle_step_f32_bf16", "oracle_step_f32_f32", "oracle_step_f32_f16"):
            getattr(L, name).argtypes = [C.POINTER(Consts), C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
            getattr(L, name).restype = None
        L.oracle_f32_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        for name in ("oracle_mean_bf16", "oracle_mean_f32"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_size_t]
        _LIB = L
    return _LIB


def _ptr(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


class OracleAdam:
    """Scalar block + element loops of one reference optimizer id."""

    def __init__(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, adamw_mode=True):
        self._s = _Adam()
        lib().oracle_adam_init(C.byref(self._s), lr, beta1, beta2, eps, weight_decay, int(adamw_mode))

    def scalars(self, step, lr, beta1, beta2, eps, weight_decay, bias_correction) -> Consts:
        """IncrementStep + update_state + the constants Step_AVX derives (one per adam_update)."""
        L = lib()
        L.oracle_increment_step(C.byref(self._s), int(step), beta1, beta2)
        L.oracle_update_state(C.byref(self._s), lr, eps, weight_decay, int(bool(bias_correction)))
        c = Consts()
        L.oracle_consts(C.byref(self._s), C.byref(c))
        return c

    def adam_update(self, step, lr, beta1, beta2, eps, weight_decay, bias_correction,
                    p: np.ndarray, g: np.ndarray, m: np.ndarray, v: np.ndarray,
                    p_bf16: np.ndarray | None = None, vec_n: int | None = None) -> Consts:
        c = self.scalars(step, lr, beta1, beta2, eps, weight_decay, bias_correction)
        apply_step(c, p, g, m, v, p_bf16, vec_n)
        return c


def apply_step(c: Consts, p, g, m, v, p_bf16=None, vec_n=None):
    n = p.size
    assert p.dtype == np.float32 and m.dtype == np.float32 and v.dtype == np.float32
    assert g.size == n and m.size == n and v.size == n
    if vec_n is None:
        vec_n = n & ~15
    if g.dtype == np.uint16:
        fn = lib().oracle_step_f32_bf16
    elif g.dtype == np.float32:
        fn = lib().oracle_step_f32_f32
    elif g.dtype == np.float16:
        fn = lib().oracle_step_f32_f16
    else:
        raise TypeError(f"unsupported gradient dtype {g.dtype}")
    if p_bf16 is not None:
        assert p_bf16.dtype == np.uint16 and p_bf16.size == n
    fn(C.byref(c), _ptr(p), _ptr(g), _ptr(m), _ptr(v), _ptr(p_bf16), n, vec_n)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_ptr(x), _ptr(out), x.size)
    return out


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def rank_mean(rows: np.ndarray) -> np.ndarray:
    """fp32 mean over axis 0 in rank order (shared_data_parallel.py:130-133)."""
    rows = np.ascontiguousarray(rows)
    world, n = rows.shape
    out = np.empty(n, dtype=np.float32)
    fn = lib().oracle_mean_bf16 if rows.dtype == np.uint16 else lib().oracle_mean_f32
    fn(_ptr(rows), n, world, _ptr(out), n)
    return out
