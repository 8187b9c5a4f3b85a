"""ctypes binding of libslideformer_b200.so (the C ABI in include/slideformer_b200.h).

There is no Python or CPU implementation behind these calls.  If the shared library is
missing it is built in-tree with nvcc; if that is impossible the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libslideformer_b200.so"

SF_OK = 0
SF_ERR_NULL, SF_ERR_ALIGN, SF_ERR_SIZE, SF_ERR_UNKNOWN_ID, SF_ERR_CUDA, SF_ERR_DTYPE, SF_ERR_ARG = range(1, 8)
SF_GRAD_BF16, SF_GRAD_F32, SF_GRAD_F16 = 0, 1, 2
SF_IPC_HANDLE_BYTES = 64
SF_ABI_VERSION = 2
SF_STATIC_SCRATCH_MAX_ELEMS = 4 << 20  # sf_adam_update_dp_static: largest n per call


SF_STATS_LANES = 32


class SfGradStats(C.Structure):
    """Device-resident block the kernels accumulate gradient statistics into (256 bytes)."""
    _fields_ = [("sumsq", C.c_float * SF_STATS_LANES), ("nonfinite", C.c_uint32), ("reserved", C.c_uint32 * 31)]


class SfAdamScalars(C.Structure):
    _fields_ = [("beta1", C.c_float), ("beta2", C.c_float), ("omb1", C.c_float), ("omb2", C.c_float),
                ("bc2", C.c_float), ("eps", C.c_float), ("step_size", C.c_float),
                ("w_decay", C.c_float), ("weight_decay", C.c_float), ("adamw_mode", C.c_int32),
                ("grad_scale", C.c_float), ("grad_stats", C.c_void_p)]

    def as_tuple(self):
        return tuple(getattr(self, k) for k, _ in self._fields_)


SF_MAX_SEGMENTS = 32


class SfPushSegment(C.Structure):
    _fields_ = [("s", SfAdamScalars), ("p", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("peer_g", C.POINTER(C.c_void_p)), ("peer_out", C.POINTER(C.c_void_p)),
                ("n", C.c_uint64), ("vec_n", C.c_uint64)]


class SfError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"slideformer_b200 error {code}: {message}")
        self.code = code


# name -> (restype, argtypes); every symbol the header declares appears here.
_f, _u64, _vp, _i = C.c_float, C.c_uint64, C.c_void_p, C.c_int
SIGNATURES = {
    "sf_adam_create": (_i, [_i, _f, _f, _f, _f, _f, _i, _i]),
    "sf_adam_destroy": (_i, [_i]),
    "sf_adam_set_grad_hooks": (_i, [_i, _f, _vp]),
    "sf_adam_scalars": (_i, [_i, _u64, _f, _f, _f, _f, _f, _i, C.POINTER(SfAdamScalars)]),
    "sf_adam_update": (_i, [_i, _u64, _f, _f, _f, _f, _f, _i, _vp, _vp, _i, _vp, _vp, _vp, _u64, _vp]),
    "sf_adam_step": (_i, [C.POINTER(SfAdamScalars), _vp, _vp, _i, _vp, _vp, _vp, _u64, _u64, _vp]),
    "sf_adam_step_sharded": (_i, [C.POINTER(SfAdamScalars), _vp, C.POINTER(_vp), _i, _i, _vp, _vp, _vp,
                                  _u64, _u64, _vp]),
    "sf_adam_step_sharded_push": (_i, [C.POINTER(SfAdamScalars), _vp, C.POINTER(_vp), C.POINTER(_vp), _i, _i, _vp, _vp,
                                       _u64, _u64, _vp]),
    "sf_adam_step_sharded_push_multi": (_i, [C.POINTER(SfPushSegment), _i, _i, _i, _vp]),
    "sf_adam_step_sharded_nvls": (_i, [C.POINTER(SfAdamScalars), _vp, _vp, _vp, C.POINTER(_vp), C.POINTER(_vp), _i, _vp, _vp,
                                       _u64, _u64, _vp]),
    "sf_dp_mean": (_i, [C.POINTER(_vp), _i, _i, _vp, _u64, _vp]),
    "sf_adam_update_dp_static": (_i, [_i, _u64, _f, _f, _f, _f, _f, _i, _vp, C.POINTER(_vp), _i, _i, _vp, _vp, _vp,
                                      _u64, _vp]),
    "sf_adam_host_scratch_bytes": (C.c_size_t, [_u64, _i, _i]),
    "sf_adam_update_host": (_i, [_i, _u64, _f, _f, _f, _f, _f, _i, _vp, _vp, _i, _i, _vp, _vp, _vp, _u64,
                                 _u64, _i, _vp, C.c_size_t, _vp]),
    "sf_last_error": (C.c_char_p, []),
    "sf_abi_version": (_i, []),
    "sf_launch_count": (_u64, []),
    "sf_set_tuning": (_i, [_i, _i]),
    "sf_set_push_tuning": (_i, [_i, _i]),
    "sf_set_nvls_tuning": (_i, [_i]),
    "sf_set_host_piece": (_i, [_u64]),
    "sf_copy_bytes": (_i, [_vp, _vp, C.c_size_t, _vp]),
    "sf_dev_alloc": (_i, [C.c_size_t, C.POINTER(_vp)]),
    "sf_dev_free": (_i, [_vp]),
    "sf_ipc_export": (_i, [_vp, _vp]),
    "sf_ipc_open": (_i, [_vp, C.POINTER(_vp)]),
    "sf_ipc_close": (_i, [_vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load (building first if needed) the native library and bind every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        from . import build as _build
        try:
            _build.build()
        except Exception as exc:  # no nvcc, or the compile failed
            raise ImportError(
                f"{LIB_PATH.name} is missing and could not be built ({exc}). "
                "Run `python -m slideformer_b200.build` where nvcc is available; "
                "there is no fallback implementation.") from exc
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    if lib.sf_abi_version() != SF_ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.sf_abi_version()}, expected {SF_ABI_VERSION}; rebuild it")
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != SF_OK:
        raise SfError(code, load().sf_last_error().decode("utf-8", "replace"))
