"""ctypes binding of libloopback_b200.so (the C ABI declared in include/loopback_b200.h).

There is no fallback of any kind: if the library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LOOPBACK_B200_LIB overrides the library file (for trying an experimental build without touching the package)
LIB_PATH = os.environ.get("LOOPBACK_B200_LIB") or os.path.join(_HERE, "libloopback_b200.so")

LB_DTYPE_F32 = 0
LB_DTYPE_BF16 = 1
LB_MAX_SOURCES = 128
LB_MAX_PEERS = 16

# every symbol include/loopback_b200.h declares: (name, restype, argtypes)
_vp, _i, _i64, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
SYMBOLS = {
    "lb_version": (_i, []),
    "lb_last_error_string": (ctypes.c_char_p, []),
    "lb_device_error": (_i, [_i]),
    "lb_set_option": (_i, [ctypes.c_char_p, _i]),
    "lb_write": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _f, _i, _vp]),
    "lb_write_bwd_dx": (_i, [_vp, _vp, _i64, _i, _vp]),
    "lb_rstd_fwd": (_i, [_vp, _vp, _i64, _i, _f, _i, _vp]),
    "lb_rstd_bwd": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _vp]),
    "lb_rstd_bwd_acc": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _i, _vp]),
    "lb_scores": (_i, [_vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp]),
    "lb_read_fwd": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp]),
    "lb_step_fwd": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _f, _i,
                         _vp]),
    "lb_read_bwd_scratch_bytes": (ctypes.c_size_t, [_i]),
    "lb_read_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i,
                         _i, _i, _vp]),
    "lb_read_bwd_final": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i,
                               _i, _i, _i, _vp]),
    "lb_combine_fwd": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _f, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i,
                            _vp]),
    "lb_combine_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64,
                            _i, _i, _i, _i, _i, _vp]),
    "lb_step_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                         _f, _i64, _i, _i, _i, _i, _i, _vp]),
    "lb_permuted_query_row_floats": (ctypes.c_size_t, [_i, _i]),
    "lb_permute_queries": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "lb_step_bwd_deferred": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                  _vp, _vp, _i, _i, _f, _vp, _vp, _i64, _i, _i, _i, _i, _i, _vp]),
    "lb_peer_flag_words": (_i, []),
    "lb_peer_allreduce": (_i, [_vp, _vp, _i, _i, _vp, _i64, _vp]),
    "lb_read_bwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i,
                                 _i, _i, _vp]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (python -m loopback_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA kernels of loopback_b200 are not built "
                "(run `python -m loopback_b200.build`); there is no fallback path")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)       # AttributeError if the library does not export the symbol
            fn.restype = res
            fn.argtypes = args
        if handle.lb_version() != 1:
            raise RuntimeError(f"{LIB_PATH}: unexpected ABI version {handle.lb_version()}")
        _lib = handle
    return _lib


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return LB_DTYPE_BF16
    if dtype == torch.float32:
        return LB_DTYPE_F32
    raise RuntimeError(f"loopback_b200 stores activations as bfloat16 or float32, got {dtype}")


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# kernels launched through this binding since import (lb_read_bwd launches two: the backward and the reduction
# of its query-gradient partials); read by the benchmark
LAUNCHES = {"count": 0}
_KERNELS_PER_CALL = {"read backward": 2, "read backward (final)": 2, "combine backward": 2, "step backward": 2,
                     "step backward (deferred)": 2}


def check(rc: int, what: str) -> None:
    LAUNCHES["count"] += _KERNELS_PER_CALL.get(what, 1)
    if rc != 0:
        msg = lib().lb_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"loopback_b200 {what} failed (status {rc}): {msg}")


def device_error(clear: bool = True) -> int:
    """Synchronises and returns the device error word (0 = every kernel wait completed)."""
    return int(lib().lb_device_error(int(clear)))


def set_option(name: str, value: int) -> None:
    check(lib().lb_set_option(name.encode(), int(value)), f"set_option({name})")


def reset_options() -> None:
    """Every tuning knob back to its default (the choice by size)."""
    check(lib().lb_set_option(b"reset_all", 0), "set_option(reset_all)")
