"""ctypes binding of libmegafold_b200.so (C ABI declared in include/megafold_b200.h).

The structures below mirror the C structs field for field.  There is no CPU fallback: if the
library cannot be loaded, or an entry point returns an error, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmegafold_b200_trace.so" if os.environ.get("MF_TRACE") == "1" else "libmegafold_b200.so")

MF_F32, MF_BF16, MF_F16, MF_U8 = 0, 1, 2, 3
MF_FLAG_FORCE_SIMT = 1

_DTYPES = {torch.float32: MF_F32, torch.bfloat16: MF_BF16, torch.float16: MF_F16,
           torch.bool: MF_U8, torch.uint8: MF_U8}

_i32, _u32, _i64, _vp, _f32, _sz = C.c_int32, C.c_uint32, C.c_int64, C.c_void_p, C.c_float, C.c_size_t


class EvoFwdArgs(C.Structure):
    _fields_ = [("B", _i32), ("N", _i32), ("L", _i32), ("H", _i32), ("D", _i32),
                ("dtype", _i32), ("bias_dtype", _i32), ("mask_dtype", _i32), ("flags", _u32),
                ("q", _vp), ("k", _vp), ("v", _vp),
                ("q_strides", _i64 * 5), ("k_strides", _i64 * 5), ("v_strides", _i64 * 5),
                ("mask", _vp), ("mask_strides", _i64 * 3),
                ("bias", _vp), ("bias_strides", _i64 * 4),
                ("o", _vp), ("lse", _vp)]


class EvoBwdArgs(C.Structure):
    _fields_ = [("B", _i32), ("N", _i32), ("L", _i32), ("H", _i32), ("D", _i32),
                ("dtype", _i32), ("bias_dtype", _i32), ("mask_dtype", _i32), ("dbias_dtype", _i32), ("flags", _u32),
                ("q", _vp), ("k", _vp), ("v", _vp),
                ("q_strides", _i64 * 5), ("k_strides", _i64 * 5), ("v_strides", _i64 * 5),
                ("mask", _vp), ("mask_strides", _i64 * 3),
                ("bias", _vp), ("bias_strides", _i64 * 4),
                ("o", _vp), ("d_o", _vp), ("lse", _vp),
                ("dq", _vp), ("dk", _vp), ("dv", _vp), ("d_bias", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz),
                ("dbias_ready_event", _vp)]


class LnlFwdArgs(C.Structure):
    _fields_ = [("M", _i64), ("K", _i32), ("N", _i32), ("dtype", _i32), ("flags", _u32), ("eps", _f32),
                ("x", _vp), ("ln_w", _vp), ("ln_b", _vp), ("w", _vp), ("b", _vp),
                ("y", _vp), ("mean", _vp), ("rstd", _vp)]


class LnlBwdArgs(C.Structure):
    _fields_ = [("M", _i64), ("K", _i32), ("N", _i32), ("dtype", _i32), ("flags", _u32),
                ("x", _vp), ("ln_w", _vp), ("ln_b", _vp), ("w", _vp), ("dy", _vp),
                ("mean", _vp), ("rstd", _vp),
                ("dx", _vp), ("dw", _vp), ("db", _vp), ("d_ln_w", _vp), ("d_ln_b", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz)]


class TransitionFwdArgs(C.Structure):
    _fields_ = [("M", _i64), ("dim", _i32), ("inner", _i32), ("dtype", _i32), ("flags", _u32), ("eps", _f32),
                ("x", _vp), ("ln_w", _vp), ("ln_b", _vp), ("w1", _vp), ("w2", _vp),
                ("y", _vp), ("mean", _vp), ("rstd", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz)]


class TransitionBwdArgs(C.Structure):
    _fields_ = [("M", _i64), ("dim", _i32), ("inner", _i32), ("dtype", _i32), ("flags", _u32),
                ("x", _vp), ("ln_w", _vp), ("ln_b", _vp), ("w1", _vp), ("w2", _vp), ("dy", _vp),
                ("mean", _vp), ("rstd", _vp),
                ("dx", _vp), ("dw1", _vp), ("dw2", _vp), ("d_ln_w", _vp), ("d_ln_b", _vp),
                ("workspace", _vp), ("workspace_bytes", _sz)]


# every symbol include/megafold_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "mf_evo_fwd": (C.c_int, [C.POINTER(EvoFwdArgs), _vp]),
    "mf_evo_bwd_workspace_bytes": (_sz, [C.POINTER(EvoBwdArgs)]),
    "mf_evo_bwd": (C.c_int, [C.POINTER(EvoBwdArgs), _vp]),
    "mf_evo_bwd_noalloc": (C.c_int, [C.POINTER(EvoBwdArgs), _vp]),
    "mf_evo_bwd_noalloc_max_rows": (_sz, []),
    "mf_lnl_fwd": (C.c_int, [C.POINTER(LnlFwdArgs), _vp]),
    "mf_lnl_bwd_workspace_bytes": (_sz, [C.POINTER(LnlBwdArgs)]),
    "mf_lnl_bwd": (C.c_int, [C.POINTER(LnlBwdArgs), _vp]),
    "mf_swiglu_fwd": (C.c_int, [_vp, _vp, _i64, _i32, _i32, _vp]),
    "mf_swiglu_bwd": (C.c_int, [_vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "mf_transition_fwd_workspace_bytes": (_sz, [C.POINTER(TransitionFwdArgs)]),
    "mf_transition_fwd": (C.c_int, [C.POINTER(TransitionFwdArgs), _vp]),
    "mf_transition_bwd_workspace_bytes": (_sz, [C.POINTER(TransitionBwdArgs)]),
    "mf_transition_bwd": (C.c_int, [C.POINTER(TransitionBwdArgs), _vp]),
    "mf_last_error_string": (C.c_char_p, []),
    "mf_version": (C.c_int, []),
    "mf_kernel_launch_count": (C.c_uint64, []),
    "mf_last_path": (C.c_char_p, []),
    "mf_async_status": (C.c_int, []),
    "mf_selftest_bounded_wait": (C.c_int, [_vp]),
}

_lib = None
_lock = threading.Lock()


def lib() -> C.CDLL:
    """The loaded library; built in-tree with nvcc on first use if the .so is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                from . import build as _build
                _build.build()
            handle = C.CDLL(LIB_PATH)
            for name, (res, args) in SYMBOLS.items():
                fn = getattr(handle, name)       # AttributeError if the library lacks a declared symbol
                fn.restype, fn.argtypes = res, args
            _lib = handle
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"megafold_b200: unsupported dtype {dt}") from None


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().mf_last_error_string().decode()
        raise RuntimeError(f"megafold_b200 {what} failed (status {status}): {msg}")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("megafold_b200 operators run on CUDA tensors only (there is no CPU path); "
                               f"got a tensor on {t.device}")


def workspace(nbytes: int, device) -> torch.Tensor:
    """Scratch from the torch caching allocator (256-byte aligned by the allocator's own granularity)."""
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def launch_count() -> int:
    return int(lib().mf_kernel_launch_count())


def last_path() -> str:
    return lib().mf_last_path().decode()
