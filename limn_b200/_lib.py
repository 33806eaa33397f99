"""ctypes binding of liblimn_b200.so (declared in include/limn_b200.h).

There is no fallback of any kind: if the shared library is missing or fails to load, every
use raises. Build it with `python -m limn_b200.build`.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "liblimn_b200.so"

# dtype codes of enum limn_b200_dtype, by the names limn's DType carries (limn/ops.py:24-27)
DTYPE_CODES = {"float32": 0, "float16": 1, "bfloat16": 2, "float64": 3}
PATH_GENERAL, PATH_TCGEN05, PATH_DECODE = 0, 1, 2
OK, BAD_ARGUMENT, UNSUPPORTED, CUDA_ERROR, DEVICE_TIMEOUT = 0, 1, 2, 3, 4  # enum limn_b200_status

_P = c_void_p
_SHAPE = (c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_double, _P)  # dtype, bh, t_q, t_k, hd, hd_v, causal, scale, stream

# layout, dtype, batch, heads, t_q, t_k, hd, hd_v, causal, scale, stream
_LAYOUT_SHAPE = (c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_double, _P)
LAYOUT_CODES = {"bhtd": 0, "bthd": 1}
# strides, dtype, batch, heads, t_q, t_k, hd, hd_v, causal, scale, stream
_STRIDED_SHAPE = (POINTER(c_longlong), c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_double, _P)
SIGNATURES = {
    "limn_b200_sdpa_fwd": (c_int, (_P, _P, _P, _P, _P, _P) + _SHAPE),
    "limn_b200_sdpa_bwd_q": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P) + _SHAPE),
    "limn_b200_sdpa_bwd_q_fused": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _SHAPE),
    "limn_b200_sdpa_bwd_kv": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _SHAPE),
    "limn_b200_sdpa_bwd_q_static": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _SHAPE),
    "limn_b200_sdpa_delta": (c_int, (_P, _P, _P, c_int, c_longlong, c_int, _P)),
    "limn_b200_sdpa_fwd_layout": (c_int, (_P, _P, _P, _P, _P, _P) + _LAYOUT_SHAPE),
    "limn_b200_sdpa_bwd_q_layout": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P) + _LAYOUT_SHAPE),
    "limn_b200_sdpa_bwd_q_fused_layout": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _LAYOUT_SHAPE),
    "limn_b200_sdpa_bwd_kv_layout": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _LAYOUT_SHAPE),
    "limn_b200_sdpa_fwd_strided": (c_int, (_P, _P, _P, _P, _P, _P) + _STRIDED_SHAPE),
    "limn_b200_sdpa_bwd_q_fused_strided": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _STRIDED_SHAPE),
    "limn_b200_sdpa_bwd_kv_strided": (c_int, (_P, _P, _P, _P, _P, _P, _P, _P, _P) + _STRIDED_SHAPE),
    "limn_b200_sdpa_delta_layout": (c_int, (_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P)),
    "limn_b200_sdpa_path": (c_int, (c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_double)),
    "limn_b200_last_launch_count": (c_int, ()),
    "limn_b200_last_error": (c_char_p, ()),
    "limn_b200_version": (c_int, ()),
    "limn_b200_device_status": (c_int, (POINTER(c_uint),)),
    "limn_b200_wait_probe": (c_int, (c_longlong, _P, _P)),
    "limn_b200_nccl_unique_id": (c_int, (_P,)),
    "limn_b200_nccl_init": (c_int, (c_int, c_int, _P)),
    "limn_b200_nccl_all_gather": (c_int, (_P, _P, c_ulonglong, _P)),
    "limn_b200_nccl_destroy": (c_int, ()),
    "limn_b200_device_count": (c_int, (POINTER(c_int),)),
    "limn_b200_set_device": (c_int, (c_int,)),
    "limn_b200_mem_alloc": (c_int, (POINTER(c_void_p), c_ulonglong)),
    "limn_b200_mem_free": (c_int, (_P,)),
    "limn_b200_mem_set": (c_int, (_P, c_int, c_ulonglong, _P)),
    "limn_b200_host_alloc": (c_int, (POINTER(c_void_p), c_ulonglong)),
    "limn_b200_host_free": (c_int, (_P,)),
    "limn_b200_copy_h2d": (c_int, (_P, _P, c_ulonglong, _P)),
    "limn_b200_copy_d2h": (c_int, (_P, _P, c_ulonglong, _P)),
    "limn_b200_copy_d2d": (c_int, (_P, _P, c_ulonglong, _P)),
    "limn_b200_stream_create": (c_int, (POINTER(c_void_p),)),
    "limn_b200_stream_destroy": (c_int, (_P,)),
    "limn_b200_stream_wait_event": (c_int, (_P, _P)),
    "limn_b200_stream_sync": (c_int, (_P,)),
    "limn_b200_device_sync": (c_int, ()),
    "limn_b200_event_create": (c_int, (POINTER(c_void_p),)),
    "limn_b200_event_destroy": (c_int, (_P,)),
    "limn_b200_event_record": (c_int, (_P, _P)),
    "limn_b200_event_elapsed_ms": (c_int, (_P, _P, POINTER(c_float))),
}

_lib: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    """The loaded library with every export typed; raises if it is not there."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"limn_b200: {LIB_PATH} is missing; build it with `python -m limn_b200.build` "
                "(there is no CPU or interpreted fallback)"
            )
        loaded = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(loaded, name)  # AttributeError names a missing export
            fn.restype, fn.argtypes = restype, list(argtypes)
        _lib = loaded
    return _lib


def last_error() -> str:
    return lib().limn_b200_last_error().decode()


def check(code: int, doing: str) -> None:
    """Raise the way limn's driver check does (limn/backend_cuda.py:154-162): RuntimeError
    naming what was being done and what the library said."""
    if code != 0:
        raise RuntimeError(f"limn_b200: {doing}: {last_error() or f'status {code}'}")
