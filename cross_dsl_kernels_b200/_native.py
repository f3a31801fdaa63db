"""ctypes binding of ``libxdk_b200.so`` (the C ABI declared in include/xdk_b200.h).

There is no fallback: if the library is missing or a call returns an error
status, the caller gets an exception.  Nothing here computes on the CPU.
"""

from __future__ import annotations

import ctypes
import functools
import pathlib

LIB_PATH = pathlib.Path(__file__).resolve().parent / "libxdk_b200.so"

XDK_F32, XDK_BF16, XDK_F16 = 0, 1, 2
XDK_STRICT_FP32, XDK_DEPENDENT_LAUNCH = 1, 2  # flags of the *_v2 entry points

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_uint = ctypes.c_uint

# name -> (restype, argtypes); one row per symbol declared in include/xdk_b200.h
SIGNATURES = {
    "xdk_strerror": (ctypes.c_char_p, [_int]),
    "xdk_abi_version": (_int, []),
    "xdk_last_cuda_error": (_int, []),
    "xdk_device_supported": (_int, [_int]),
    "xdk_fault_flags": (ctypes.c_uint, []),
    "xdk_noop": (_int, [_uint, _p]),
    "xdk_rmsnorm": (_int, [_p, _p, _p, _p, _p, _i64, _i64, ctypes.c_float, _int, _p]),
    "xdk_rmsnorm_v2": (_int, [_p, _p, _p, _p, _p, _i64, _i64, ctypes.c_float, _int, _uint, _p]),
    "xdk_gemv_f32": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, ctypes.c_size_t, _p]),
    "xdk_gemv_f32_v2": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, ctypes.c_size_t, _uint, _p]),
    "xdk_gemv_tc_plan": (_int, [_i64, _i64, _i64, _int, _p]),
    "xdk_gemv_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _int]),
    "xdk_gemv_f32_static_scratch": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _p]),
    "xdk_rope_kv_append": (_int, [_p] * 11 + [_i64] * 11 + [_int, _int, _int, _p]),
    "xdk_rope_kv_append_v2": (_int, [_p] * 11 + [_i64] * 11 + [_int, _int, _int, _uint, _p]),
    "xdk_w4a16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _p]),
    "xdk_w4a16_v2": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _uint, _p]),
    "xdk_paged_decode_attention": (_int, [_p] * 7 + [_i64] * 6 + [_int, ctypes.c_float, _i64, _int, _uint, _p]),
    "xdk_swiglu": (_int, [_p, _p, _i64, _i64, _i64, _i64, _int, _uint, _p]),
    "xdk_paged_decode_attention_peer": (_int, [_p] * 7 + [_i64] * 6 + [_int, ctypes.c_float, _i64, _int, _uint, _p]),
    "xdk_swiglu_peer": (_int, [_p, _p, _i64, _i64, _i64, _int, _uint, _p]),
    "xdk_quantize_int4": (_int, [_p, _int, _i64, _i64, _int, _p, _p, _p, _p]),
    "xdk_peer_fault_flags": (ctypes.c_uint, []),
    "xdk_peer_alloc": (_int, [ctypes.c_size_t, _p]),
    "xdk_peer_free": (_int, [_p]),
    "xdk_peer_export": (_int, [_p, _p]),
    "xdk_peer_open": (_int, [_p, _p]),
    "xdk_peer_close": (_int, [_p]),
    "xdk_peer_barrier": (_int, [_p, _int, _int, _int, _uint, _uint, _p]),
    "xdk_gemv_f32_peer": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, ctypes.c_size_t, _uint, _p]),
    "xdk_w4a16_peer": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _uint, _p]),
    "xdk_rope_kv_append_peer": (_int, [_p] * 11 + [_i64] * 11 + [_int, _int, _int, _uint, _p]),
    "xdk_unshard_columns": (_int, [_p, _p, _i64, _i64, _i64, _int, _p]),
}


XDK_MAX_PEERS = 8
XDK_PEER_FLAG_BYTES = 8192


class PeerOutStruct(ctypes.Structure):
    """``xdk_peer_out`` of include/xdk_b200.h."""

    _fields_ = [("ptr", ctypes.c_void_p * XDK_MAX_PEERS), ("world", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("ld", ctypes.c_int64), ("col0", ctypes.c_int64)]


class NativeLibraryError(RuntimeError):
    """The CUDA library is missing, or one of its entry points reported an error."""


@functools.lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise NativeLibraryError(
            f"{LIB_PATH} is not built; run `python -m cross_dsl_kernels_b200.build` "
            "(needs nvcc; there is no CPU fallback)"
        )
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def check(status: int, what: str) -> None:
    if status == 0:
        return
    handle = lib()
    text = handle.xdk_strerror(status).decode()
    raise NativeLibraryError(f"{what}: {text} (status {status}, cudaError {handle.xdk_last_cuda_error()})")


def fault_flags() -> int:
    """OR of the kernels' wait-timeout bits on the current device (0 = healthy); synchronises."""
    return int(lib().xdk_fault_flags())


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float32: XDK_F32, torch.bfloat16: XDK_BF16, torch.float16: XDK_F16}[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}") from None


def stream_ptr(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
