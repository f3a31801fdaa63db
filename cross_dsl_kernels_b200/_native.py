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

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int

# name -> (restype, argtypes); one row per symbol declared in include/xdk_b200.h
SIGNATURES = {
    "xdk_strerror": (ctypes.c_char_p, [_int]),
    "xdk_abi_version": (_int, []),
    "xdk_last_cuda_error": (_int, []),
    "xdk_device_supported": (_int, [_int]),
    "xdk_fault_flags": (ctypes.c_uint, []),
    "xdk_rmsnorm": (_int, [_p, _p, _p, _p, _p, _i64, _i64, ctypes.c_float, _int, _p]),
    "xdk_gemv_f32": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _int, _p, ctypes.c_size_t, _p]),
    "xdk_gemv_tc_plan": (_int, [_i64, _i64, _i64, _int, _p]),
    "xdk_gemv_scratch_bytes": (ctypes.c_size_t, [_i64, _i64, _i64, _int]),
    "xdk_gemv_f32_static_scratch": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _p]),
    "xdk_rope_kv_append": (_int, [_p] * 11 + [_i64] * 11 + [_int, _int, _int, _p]),
    "xdk_w4a16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _p]),
    "xdk_unshard_columns": (_int, [_p, _p, _i64, _i64, _i64, _int, _p]),
}


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
