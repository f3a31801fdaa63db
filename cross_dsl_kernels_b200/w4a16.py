"""``w4a16_linear``: the W4A16 projection behind upstream's signature
(src/crossdsl_kernels/w4a16.py:34-80).

``backend="cuda"`` is the only backend this library has.  ``"reference"``,
``"triton"`` and ``"cute"`` are refused with ValueError: there is no CPU
fallback and no second code path.  ``rows_per_block`` is validated as upstream
does (1 or 4) and otherwise ignored -- the launch configuration is chosen by
the library.
"""

from __future__ import annotations

import torch

from . import _native
from .quantization import validate_w4a16


def linear_out(x, packed, scales, bias, y, group_size, rows_per_block, has_bias, *, dependent_launch=False,
               peer_out=None) -> None:
    """Same call shape as upstream's pybind ``linear_out``
    (csrc/w4a16/w4a16_ext.cpp:7-43): writes the caller-owned ``y``; ``bias`` is a
    placeholder FP16 tensor when ``has_bias`` is false."""
    if type(rows_per_block) is not int or rows_per_block not in (1, 4):
        raise ValueError("rows_per_block must be 1 or 4")
    m, k, n = validate_w4a16(x, packed, scales, bias if has_bias else None, group_size=group_size, out=y)
    if torch.cuda.get_device_capability(x.device)[0] != 10:
        raise ValueError("these kernels are built for sm_100a (B200) only")
    flags = _native.XDK_DEPENDENT_LAUNCH if dependent_launch else 0
    with torch.cuda.device(x.device):
        if peer_out is not None:  # multi-GPU: this rank's columns of the full-width matrix on every rank
            import ctypes
            if peer_out.ld < peer_out.col0 + n:
                raise ValueError("peer_out is narrower than col0 + N")
            status = _native.lib().xdk_w4a16_peer(x.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                                  bias.data_ptr() if has_bias else None, ctypes.byref(peer_out), m, k, n,
                                                  group_size, flags, _native.stream_ptr(x.device))
        else:
            status = _native.lib().xdk_w4a16_v2(x.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                                bias.data_ptr() if has_bias else None, y.data_ptr(), m, k, n, group_size,
                                                flags, _native.stream_ptr(x.device))
    _native.check(status, "xdk_w4a16")


def w4a16_linear(x, packed, scales, bias=None, *, group_size=128, backend="cuda", rows_per_block=1, out=None,
                 dependent_launch=False, peer_out=None):
    """``dependent_launch=True``: launch as a programmatic dependent of the preceding kernel on the stream (the
    packed codes, scales and bias must not be that kernel's output; ``x`` may be).  ``peer_out`` (multi-GPU, from
    ``PeerMatrix.out_for``): store the result into this rank's columns of the full-width matrix on every rank;
    nothing is allocated and None is returned."""
    if backend != "cuda":
        if backend in ("reference", "triton", "cute"):
            raise ValueError(f"backend {backend!r} is not part of this library: it runs the sm_100a CUDA kernel only")
        raise ValueError("backend must be reference, cuda, triton or cute")
    if type(rows_per_block) is not int or rows_per_block not in (1, 4):
        raise ValueError("rows_per_block must be 1 (baseline) or 4 (reuse candidate)")
    m, _, n = validate_w4a16(x, packed, scales, bias, group_size=group_size, out=out)
    placeholder = scales if bias is None else bias
    if peer_out is not None:
        if out is not None:
            raise ValueError("pass either out or peer_out")
        linear_out(x, packed, scales, placeholder, None, group_size, rows_per_block, bias is not None,
                   dependent_launch=dependent_launch, peer_out=peer_out)
        return None
    y = out if out is not None else torch.empty((m, n), device=x.device, dtype=x.dtype)
    linear_out(x, packed, scales, placeholder, y, group_size, rows_per_block, bias is not None,
               dependent_launch=dependent_launch)
    return y
