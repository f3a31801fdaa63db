"""The INT4 interchange format of the W4A16 projection (host-side helpers).

Same public names and behaviour as upstream's
src/crossdsl_kernels/quantization.py:7-121.  Weights are stored NK as
``uint8 [N, ceil(K/2)]``: two 4-bit codes per byte, the even-k one in the low
nibble, ``code = q + 8`` for a signed value q in [-8, 7]; an odd K leaves code 8
(value zero) in the last high nibble.  Read as little-endian 32-bit words this
is "eight codes per int32 along K".  Scales are FP16 ``[N, ceil(K/group)]`` and
a weight is *defined* as ``half(float(q) * float(scale))``.

These functions work on CPU or CUDA tensors and are set-up tools (they check
values, so they can synchronise); the projection itself is
:func:`cross_dsl_kernels_b200.w4a16.w4a16_linear`.
"""

from __future__ import annotations

import torch

GROUP_SIZES = (32, 64, 128, 256)


def _require_group(group_size) -> None:
    # bool is an int subclass; upstream rejects it too (quantization.py:10-12)
    if type(group_size) is not int or group_size not in GROUP_SIZES:
        raise ValueError(f"group_size must be one of {GROUP_SIZES}")


def _groups(k: int, group_size: int) -> int:
    return -(-k // group_size)


def pack_int4(q: torch.Tensor) -> torch.Tensor:
    """int8 [N, K] with values in [-8, 7] -> uint8 [N, ceil(K/2)]."""
    if q.dtype != torch.int8 or q.ndim != 2 or q.numel() == 0:
        raise ValueError("q must be a nonempty int8 matrix [N, K]")
    if bool((q < -8).any()) or bool((q > 7).any()):
        raise ValueError("INT4 values must lie in [-8, 7]")
    codes = (q.to(torch.int32) + 8)
    if codes.shape[1] & 1:
        pad = torch.full((codes.shape[0], 1), 8, dtype=codes.dtype, device=codes.device)
        codes = torch.cat((codes, pad), dim=1)
    pairs = codes.view(codes.shape[0], -1, 2)
    return (pairs[..., 0] + 16 * pairs[..., 1]).to(torch.uint8).contiguous()


def unpack_int4(packed: torch.Tensor, k: int) -> torch.Tensor:
    """uint8 [N, ceil(K/2)] -> int8 [N, K]; the pad nibble of an odd K is dropped."""
    if type(k) is not int or k < 1:
        raise ValueError("K must be a positive integer")
    if packed.dtype != torch.uint8 or packed.ndim != 2:
        raise ValueError("packed must be a uint8 matrix")
    if packed.shape[0] < 1 or packed.shape[1] != (k + 1) // 2:
        raise ValueError("packed shape must be [N, ceil(K/2)]")
    wide = packed.to(torch.int16)
    nibbles = torch.stack((wide % 16, wide // 16), dim=2).reshape(packed.shape[0], -1)
    return (nibbles[:, :k] - 8).to(torch.int8).contiguous()


def quantize_int4(weight: torch.Tensor, group_size: int = 128):
    """Symmetric round-to-nearest quantisation -> (packed, scales).

    Per (row, group): scale = half(max|w| / 7) (at least 2**-24; 1 for an
    all-zero group), chosen BEFORE q = clamp(round(w / scale), -7, 7), so the
    stored scale is the one the values were rounded against.
    """
    _require_group(group_size)
    if weight.ndim != 2 or weight.numel() == 0 or not weight.is_floating_point():
        raise ValueError("weight must be a nonempty floating-point [N, K] matrix")
    if weight.requires_grad:
        raise ValueError("quantization is forward-only; detach weight explicitly")
    if not bool(torch.isfinite(weight).all()):
        raise ValueError("weight must be finite")
    n, k = weight.shape
    g = _groups(k, group_size)
    w = torch.zeros((n, g * group_size), dtype=torch.float32, device=weight.device)
    w[:, :k] = weight
    w = w.view(n, g, group_size)
    amax = w.abs().amax(dim=2)
    scale = torch.where(amax == 0, torch.ones_like(amax), (amax / 7).clamp_min(2.0 ** -24)).to(torch.float16)
    if not bool(torch.isfinite(scale).all()):
        raise ValueError("group scales cannot be represented in FP16")
    step = scale.to(torch.float32).unsqueeze(2)
    q = torch.round(w / step).clamp_(-7, 7).to(torch.int8)
    if not bool(torch.isfinite((q.to(torch.float32) * step).to(torch.float16)).all()):
        raise ValueError("dequantized weights cannot be represented in FP16")
    return pack_int4(q.view(n, -1)[:, :k]), scale.contiguous()


def quantize_int4_device(weight: torch.Tensor, group_size: int = 128):
    """:func:`quantize_int4` for a weight matrix that already lives on a B200: one CUDA kernel, no FP32 copy of
    the matrix, packed bytes and scales bit-identical to the host function.  Raises the same ValueErrors
    (it reads a status word back, so it synchronises: a set-up step, like the host function)."""
    from . import _native

    _require_group(group_size)
    if weight.ndim != 2 or weight.numel() == 0 or not weight.is_floating_point():
        raise ValueError("weight must be a nonempty floating-point [N, K] matrix")
    if weight.requires_grad:
        raise ValueError("quantization is forward-only; detach weight explicitly")
    if not weight.is_cuda:
        raise ValueError("quantize_int4_device needs a CUDA tensor; use quantize_int4 on the host")
    if weight.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        weight = weight.float()
    weight = weight.contiguous()
    n, k = weight.shape
    with torch.cuda.device(weight.device):
        packed = torch.empty((n, (k + 1) // 2), dtype=torch.uint8, device=weight.device)
        scales = torch.empty((n, _groups(k, group_size)), dtype=torch.float16, device=weight.device)
        status = torch.zeros(1, dtype=torch.int32, device=weight.device)
        rc = _native.lib().xdk_quantize_int4(weight.data_ptr(), _native.dtype_code(weight.dtype), n, k, group_size,
                                             packed.data_ptr(), scales.data_ptr(), status.data_ptr(),
                                             _native.stream_ptr(weight.device))
    _native.check(rc, "xdk_quantize_int4")
    flags = int(status.item())
    if flags & 1:
        raise ValueError("weight must be finite")
    if flags & 2:
        raise ValueError("group scales cannot be represented in FP16")
    if flags & 4:
        raise ValueError("dequantized weights cannot be represented in FP16")
    return packed, scales


def dequantize_int4(packed: torch.Tensor, scales: torch.Tensor, k: int, group_size: int = 128) -> torch.Tensor:
    """FP16 [N, K] weights, each rounded once from the FP32 product q * scale."""
    _require_group(group_size)
    q = unpack_int4(packed, k)
    if scales.dtype != torch.float16 or tuple(scales.shape) != (q.shape[0], _groups(k, group_size)):
        raise ValueError("scales must be FP16 [N, ceil(K/group_size)]")
    if scales.device != packed.device:
        raise ValueError("packed and scales must be on the same device")
    per_column = scales.to(torch.float32).repeat_interleave(group_size, dim=1)[:, :k]
    return (q.to(torch.float32) * per_column).to(torch.float16).contiguous()


def validate_w4a16(x, packed, scales, bias=None, *, group_size=128, out=None, cuda=True):
    """Launch checks on shapes, dtypes, devices and aliasing only (finite values
    are the caller's precondition).  Returns (M, K, N)."""
    _require_group(group_size)
    if x.ndim != 2 or x.dtype != torch.float16:
        raise ValueError("x must be FP16 [M, K]")
    m, k = x.shape
    if m < 1 or m > 16 or k < 1:
        raise ValueError("decode requires 1 <= M <= 16 and K > 0")
    if packed.ndim != 2 or packed.dtype != torch.uint8:
        raise ValueError("packed must be uint8 [N, ceil(K/2)]")
    n = packed.shape[0]
    if n < 1 or packed.shape[1] != (k + 1) // 2:
        raise ValueError("packed shape must be [N, ceil(K/2)]")
    if scales.dtype != torch.float16 or tuple(scales.shape) != (n, _groups(k, group_size)):
        raise ValueError("scales must be FP16 [N, ceil(K/group_size)]")
    if bias is not None and (bias.dtype != torch.float16 or tuple(bias.shape) != (n,)):
        raise ValueError("bias must be FP16 [N] or None")
    inputs = [x, packed, scales] + ([] if bias is None else [bias])
    everything = list(inputs)
    if out is not None:
        if out.dtype != torch.float16 or tuple(out.shape) != (m, n):
            raise ValueError("out must be FP16 [M, N]")
        everything.append(out)
    if cuda and not x.is_cuda:
        raise ValueError("W4A16 kernels require CUDA tensors")
    for t in everything:
        if t.device != x.device or not t.is_contiguous():
            raise ValueError("all tensors must be contiguous and on the same device")
    for t in everything:
        if t.requires_grad:
            raise ValueError("W4A16 kernels are forward-only; detach tensors explicitly")
    if max([m, k, n] + [t.numel() for t in everything]) >= 2 ** 31:
        raise ValueError("this prototype requires signed 32-bit indexing")
    if out is not None:
        o0 = out.data_ptr()
        o1 = o0 + out.numel() * out.element_size()
        for t in inputs:
            t0 = t.data_ptr()
            if o0 < t0 + t.numel() * t.element_size() and t0 < o1:
                raise ValueError("out must not overlap an input")
    return m, k, n
