"""The upstream INT4 interchange format and the W4A16 projection (oracle side).

Format (src/crossdsl_kernels/quantization.py:15-37): weights are stored NK,
two signed 4-bit values per byte, the even-k value in the LOW nibble, each
value biased by +8 into a code in [0, 15]; an odd K pads the last high nibble
with code 8 (value zero).  One FP16 scale per (row, group of ``group_size``
consecutive k).  A weight is defined as ``half(float(q) * float(scale))`` --
the rounding to FP16 is part of the format (quantization.py:65-76).
"""

from __future__ import annotations

import numpy as np
import torch

GROUPS = (32, 64, 128, 256)


def codes_to_bytes(q: np.ndarray) -> np.ndarray:
    """int8 [N, K] in [-8, 7] -> uint8 [N, ceil(K/2)] (quantization.py:15-24)."""
    q = np.asarray(q)
    if q.ndim != 2 or q.size == 0 or q.dtype != np.int8:
        raise ValueError("expected a non-empty int8 matrix")
    if (q < -8).any() or (q > 7).any():
        raise ValueError("value outside the signed 4-bit range")
    c = (q.astype(np.int16) + 8).astype(np.uint8)
    if c.shape[1] & 1:
        c = np.concatenate([c, np.full((c.shape[0], 1), 8, np.uint8)], axis=1)
    return (c[:, 0::2] | (c[:, 1::2] << 4)).astype(np.uint8)


def bytes_to_codes(packed: np.ndarray, k: int) -> np.ndarray:
    """uint8 [N, ceil(K/2)] -> int8 [N, K] (quantization.py:27-37)."""
    packed = np.asarray(packed, dtype=np.uint8)
    lo = (packed & 15).astype(np.int16) - 8
    hi = (packed >> 4).astype(np.int16) - 8
    both = np.stack([lo, hi], axis=-1).reshape(packed.shape[0], -1)
    return both[:, :k].astype(np.int8)


def dequantize(packed: torch.Tensor, scales: torch.Tensor, k: int, group_size: int) -> torch.Tensor:
    """FP16 [N, K] weights with the format's rounding (quantization.py:65-76)."""
    if group_size not in GROUPS:
        raise ValueError("unsupported group size")
    q = torch.from_numpy(bytes_to_codes(packed.cpu().numpy(), k))
    column_group = torch.arange(k) // group_size
    return (q.to(torch.float32) * scales.cpu()[:, column_group].to(torch.float32)).to(torch.float16)


def w4a16_projection(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias=None, *, group_size: int = 128) -> torch.Tensor:
    """y = half(x.f64 @ W_fp16.f64^T (+ bias.f64)) (quantization.py:124-131)."""
    w = dequantize(packed, scales, x.shape[1], group_size)
    acc = x.cpu().to(torch.float64) @ w.to(torch.float64).t()
    if bias is not None:
        acc = acc + bias.cpu().to(torch.float64)
    return acc.to(torch.float16)


def w4a16_projection_f32(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias=None, *, group_size: int = 128) -> torch.Tensor:
    """The dense comparator: FP32 matmul against the dequantised weights."""
    w = dequantize(packed, scales, x.shape[1], group_size)
    acc = x.cpu().to(torch.float32) @ w.to(torch.float32).t()
    if bias is not None:
        acc = acc + bias.cpu().to(torch.float32)
    return acc
