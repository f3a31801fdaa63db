"""CPU restatement of the three floating-point decode ops (oracle side).

TEST INFRASTRUCTURE: imported by tests, the smoke check and the benchmark's
CPU-baseline leg only.  Written with torch CPU tensors because the upstream
references are themselves torch expressions whose rounding behaviour (FP32
elementwise ops, ``rsqrt``, ``matmul``) defines the expected bits.
"""

from __future__ import annotations

import numpy as np
import torch

from . import paging


def residual_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """(y, residual_out) of the fused residual RMSNorm.

    Follows src/crossdsl_kernels/references/rmsnorm.py:6-25: the sum x+residual
    is formed and normalised in FP32 *without* being rounded to the storage
    dtype first; only the two results are rounded (to x's and residual's dtype).
    """
    f32 = torch.float32
    summed = x.to(f32) + residual.to(f32)
    scale = torch.rsqrt((summed * summed).mean(dim=-1, keepdim=True) + eps)
    y = (summed * scale * weight.to(f32)).to(x.dtype)
    return y, summed.to(residual.dtype)


def decode_projection(x: torch.Tensor, weight: torch.Tensor, bias=None, *, weight_layout: str = "KN", out_dtype=None):
    """y = x W (+ b) in FP32 (src/crossdsl_kernels/references/gemv.py:6-36).

    ``weight`` is [K, N] for "KN" and [N, K] for "NK"; the same rejections as
    upstream (rank, layout string, K mismatch, bias shape) raise ValueError.
    """
    if x.dim() != 2 or weight.dim() != 2:
        raise ValueError("x and weight must be matrices")
    if weight_layout not in ("KN", "NK"):
        raise ValueError("weight_layout must be 'KN' or 'NK'")
    w = weight if weight_layout == "KN" else weight.t()
    if x.shape[1] != w.shape[0]:
        raise ValueError("x K dimension must match weight K dimension")
    if bias is not None and tuple(bias.shape) != (w.shape[1],):
        raise ValueError("bias must be shaped [N]")
    y = x.to(torch.float32) @ w.to(torch.float32)
    if bias is not None:
        y = y + bias.to(torch.float32)
    return y.to(out_dtype or x.dtype)


def split_k_bounds(k: int, split_k: int):
    """K ranges of a deterministic split-K projection.

    Chunk length is ceil(K / split_k) rounded up to a multiple of 32, the same
    rule as upstream's only split-K implementation
    (src/crossdsl_kernels/triton/gemv_rows.py:124: ``cdiv(K, 128) * 32`` for
    its fixed four-way split).  Trailing chunks may be empty.
    """
    chunk = -(-k // split_k)
    chunk = -(-chunk // 32) * 32
    return [(min(i * chunk, k), min((i + 1) * chunk, k)) for i in range(split_k)]


def rotate_heads(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, rope_dim: int, interleaved: bool):
    """Rotary embedding of the first ``rope_dim`` dims of every head.

    Follows src/crossdsl_kernels/references/rope_kv.py:8-32.  The four products
    and the add/subtract are separately rounded FP32 operations; the result is
    rounded once more to x's dtype.  Dims at and beyond ``rope_dim`` pass through.
    """
    if rope_dim <= 0 or rope_dim % 2 or rope_dim > x.shape[-1]:
        raise ValueError("rope_dim must be a positive even integer no larger than head_dim")
    half = rope_dim // 2
    f32 = torch.float32
    c = cos[positions, :half].to(f32)[:, None, :]
    s = sin[positions, :half].to(f32)[:, None, :]
    head = x[..., :rope_dim].to(f32)
    if interleaved:
        first, second = head[..., 0::2], head[..., 1::2]
    else:
        first, second = head[..., :half], head[..., half:]
    new_first = (first * c - second * s).to(x.dtype)
    new_second = (first * s + second * c).to(x.dtype)
    out = x.clone()
    if interleaved:
        out[..., 0:rope_dim:2] = new_first
        out[..., 1:rope_dim:2] = new_second
    else:
        out[..., :half] = new_first
        out[..., half:rope_dim] = new_second
    return out


def rope_paged_append(q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache, *,
                      page_size: int, rope_dim: int, interleaved: bool, kv_layout: str = "NHD"):
    """Rotate Q and K, then write rotated K and raw V into the paged caches.

    Follows src/crossdsl_kernels/references/rope_kv.py:35-70 (and its batched
    form, :106-149): token t of sequence s at position p lands in physical page
    ``page_table[s][p // page_size]`` at in-page offset ``p % page_size``.  The
    caches are modified in place; every other slot keeps its contents.
    Returns the rotated Q.
    """
    layout = kv_layout.upper()
    if layout not in ("NHD", "HND"):
        raise ValueError("kv_layout must be NHD or HND")
    q_rot = rotate_heads(q, cos, sin, positions, rope_dim, interleaved)
    k_rot = rotate_heads(k, cos, sin, positions, rope_dim, interleaved)
    pages, offsets = paging.translate(positions.numpy(), sequence_ids.numpy(), page_table.numpy(), page_size)
    pages_t, offsets_t = torch.from_numpy(pages), torch.from_numpy(offsets)
    if layout == "NHD":
        k_cache[pages_t, offsets_t] = k_rot
        v_cache[pages_t, offsets_t] = v
    else:
        k_cache[pages_t, :, offsets_t] = k_rot
        v_cache[pages_t, :, offsets_t] = v
    return q_rot


def rope_paged_append_flat(q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache, *,
                           page_size: int, rope_dim: int, interleaved: bool, kv_layout: str = "NHD"):
    """Same op, but the destination of every element comes from the flattened
    index formulas (src/crossdsl_kernels/references/paged_address.py:32-56)
    instead of tensor indexing: an independent check of the address math that
    device code has to reproduce."""
    layout = kv_layout.upper()
    q_rot = rotate_heads(q, cos, sin, positions, rope_dim, interleaved)
    k_rot = rotate_heads(k, cos, sin, positions, rope_dim, interleaved)
    tokens, heads, dim = k.shape
    pages, offsets = paging.translate(positions.numpy(), sequence_ids.numpy(), page_table.numpy(), page_size)
    t, h, d = np.meshgrid(np.arange(tokens), np.arange(heads), np.arange(dim), indexing="ij")
    index = paging.flat_index(layout, pages[t], offsets[t], h, d, page_size=page_size, num_heads=heads, head_dim=dim)
    index = torch.from_numpy(index.reshape(-1))
    k_cache.view(-1)[index] = k_rot.reshape(-1)
    v_cache.view(-1)[index] = v.reshape(-1)
    return q_rot


def check_paged_indices(positions, page_table, sequence_ids, *, page_size: int, num_cache_pages: int, max_position: int):
    """Set-up validator (src/crossdsl_kernels/references/rope_kv.py:73-103):
    bounds of every index plus pairwise-distinct destination slots."""
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    pos = np.asarray(positions, dtype=np.int64)
    seq = np.asarray(sequence_ids, dtype=np.int64)
    table = np.asarray(page_table, dtype=np.int64)
    if pos.ndim != 1 or seq.shape != pos.shape or table.ndim != 2:
        raise ValueError("positions/sequence_ids must be matching vectors and page_table a matrix")
    if ((seq < 0) | (seq >= table.shape[0])).any():
        raise ValueError("sequence ID is out of bounds")
    if ((pos < 0) | (pos >= max_position)).any():
        raise ValueError("position is outside the trigonometric table")
    pages, offsets = paging.translate(pos, seq, table, page_size)
    if (pages >= num_cache_pages).any():
        raise ValueError("physical page ID is outside the cache")
    slots = pages * page_size + offsets
    if np.unique(slots).size != slots.size:
        raise ValueError("tokens must write distinct physical cache slots")
