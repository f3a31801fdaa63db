"""GPU entry points of the three floating-point decode ops.

Each function keeps the positional/keyword layout of the upstream PyTorch
reference it stands in for, so ``functools.partial(op, *case["args"],
**case["kwargs"])`` written for the reference works unchanged:

* :func:`fused_residual_rmsnorm`  <- fused_residual_rmsnorm_reference
  (src/crossdsl_kernels/references/rmsnorm.py:6-25)
* :func:`decode_linear`           <- decode_linear_reference
  (src/crossdsl_kernels/references/gemv.py:6-36)
* :func:`rope_gqa_paged_kv_append` <- rope_gqa_paged_kv_append_reference
  (src/crossdsl_kernels/references/rope_kv.py:35-70)

Checks mirror upstream's native bindings (csrc/*/*_ext.cpp) and raise
ValueError; the kernels run on the tensor's device, on torch's current stream,
without synchronising, and are safe under CUDA-graph capture.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _native
from .contracts import validate_cache_storage

_RMS_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise ValueError(message)


def _gate(t: torch.Tensor) -> None:
    _need(t.is_cuda, "tensors must live on a CUDA device (there is no CPU path)")
    if torch.cuda.get_device_capability(t.device)[0] != 10:
        raise ValueError("these kernels are built for sm_100a (B200) only")


def _flags(dependent_launch: bool, strict_fp32: bool = False) -> int:
    return (_native.XDK_DEPENDENT_LAUNCH if dependent_launch else 0) | (_native.XDK_STRICT_FP32 if strict_fp32 else 0)


def fused_residual_rmsnorm(x, residual, weight, eps, *, return_residual: bool = True, dependent_launch: bool = False):
    """(y, residual_out) = RMSNorm(x + residual) * weight and the FP32 sum rounded to dtype.

    ``dependent_launch=True`` (every op of this module takes it) launches the kernel as a programmatic
    dependent of the preceding kernel on the stream, so that its scheduling and set-up overlap that
    kernel's tail; the caller promises that ``weight`` was not written by that kernel."""
    _gate(x)
    _need(residual.is_cuda and weight.is_cuda, "residual and weight must be CUDA tensors")
    _need(x.dtype in _RMS_DTYPES, "x must be float32, bfloat16 or float16")
    _need(residual.dtype == x.dtype, "residual dtype must match x")
    _need(weight.dtype == x.dtype, "weight dtype must match x")
    _need(x.dim() == 2, "x must be a 2D tensor shaped [rows, hidden]")
    _need(residual.shape == x.shape, "residual must match x shape")
    _need(weight.dim() == 1 and weight.shape[0] == x.shape[1], "weight must be shaped [hidden]")
    _need(x.is_contiguous() and residual.is_contiguous() and weight.is_contiguous(), "tensors must be contiguous")
    _need(residual.device == x.device and weight.device == x.device, "tensors must share one CUDA device")
    _need(x.shape[0] > 0 and x.shape[1] > 0, "rows and hidden size must be positive")
    eps = float(eps)
    _need(math.isfinite(eps) and eps > 0.0, "eps must be finite and positive")
    with torch.cuda.device(x.device):
        y = torch.empty_like(x)
        residual_out = torch.empty_like(residual)
        status = _native.lib().xdk_rmsnorm_v2(
            x.data_ptr(), residual.data_ptr(), weight.data_ptr(), y.data_ptr(), residual_out.data_ptr(),
            x.shape[0], x.shape[1], eps, _native.dtype_code(x.dtype), _flags(dependent_launch),
            _native.stream_ptr(x.device))
    _native.check(status, "xdk_rmsnorm")
    return y, (residual_out if return_residual else None)


def decode_linear(x, weight, bias=None, *, out_dtype=None, weight_layout: str = "KN", split_k: int = 0,
                  strict_fp32: bool = False, dependent_launch: bool = False, peer_out=None):
    """y = x @ W (+ bias) in FP32.  ``split_k`` in {0 (auto), 1, 2, 4, 8}.

    With ``split_k=0`` and 4 < M <= 16 a large projection runs on the tensor cores as split-TF32
    products with FP32 accumulation (relative L2 error ~1e-6 against an FP64 product, inside the
    projection's 1e-5 gate).  ``strict_fp32=True`` keeps such shapes on the CUDA-core tile-stream
    kernel, whose every product and sum is an FP32 FMA; it needs a scratch block per call.

    ``peer_out`` (multi-GPU; from :meth:`cross_dsl_kernels_b200.peer.PeerMatrix.out_for`): the kernel stores its
    [M, N] result into columns [col0, col0 + N) of the full-width matrix on every rank instead of allocating
    an output; the call then returns None and the caller orders readers with ``PeerArena.barrier``."""
    _need(x.dim() == 2, "x must be a 2D tensor shaped [M, K]")
    _need(weight.dim() == 2, "weight must be a 2D tensor")
    _need(weight_layout in ("KN", "NK"), "weight_layout must be 'KN' or 'NK'")
    _gate(x)
    _need(weight.is_cuda and weight.device == x.device, "x and weight must be on the same CUDA device")
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "x and weight must be float32")
    _need(out_dtype in (None, torch.float32), "the CUDA projection writes float32")
    nk = weight_layout == "NK"
    m, k = x.shape
    n = weight.shape[0] if nk else weight.shape[1]
    _need(m > 0 and k > 0 and n > 0, "M, K and N must be positive")
    _need((weight.shape[1] if nk else weight.shape[0]) == k, "x K dimension must match weight K dimension")
    _need(x.is_contiguous() and weight.is_contiguous(), "x and weight must be contiguous")
    _need(type(split_k) is int and split_k in (0, 1, 2, 4, 8), "split_k must be 0 (auto), 1, 2, 4 or 8")
    bias_ptr = None
    if bias is not None:
        _need(bias.is_cuda and bias.device == x.device, "bias must be on the same CUDA device")
        _need(bias.dtype == torch.float32, "bias must be float32")
        _need(bias.dim() == 1 and bias.shape[0] == n, "bias must be a 1D tensor shaped [N]")
        _need(bias.is_contiguous(), "bias must be contiguous")
        bias_ptr = bias.data_ptr()
    with torch.cuda.device(x.device):
        lib = _native.lib()
        if peer_out is not None:
            _need(peer_out.ld >= peer_out.col0 + n, "peer_out is narrower than col0 + N")
            need = lib.xdk_gemv_scratch_bytes(m, k, n, int(nk)) if (split_k == 0 and strict_fp32) else 0
            scratch = torch.empty(need, device=x.device, dtype=torch.uint8) if need else None
            import ctypes
            status = lib.xdk_gemv_f32_peer(x.data_ptr(), weight.data_ptr(), bias_ptr, ctypes.byref(peer_out), m, k, n,
                                           int(nk), split_k, scratch.data_ptr() if need else None, need,
                                           _flags(dependent_launch, strict_fp32), _native.stream_ptr(x.device))
            _native.check(status, "xdk_gemv_f32_peer")
            return None
        y = torch.empty((m, n), device=x.device, dtype=torch.float32)
        # Scratch lets strict-FP32 calls use the balanced tile-stream path (4 < M <= 16, split_k = 0).  A fresh block from
        # torch's caching allocator per call: stream-ordered, so overlapping calls never share it,
        # and under graph capture it lives in the graph's private pool.
        need = lib.xdk_gemv_scratch_bytes(m, k, n, int(nk)) if (split_k == 0 and strict_fp32) else 0
        scratch = torch.empty(need, device=x.device, dtype=torch.uint8) if need else None
        status = lib.xdk_gemv_f32_v2(x.data_ptr(), weight.data_ptr(), bias_ptr, y.data_ptr(), m, k, n, int(nk), split_k,
                                     scratch.data_ptr() if need else None, need, _flags(dependent_launch, strict_fp32),
                                     _native.stream_ptr(x.device))
    _native.check(status, "xdk_gemv_f32")
    return y


def rope_gqa_paged_kv_append(q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache, *,
                             page_size: int, rope_dim: int, interleaved: bool, kv_layout: str = "NHD",
                             dependent_launch: bool = False, q_peer_out=None):
    """Rotate Q and K, write rotated K and V into the paged caches in place, return rotated Q.

    Index values are trusted: validate them once at set-up with
    :func:`cross_dsl_kernels_b200.references.validate_paged_kv_indices`.
    """
    _gate(q)
    dtype = q.dtype
    _need(dtype in _RMS_DTYPES, "q must be float32, bfloat16 or float16")
    for name, t, want in (("k", k, dtype), ("v", v, dtype), ("k_cache", k_cache, dtype), ("v_cache", v_cache, dtype),
                          ("cos", cos, torch.float32), ("sin", sin, torch.float32),
                          ("positions", positions, torch.int64), ("page_table", page_table, torch.int64),
                          ("sequence_ids", sequence_ids, torch.int64)):
        _need(t.is_cuda and t.device == q.device, f"{name} must be on the same CUDA device as q")
        _need(t.dtype == want, f"{name} has an unexpected dtype")
        _need(name in ("k", "v") or t.is_contiguous(), f"{name} must be contiguous")
    for name, t in (("q", q), ("k", k), ("v", v)):
        # contiguous, or a column slice of a wider row-major matrix (fused QKV output):
        # heads and dims dense, tokens a fixed number of elements apart
        dense = t.dim() == 3 and t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) >= t.shape[1] * t.shape[2]
        _need(t.is_contiguous() or dense, f"{name} must be contiguous or a column slice of a row-major matrix")
    _need(q.dim() == 3 and k.dim() == 3 and v.dim() == 3, "q, k, v must be [tokens, heads, head_dim]")
    _need(cos.dim() == 2 and sin.dim() == 2, "cos and sin must be [max_position, >= rope_dim / 2]")
    _need(positions.dim() == 1 and sequence_ids.dim() == 1, "positions and sequence_ids must be vectors")
    _need(page_table.dim() == 2, "page_table must be [sequences, max_pages]")
    _need(k_cache.dim() == 4 and v_cache.dim() == 4, "caches must be 4D paged tensors")
    tokens, q_heads, head_dim = q.shape
    kv_heads = k.shape[1]
    _need(tokens > 0 and q_heads > 0 and kv_heads > 0 and head_dim > 0, "tokens, heads and head_dim must be positive")
    _need(q_heads % kv_heads == 0, "q_heads must be divisible by kv_heads")
    _need(k.shape[0] == tokens and v.shape[0] == tokens, "q, k and v token counts must match")
    _need(k.shape[2] == head_dim and v.shape[2] == head_dim, "q, k and v head_dim must match")
    _need(v.shape[1] == kv_heads, "k and v kv_heads must match")
    _need(positions.shape[0] == tokens and sequence_ids.shape[0] == tokens, "index vectors must have one entry per token")
    _need(type(page_size) is int and page_size > 0, "page_size must be positive")
    _need(type(rope_dim) is int and rope_dim > 0 and rope_dim % 2 == 0, "rope_dim must be a positive even integer")
    _need(rope_dim <= head_dim, "rope_dim cannot exceed head_dim")
    _need(cos.shape[1] >= rope_dim // 2 and sin.shape == cos.shape, "cos/sin need >= rope_dim / 2 columns and equal shapes")
    _need(page_table.shape[1] > 0, "page_table must contain at least one page per sequence row")
    layout = kv_layout.upper()
    _need(layout in ("NHD", "HND"), "kv_layout must be NHD or HND")
    _need(k_cache.shape == v_cache.shape, "k_cache and v_cache shapes must match")
    want = (page_size, kv_heads, head_dim) if layout == "NHD" else (kv_heads, page_size, head_dim)
    _need(tuple(k_cache.shape[1:]) == want, f"{layout} cache dimensions must be (pages, {want})")
    validate_cache_storage((q, k, v, cos, sin, positions, page_table, sequence_ids), k_cache, v_cache)
    with torch.cuda.device(q.device):
        import ctypes
        if q_peer_out is None:  # rotated Q into a fresh contiguous tensor
            q_out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            dst = _native.PeerOutStruct()
            dst.ptr[0], dst.world, dst.ld, dst.col0 = q_out.data_ptr(), 1, q_heads * head_dim, 0
        else:  # multi-GPU: rotated Q into this rank's columns of the full-width matrix on every rank
            q_out, dst = None, q_peer_out
            _need(dst.ld >= dst.col0 + q_heads * head_dim, "q_peer_out is narrower than col0 + q_heads * head_dim")
        status = _native.lib().xdk_rope_kv_append_peer(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(),
            page_table.data_ptr(), sequence_ids.data_ptr(), ctypes.byref(dst), k_cache.data_ptr(), v_cache.data_ptr(),
            tokens, q_heads, kv_heads, head_dim, cos.shape[1], page_table.shape[1], page_size, rope_dim,
            q.stride(0) if tokens > 1 else q_heads * head_dim, k.stride(0) if tokens > 1 else kv_heads * head_dim,
            v.stride(0) if tokens > 1 else kv_heads * head_dim, int(bool(interleaved)), int(layout == "HND"), _native.dtype_code(dtype), _flags(dependent_launch),
            _native.stream_ptr(q.device))
    _native.check(status, "xdk_rope_kv_append")
    return q_out


def paged_decode_attention(q, k_cache, v_cache, positions, page_table, sequence_ids, *, page_size: int,
                           kv_layout: str = "NHD", scale=None, context_hint: int = 0, dependent_launch: bool = False,
                           peer_out=None):
    """Decode attention of one query token per sequence over the paged K/V cache that
    :func:`rope_gqa_paged_kv_append` wrote (the token's own K/V included): FP32 softmax(scale * q.K) . V per head,
    GQA with q_heads / kv_heads in {1, 2, 4, 8}, head_dim in {64, 128, 256}.  Not part of upstream.

    ``peer_out`` (multi-GPU; :meth:`cross_dsl_kernels_b200.peer.PeerMatrix.out_for`): the result goes to columns
    [col0, col0 + q_heads * head_dim) of every rank's copy of a [tokens, all heads * head_dim] matrix instead of a
    fresh tensor, and the call returns None; readers wait for the arena's flag barrier."""
    _gate(q)
    dtype = q.dtype
    _need(dtype in _RMS_DTYPES, "q must be float32, bfloat16 or float16")
    for name, t, want in (("k_cache", k_cache, dtype), ("v_cache", v_cache, dtype), ("positions", positions, torch.int64),
                          ("page_table", page_table, torch.int64), ("sequence_ids", sequence_ids, torch.int64)):
        _need(t.is_cuda and t.device == q.device, f"{name} must be on the same CUDA device as q")
        _need(t.dtype == want, f"{name} has an unexpected dtype")
        _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(q.dim() == 3 and q.is_contiguous(), "q must be contiguous [tokens, q_heads, head_dim]")
    _need(k_cache.dim() == 4 and k_cache.shape == v_cache.shape, "caches must be 4D paged tensors of one shape")
    _need(positions.dim() == 1 and sequence_ids.dim() == 1 and page_table.dim() == 2, "index tensors have the wrong rank")
    tokens, q_heads, head_dim = q.shape
    layout = kv_layout.upper()
    _need(layout in ("NHD", "HND"), "kv_layout must be NHD or HND")
    _need(type(page_size) is int and page_size > 0, "page_size must be positive")
    kv_heads = k_cache.shape[2] if layout == "NHD" else k_cache.shape[1]
    want = (page_size, kv_heads, head_dim) if layout == "NHD" else (kv_heads, page_size, head_dim)
    _need(tuple(k_cache.shape[1:]) == want, f"{layout} cache dimensions must be (pages, {want})")
    _need(q_heads % kv_heads == 0 and q_heads // kv_heads in (1, 2, 4, 8), "q_heads / kv_heads must be 1, 2, 4 or 8")
    _need(head_dim in (64, 128, 256), "head_dim must be 64, 128 or 256")
    _need(positions.shape[0] == tokens and sequence_ids.shape[0] == tokens, "index vectors must have one entry per token")
    scale = float(head_dim) ** -0.5 if scale is None else float(scale)
    _need(math.isfinite(scale), "scale must be finite")
    with torch.cuda.device(q.device):
        tail = (tokens, q_heads, kv_heads, head_dim, page_table.shape[1], page_size, int(layout == "HND"), scale,
                int(context_hint), _native.dtype_code(dtype), _flags(dependent_launch), _native.stream_ptr(q.device))
        head = (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(), page_table.data_ptr(),
                sequence_ids.data_ptr())
        if peer_out is None:
            out = torch.empty_like(q)
            status = _native.lib().xdk_paged_decode_attention(*head, out.data_ptr(), *tail)
        else:
            _need(peer_out.ld >= peer_out.col0 + q_heads * head_dim, "peer_out is narrower than col0 + q_heads * head_dim")
            out = None
            status = _native.lib().xdk_paged_decode_attention_peer(*head, ctypes.byref(peer_out), *tail)
    _native.check(status, "xdk_paged_decode_attention")
    return out


def swiglu(upgate, *, dependent_launch: bool = False, peer_out=None):
    """silu(gate) * up for a fused projection output ``[rows, 2 * width]`` laid out [up | gate]; returns [rows, width].
    Rows may be a fixed number of elements apart (a column slice of a wider matrix).  Not part of upstream.
    ``peer_out``: as for :func:`paged_decode_attention` (columns [col0, col0 + width) of every rank's matrix)."""
    _gate(upgate)
    _need(upgate.dtype in _RMS_DTYPES, "upgate must be float32, bfloat16 or float16")
    _need(upgate.dim() == 2 and upgate.shape[1] % 2 == 0 and upgate.shape[0] > 0 and upgate.shape[1] > 0,
          "upgate must be [rows, 2 * width]")
    _need(upgate.stride(1) == 1 and upgate.stride(0) >= upgate.shape[1], "upgate rows must be dense")
    rows, width = upgate.shape[0], upgate.shape[1] // 2
    with torch.cuda.device(upgate.device):
        in_ld = upgate.stride(0) if rows > 1 else 2 * width
        if peer_out is None:
            out = torch.empty((rows, width), dtype=upgate.dtype, device=upgate.device)
            status = _native.lib().xdk_swiglu(upgate.data_ptr(), out.data_ptr(), rows, width, in_ld, width,
                                              _native.dtype_code(upgate.dtype), _flags(dependent_launch),
                                              _native.stream_ptr(upgate.device))
        else:
            _need(peer_out.ld >= peer_out.col0 + width, "peer_out is narrower than col0 + width")
            out = None
            status = _native.lib().xdk_swiglu_peer(upgate.data_ptr(), ctypes.byref(peer_out), rows, width, in_ld,
                                                   _native.dtype_code(upgate.dtype), _flags(dependent_launch),
                                                   _native.stream_ptr(upgate.device))
    _native.check(status, "xdk_swiglu")
    return out
