"""The call shapes of upstream's four native (pybind11) modules, served by this library.

Upstream JIT-builds one extension per op and calls module-level functions with
positional arguments; a harness written against those modules can import this
module in their place:

* csrc/rmsnorm/rmsnorm_ext.cpp:37-44    ``fused_residual_rmsnorm(x, residual, weight, eps, fast=False) -> [y, residual_out]``
* csrc/gemv/gemv_ext.cpp:77-85          ``decode_gemv{,_warp,_rows}(x, weight, bias_or_empty, layout) -> y``
  -- an EMPTY tensor of any dtype means "no bias" (gemv_ext.cpp:34,48; exercised by scripts/verify_optimized.py:100-116)
* csrc/gemv/gemv_simt_ext.cpp:87-97     ``decode_gemv_simt_{warp,rows}`` / ``decode_gemm_tiled(x, weight, bias=None, layout="KN") -> y``
  -- ``None`` means "no bias"; an empty tensor is a shape error there (scripts/verify_gemv_simt.py:108)
* csrc/rope_kv/rope_kv_ext.cpp:133-144  ``rope_gqa_paged_kv_append(q, k, v, cos, sin, positions, page_table, sequence_ids,
  k_cache, v_cache, page_size, rope_dim, interleaved, kv_layout, fused=False) -> q_out``
* csrc/w4a16/w4a16_ext.cpp:41-43        ``linear_out(x, packed, scales, bias_or_placeholder, y, group_size, rows_per_block, has_bias)``

Upstream's variants of one op (v0 / warp / rows / tiled kernels, ``fast``,
``fused``) differ only in how the kernel is organised; here every name of an
op reaches the same sm_100a kernel selection, and the switches are accepted
and ignored.  The cuBLAS / cuBLASLt comparators (``decode_gemv_cublas``,
``decode_gemv_cublaslt``) are library baselines of upstream's study, not part
of the path, and are not provided.  Invalid arguments raise ValueError where
upstream's TORCH_CHECK raises RuntimeError; upstream's callers accept either.
All projections here use FP32 FMA arithmetic (``strict_fp32``): these entry
points stand in for upstream's strict-FP32 SIMT kernels.
"""

from __future__ import annotations

from . import ops
from .w4a16 import linear_out  # noqa: F401  (same call shape as upstream's module function)


def fused_residual_rmsnorm(x, residual, weight, eps, fast=False):
    y, residual_out = ops.fused_residual_rmsnorm(x, residual, weight, eps)
    return [y, residual_out]


def _legacy_gemv(x, weight, bias, layout):
    if bias is None:
        raise ValueError("bias must be a tensor; pass an empty tensor for no bias")
    if bias.numel() == 0:
        bias = None  # any dtype, any device: upstream checks neither for an empty tensor
    return ops.decode_linear(x, weight, bias, weight_layout=layout, strict_fp32=True)


def decode_gemv(x, weight, bias, layout):
    return _legacy_gemv(x, weight, bias, layout)


def decode_gemv_warp(x, weight, bias, layout):
    return _legacy_gemv(x, weight, bias, layout)


def decode_gemv_rows(x, weight, bias, layout):
    return _legacy_gemv(x, weight, bias, layout)


def _simt_gemv(x, weight, bias=None, layout="KN"):
    return ops.decode_linear(x, weight, bias, weight_layout=layout, strict_fp32=True)


def decode_gemv_simt_warp(x, weight, bias=None, layout="KN"):
    return _simt_gemv(x, weight, bias, layout)


def decode_gemv_simt_rows(x, weight, bias=None, layout="KN"):
    return _simt_gemv(x, weight, bias, layout)


def decode_gemm_tiled(x, weight, bias=None, layout="KN"):
    return _simt_gemv(x, weight, bias, layout)


def rope_gqa_paged_kv_append(q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache,
                             page_size, rope_dim, interleaved, kv_layout, fused=False):
    return ops.rope_gqa_paged_kv_append(q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache,
                                        page_size=int(page_size), rope_dim=int(rope_dim), interleaved=bool(interleaved),
                                        kv_layout=kv_layout)
