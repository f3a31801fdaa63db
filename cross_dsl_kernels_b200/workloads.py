"""Seeded synthetic inputs for the decode ops and their algorithmic byte counts.

Inputs are drawn on the CPU from ``torch.Generator().manual_seed(seed)`` and
then moved to the device, so a CPU checker and the GPU see identical bits (the
convention of upstream's benchmarks/comparison_cases.py:24-28).  The byte
models are upstream's ``logical_bytes`` (comparison_cases.py:42, 59, 113-117;
benchmarks/rmsnorm_bf16.py:74): every tensor the op must read or write, once.
"""

from __future__ import annotations

import torch

from .quantization import pack_int4


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def rmsnorm_inputs(rows: int, hidden: int, dtype=torch.float32, seed: int = 0):
    """x, residual ~ N(0,1); weight ~ N(1, 0.1); returns CPU tensors."""
    g = _gen(seed)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    r = torch.randn(rows, hidden, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return x, r, w


def rmsnorm_bytes(rows: int, hidden: int, dtype) -> int:
    return torch.empty(0, dtype=dtype).element_size() * (4 * rows * hidden + hidden)


def projection_inputs(m: int, k: int, n: int, layout: str = "KN", bias: bool = True, seed: int = 0):
    """x ~ N(0,1), W ~ N(0, 1/sqrt(K)) stored KN or NK (same values), bias ~ N(0, 0.02)."""
    g = _gen(seed)
    x = torch.randn(m, k, generator=g)
    w = torch.randn(k, n, generator=g) / k ** 0.5
    b = 0.02 * torch.randn(n, generator=g) if bias else None
    if layout == "NK":
        w = w.t().contiguous()
    return x, w, b


def projection_bytes(m: int, k: int, n: int, bias: bool = True) -> int:
    return 4 * (m * k + k * n + m * n + (n if bias else 0))


def rope_inputs(tokens=16, q_heads=32, kv_heads=8, head_dim=128, rope_dim=64, page_size=16, pages=4096,
                max_position=4096, layout="NHD", dtype=torch.float32, theta=10000.0, seed: int = 0):
    """Decode batch with positions uniform in [0, max_position); the block tables
    are rows of ONE random permutation of all pages, so sequences never share a
    page and every token has its own slot.  Caches are not created here."""
    g = _gen(seed)
    pages_per_seq = pages // tokens
    if pages_per_seq * page_size < max_position:
        raise ValueError("not enough pages per sequence for max_position")
    q = torch.randn(tokens, q_heads, head_dim, generator=g).to(dtype)
    k = torch.randn(tokens, kv_heads, head_dim, generator=g).to(dtype)
    v = torch.randn(tokens, kv_heads, head_dim, generator=g).to(dtype)
    positions = torch.randint(0, max_position, (tokens,), generator=g)
    sequence_ids = torch.arange(tokens)
    page_table = torch.randperm(pages, generator=g)[: tokens * pages_per_seq].reshape(tokens, pages_per_seq)
    inv_freq = theta ** (-torch.arange(0, rope_dim, 2).float() / rope_dim)
    angle = torch.arange(max_position).float()[:, None] * inv_freq[None, :]
    shape = (pages, page_size, kv_heads, head_dim) if layout == "NHD" else (pages, kv_heads, page_size, head_dim)
    return dict(q=q, k=k, v=v, cos=angle.cos(), sin=angle.sin(), positions=positions, page_table=page_table,
                sequence_ids=sequence_ids, cache_shape=shape, page_size=page_size, rope_dim=rope_dim, kv_layout=layout)


def rope_bytes(tokens: int, q_heads: int, kv_heads: int, head_dim: int, rope_dim: int, dtype) -> int:
    elt = torch.empty(0, dtype=dtype).element_size()
    return 2 * elt * tokens * head_dim * (q_heads + 2 * kv_heads) + 2 * 4 * tokens * (rope_dim // 2) + 24 * tokens


def w4a16_inputs(m: int, k: int, n: int, group: int = 128, bias: bool = False, seed: int = 0):
    """Codes uniform in [0,15] (zero point 8), FP16 scales uniform in [0.005, 0.02], x ~ N(0,1) FP16."""
    g = _gen(seed)
    codes = torch.randint(0, 16, (n, k), generator=g)
    packed = pack_int4((codes - 8).to(torch.int8))
    scales = (0.005 + 0.015 * torch.rand(n, -(-k // group), generator=g)).half()
    x = torch.randn(m, k, generator=g).half()
    b = (0.02 * torch.randn(n, generator=g)).half() if bias else None
    return x, packed, scales, b


def w4a16_bytes(m: int, k: int, n: int, group: int = 128, bias: bool = False) -> int:
    return n * ((k + 1) // 2) + 2 * n * (-(-k // group)) + 2 * m * k + 2 * m * n + (2 * n if bias else 0)
