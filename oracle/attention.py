"""CPU restatement of the two ops that follow the path in a decoder layer: paged decode attention and SwiGLU.

TEST INFRASTRUCTURE (tests, smoke and the benchmark's checker only).  **Parity unpinned**: upstream has neither op
(its chain stops at the K/V append and at the up+gate projection), so there is no upstream function, test or golden
vector to pin these against; they restate the textbook formulas in FP32 on top of upstream's cache layouts
(src/crossdsl_kernels/references/paged_address.py:32-56) and the oracle's own address translation (paging.py).
"""

from __future__ import annotations

import torch

from . import paging


def paged_decode_attention(q, k_cache, v_cache, positions, page_table, sequence_ids, *, page_size: int,
                           kv_layout: str = "NHD", scale=None):
    """out[t, h] = softmax_j(scale * q[t, h] . K[j, h // G]) @ V[j, h // G] over j = 0 .. positions[t], in FP32,
    rounded to q's dtype.  The token's own K/V are expected in the cache (the append runs first)."""
    tokens, q_heads, dim = q.shape
    layout = kv_layout.upper()
    kv_heads = k_cache.shape[2] if layout == "NHD" else k_cache.shape[1]
    group = q_heads // kv_heads
    scale = dim ** -0.5 if scale is None else scale
    out = torch.empty_like(q)
    for t in range(tokens):
        ctx = int(positions[t]) + 1
        js = torch.arange(ctx)
        pages, offs = paging.translate(js.numpy(), sequence_ids[t].repeat(ctx).numpy(), page_table.numpy(), page_size)
        pages, offs = torch.from_numpy(pages), torch.from_numpy(offs)
        if layout == "NHD":
            k, v = k_cache[pages, offs], v_cache[pages, offs]          # [ctx, kv_heads, dim]
        else:
            k, v = k_cache[pages, :, offs], v_cache[pages, :, offs]
        k, v = k.float(), v.float()
        for h in range(q_heads):
            scores = (k[:, h // group] @ q[t, h].float()) * scale
            p = torch.softmax(scores, dim=0)
            out[t, h] = (p @ v[:, h // group]).to(q.dtype)
    return out


def swiglu(upgate: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for [rows, 2 * width] laid out [up | gate]; FP32 arithmetic, one rounding."""
    width = upgate.shape[1] // 2
    up, gate = upgate[:, :width].float(), upgate[:, width:].float()
    return (gate / (1 + torch.exp(-gate)) * up).to(upgate.dtype)
