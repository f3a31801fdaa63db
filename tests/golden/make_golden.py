"""Writes the golden fixtures of this folder by running the UPSTREAM Python
references (not this repository's code) on seeded CPU inputs.

Usage (needs a checkout of AmanPandey28/cross_dsl_kernels):

    python tests/golden/make_golden.py /path/to/cross_dsl_kernels

Every fixture is one ``torch.save`` file holding a list of cases; a case is a
dict with the inputs, the keyword arguments and the outputs upstream produced.
The files are small (tens of KB) and committed; the tests read them and never
need the upstream checkout.
"""

from __future__ import annotations

import importlib
import pathlib
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent


def _load(root: pathlib.Path, dotted: str):
    """Import one upstream module from the checkout (its package name,
    ``crossdsl_kernels``, differs from this repository's, so nothing shadows)."""
    src = str(root / "src")
    if src not in sys.path:
        sys.path.insert(0, src)
    return importlib.import_module("crossdsl_kernels." + dotted)


def rmsnorm_cases(up):
    cases = []
    for seed, rows, hidden, dtype, eps in [
        (0, 3, 8, torch.float32, 1e-5),
        (1, 5, 513, torch.float32, 1e-6),
        (2, 4, 1024, torch.float32, 1e-6),
        (3, 2, 4096, torch.float32, 1e-6),
        (4, 3, 8, torch.bfloat16, 1e-5),
        (5, 5, 513, torch.bfloat16, 1e-6),
        (6, 2, 4096, torch.bfloat16, 1e-6),
        (7, 3, 257, torch.float16, 1e-6),
        (8, 1, 1, torch.float32, 1e-6),
    ]:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, hidden, generator=g).to(dtype)
        r = torch.randn(rows, hidden, generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
        y, r_out = up.fused_residual_rmsnorm_reference(x, r, w, eps)
        cases.append(dict(x=x, residual=r, weight=w, eps=eps, y=y, residual_out=r_out))
    # The rounding-order discriminator of upstream tests/unit/test_rmsnorm_bf16.py:21-41:
    # the unrounded FP32 sum is normalised, not its BF16 rounding.
    x = torch.tensor([[1.0, 1.0, 0.0, 0.0]], dtype=torch.bfloat16)
    r = torch.tensor([[2.0 ** -8, -(2.0 ** -8), 0.0, 0.0]], dtype=torch.bfloat16)
    w = torch.ones(4, dtype=torch.bfloat16)
    y, r_out = up.fused_residual_rmsnorm_reference(x, r, w, 1e-6)
    cases.append(dict(x=x, residual=r, weight=w, eps=1e-6, y=y, residual_out=r_out))
    return cases


def gemv_cases(up):
    cases = []
    for seed, m, k, n, layout, use_bias, exact in [
        (0, 1, 64, 48, "KN", False, True),
        (1, 4, 96, 33, "NK", True, True),
        (2, 16, 128, 40, "KN", True, True),
        (3, 3, 513, 67, "KN", True, False),
        (4, 5, 257, 67, "NK", False, False),
        (5, 16, 1024, 96, "NK", True, False),
        (6, 1, 1, 1, "KN", False, False),
    ]:
        g = torch.Generator().manual_seed(seed)
        if exact:
            # small integers: every FP32 partial sum is exact, so the result does
            # not depend on summation order and can be compared bit for bit.
            x = torch.randint(-4, 5, (m, k), generator=g).float()
            w_kn = torch.randint(-4, 5, (k, n), generator=g).float()
            b = torch.randint(-8, 9, (n,), generator=g).float() if use_bias else None
        else:
            x = torch.randn(m, k, generator=g)
            w_kn = torch.randn(k, n, generator=g) / k ** 0.5
            b = 0.02 * torch.randn(n, generator=g) if use_bias else None
        w = w_kn if layout == "KN" else w_kn.t().contiguous()
        y = up.decode_linear_reference(x, w, b, weight_layout=layout)
        cases.append(dict(x=x, weight=w, bias=b, weight_layout=layout, exact=exact, y=y))
    return cases


def rope_cases(up):
    cases = []
    specs = [
        # seed, tokens, hq, hkv, dim, rope_dim, page_size, layout, interleaved, dtype
        (0, 3, 4, 2, 8, 8, 8, "NHD", False, torch.float32),
        (1, 5, 8, 2, 16, 8, 4, "HND", False, torch.float32),
        (2, 5, 8, 2, 16, 16, 4, "NHD", True, torch.float32),
        (3, 4, 4, 4, 66, 22, 7, "HND", True, torch.float32),
        (4, 6, 8, 2, 128, 64, 16, "NHD", False, torch.bfloat16),
        (5, 6, 8, 2, 128, 128, 16, "HND", False, torch.bfloat16),
        (6, 6, 8, 2, 128, 64, 16, "HND", True, torch.float16),
        (7, 16, 32, 8, 128, 64, 16, "NHD", False, torch.float32),
        (8, 16, 32, 8, 128, 128, 16, "HND", False, torch.float32),
    ]
    for seed, tokens, hq, hkv, dim, rd, ps, layout, inter, dtype in specs:
        g = torch.Generator().manual_seed(seed)
        pages_per_seq = 4
        n_pages = tokens * pages_per_seq + 1  # the last page is never mapped
        max_pos = ps * pages_per_seq
        q = torch.randn(tokens, hq, dim, generator=g).to(dtype)
        k = torch.randn(tokens, hkv, dim, generator=g).to(dtype)
        v = torch.randn(tokens, hkv, dim, generator=g).to(dtype)
        positions = torch.randint(0, max_pos, (tokens,), generator=g)
        sequence_ids = torch.arange(tokens)
        page_table = torch.randperm(tokens * pages_per_seq, generator=g).reshape(tokens, pages_per_seq)
        inv_freq = 10000.0 ** (-torch.arange(0, rd, 2).float() / rd)
        angle = torch.arange(max_pos).float()[:, None] * inv_freq[None, :]
        cos, sin = angle.cos(), angle.sin()
        shape = (n_pages, ps, hkv, dim) if layout == "NHD" else (n_pages, hkv, ps, dim)
        k_cache = torch.full(shape, -999.0, dtype=dtype)
        v_cache = torch.full(shape, -999.0, dtype=dtype)
        q_out = up.rope_gqa_paged_kv_append_reference(
            q, k, v, cos, sin, positions, page_table, sequence_ids, k_cache, v_cache,
            page_size=ps, rope_dim=rd, interleaved=inter, kv_layout=layout)
        # Caches are stored sparsely (flat index + value of every element that no
        # longer holds the -999 fill) to keep the fixture small.
        k_idx = (k_cache.view(-1) != -999.0).nonzero().view(-1)
        v_idx = (v_cache.view(-1) != -999.0).nonzero().view(-1)
        cases.append(dict(q=q, k=k, v=v, cos=cos, sin=sin, positions=positions, page_table=page_table,
                          sequence_ids=sequence_ids, page_size=ps, rope_dim=rd, interleaved=inter,
                          kv_layout=layout, q_out=q_out, cache_shape=tuple(shape),
                          k_index=k_idx, k_values=k_cache.view(-1)[k_idx].clone(),
                          v_index=v_idx, v_values=v_cache.view(-1)[v_idx].clone()))
    return cases


def w4a16_cases(quant):
    cases = []
    for seed, m, k, n, group, use_bias in [
        (0, 1, 128, 8, 128, False),
        (1, 4, 256, 24, 32, True),
        (2, 16, 512, 40, 64, True),
        (3, 2, 33, 5, 32, False),
        (4, 3, 257, 9, 256, True),
        (5, 16, 1024, 64, 128, False),
    ]:
        g = torch.Generator().manual_seed(seed)
        codes = torch.randint(0, 16, (n, k), generator=g)
        packed = quant.pack_int4((codes - 8).to(torch.int8))
        groups = -(-k // group)
        scales = (0.005 + 0.015 * torch.rand(n, groups, generator=g)).half()
        x = torch.randn(m, k, generator=g).half()
        b = (0.02 * torch.randn(n, generator=g)).half() if use_bias else None
        y = quant.w4a16_reference(x, packed, scales, b, group_size=group)
        w = quant.dequantize_int4(packed, scales, k, group)
        cases.append(dict(x=x, packed=packed, scales=scales, bias=b, group_size=group,
                          codes=(codes - 8).to(torch.int8), weight=w, y=y))
    # round-to-nearest quantiser output on normal weights (quantization.py:40-62)
    g = torch.Generator().manual_seed(9)
    wt = torch.randn(6, 200, generator=g)
    packed, scales = quant.quantize_int4(wt, 64)
    cases.append(dict(quantize_input=wt, group_size=64, packed=packed, scales=scales,
                      weight=quant.dequantize_int4(packed, scales, 200, 64)))
    return cases


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    root = pathlib.Path(sys.argv[1]).resolve()
    rms = _load(root, "references.rmsnorm")
    gemv = _load(root, "references.gemv")
    _load(root, "references.paged_address")
    rope = _load(root, "references.rope_kv")
    quant = _load(root, "quantization")
    torch.save(rmsnorm_cases(rms), HERE / "rmsnorm.pt")
    torch.save(gemv_cases(gemv), HERE / "gemv.pt")
    torch.save(rope_cases(rope), HERE / "rope_kv.pt")
    torch.save(w4a16_cases(quant), HERE / "w4a16.pt")
    for name in ("rmsnorm", "gemv", "rope_kv", "w4a16"):
        print(name, (HERE / f"{name}.pt").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
