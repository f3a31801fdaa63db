"""Pins the CPU oracle (oracle/) to outputs of the upstream Python references
(fixtures in tests/golden, produced by tests/golden/make_golden.py) and to the
known-answer vectors upstream's own unit tests hold."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import load_golden, rebuild_cache
from oracle import decode_ops, int4, paging


def test_rmsnorm_matches_upstream():
    for case in load_golden("rmsnorm"):
        y, r = decode_ops.residual_rmsnorm(case["x"], case["residual"], case["weight"], case["eps"])
        assert torch.equal(r, case["residual_out"])
        # the row mean is a reduction whose order may differ between CPUs: compare y closely, not bitwise
        torch.testing.assert_close(y.float(), case["y"].float(), rtol=2e-6 if y.dtype == torch.float32 else 1e-2, atol=1e-7)


def test_rmsnorm_normalises_the_unrounded_sum():
    # upstream tests/unit/test_rmsnorm_bf16.py:21-41: rounding the sum to BF16 first gives a different y
    case = load_golden("rmsnorm")[-1]
    x, r, w = case["x"], case["residual"], case["weight"]
    y, _ = decode_ops.residual_rmsnorm(x, r, w, case["eps"])
    assert torch.equal(y, case["y"])
    rounded_first = (x.float() + r.float()).bfloat16().float()
    y_wrong = (rounded_first * torch.rsqrt((rounded_first ** 2).mean(-1, keepdim=True) + case["eps"])).bfloat16()
    assert not torch.equal(y, y_wrong)


def test_projection_matches_upstream():
    for case in load_golden("gemv"):
        y = decode_ops.decode_projection(case["x"], case["weight"], case["bias"], weight_layout=case["weight_layout"])
        if case["exact"]:
            assert torch.equal(y, case["y"])
        else:
            torch.testing.assert_close(y, case["y"], rtol=1e-5, atol=1e-6)


def test_projection_known_answer_and_rejections():
    # upstream tests/unit/test_gemv_cuda_benchmark.py:60-69
    x = torch.tensor([[1.0, 2.0], [-1.0, 3.0]])
    w = torch.tensor([[1.0, -2.0, 3.0], [4.0, 5.0, -6.0]])
    b = torch.tensor([0.5, 1.0, -2.0])
    assert decode_ops.decode_projection(x, w, b).tolist() == [[9.5, 9.0, -11.0], [11.5, 18.0, -23.0]]
    assert decode_ops.decode_projection(x, w.t().contiguous(), b, weight_layout="NK").tolist() == [[9.5, 9.0, -11.0], [11.5, 18.0, -23.0]]
    with pytest.raises(ValueError, match="K dimension"):
        decode_ops.decode_projection(torch.randn(2, 5), torch.randn(6, 7))
    with pytest.raises(ValueError):
        decode_ops.decode_projection(x, w, weight_layout="XY")
    with pytest.raises(ValueError):
        decode_ops.decode_projection(x, w, torch.zeros(2))


def test_split_k_bounds_cover_k_once():
    for k in (1, 31, 32, 33, 513, 4096, 4100):
        for s in (1, 2, 4, 8):
            bounds = decode_ops.split_k_bounds(k, s)
            assert bounds[0][0] == 0 and bounds[-1][1] == k
            assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
            assert all((hi - lo) % 32 == 0 for lo, hi in bounds[:-1] if hi < k)
    assert decode_ops.split_k_bounds(4096, 4) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]


def _run_rope(fn, case):
    k_cache = torch.full(case["cache_shape"], -999.0, dtype=case["k"].dtype)
    v_cache = torch.full(case["cache_shape"], -999.0, dtype=case["k"].dtype)
    q_out = fn(case["q"], case["k"], case["v"], case["cos"], case["sin"], case["positions"], case["page_table"],
               case["sequence_ids"], k_cache, v_cache, page_size=case["page_size"], rope_dim=case["rope_dim"],
               interleaved=case["interleaved"], kv_layout=case["kv_layout"])
    return q_out, k_cache, v_cache


@pytest.mark.parametrize("fn", [decode_ops.rope_paged_append, decode_ops.rope_paged_append_flat])
def test_rope_append_matches_upstream_bit_for_bit(fn):
    for case in load_golden("rope_kv"):
        q_out, k_cache, v_cache = _run_rope(fn, case)
        assert torch.equal(q_out, case["q_out"])
        assert torch.equal(k_cache, rebuild_cache(case, "k"))
        assert torch.equal(v_cache, rebuild_cache(case, "v"))


def test_rope_slot_map_known_answer():
    # upstream tests/unit/test_references.py:50-91
    tokens, hq, hkv, dim = 3, 4, 2, 8
    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn(tokens, h, dim, generator=g) for h in (hq, hkv, hkv))
    positions = torch.tensor([0, 7, 8])
    table = torch.tensor([[2, 0], [1, 3]])
    seqs = torch.tensor([0, 0, 1])
    theta = torch.arange(16.0).unsqueeze(1) / 100.0
    freqs = torch.arange(dim // 2).float().unsqueeze(0) + 1.0
    k_cache = torch.full((4, 8, hkv, dim), -999.0)
    v_cache = torch.full((4, 8, hkv, dim), -999.0)
    q_out = decode_ops.rope_paged_append(q, k, v, torch.cos(theta * freqs), torch.sin(theta * freqs), positions, table,
                                         seqs, k_cache, v_cache, page_size=8, rope_dim=dim, interleaved=False)
    assert q_out.shape == q.shape
    assert torch.all(k_cache[1] == -999.0) and torch.all(v_cache[1] == -999.0)
    assert torch.equal(v_cache[2, 0], v[0]) and torch.equal(v_cache[2, 7], v[1]) and torch.equal(v_cache[3, 0], v[2])


def test_paging_known_answers():
    # upstream tests/unit/test_paged_address.py:13-39
    table = np.array([[7, 3, 5]])
    page, off = paging.translate([15, 16, 17], [0, 0, 0], table, 16)
    assert page.tolist() == [7, 3, 3] and off.tolist() == [15, 0, 1]
    with pytest.raises(ValueError):
        paging.translate([0], [0], [[1]], 0)
    with pytest.raises(ValueError):
        paging.translate([-1], [0], [[1]], 16)
    with pytest.raises(IndexError):
        paging.translate([32], [0], [[1]], 16)
    with pytest.raises(ValueError):
        paging.translate([0], [0], [[-1]], 16)
    assert paging.flat_index("NHD", 2, 3, 1, 5, page_size=16, num_heads=4, head_dim=8) == (((2 * 16 + 3) * 4 + 1) * 8) + 5
    assert paging.flat_index("HND", 2, 3, 1, 5, page_size=16, num_heads=4, head_dim=8) == (((2 * 4 + 1) * 16 + 3) * 8) + 5


def test_index_validator_rejections():
    # upstream tests/unit/test_rope_vectorized.py:49-87
    ok = dict(page_size=4, num_cache_pages=4, max_position=8)
    table = [[0, 1], [2, 3]]
    decode_ops.check_paged_indices([0, 5], table, [0, 1], **ok)
    for positions, seqs in (([0, 5], [0, 2]), ([0, 8], [0, 1]), ([-1, 5], [0, 1]), ([1, 1], [0, 0])):
        with pytest.raises(ValueError):
            decode_ops.check_paged_indices(positions, table, seqs, **ok)
    with pytest.raises(ValueError):
        decode_ops.check_paged_indices([0], [[9]], [0], **ok)


def test_int4_known_answers():
    # upstream tests/unit/test_quantization.py:16-46, 63-67
    q = np.arange(-8, 8, dtype=np.int8).reshape(2, 8)
    for k in range(1, 9):
        packed = int4.codes_to_bytes(q[:, :k])
        assert (int4.bytes_to_codes(packed, k) == q[:, :k]).all()
        if k % 2:
            assert (packed[:, -1] >> 4 == 8).all()
    assert int4.codes_to_bytes(np.array([[-8, 7, 0]], dtype=np.int8)).tolist() == [[240, 136]]
    q = np.zeros((1, 33), dtype=np.int8)
    q[0, 0], q[0, 31], q[0, 32] = -8, 7, 3
    scales = torch.tensor([[0.5, 2]], dtype=torch.float16)
    packed = torch.from_numpy(int4.codes_to_bytes(q))
    weight = int4.dequantize(packed, scales, 33, 32)
    assert weight[0, [0, 31, 32]].tolist() == [-4, 3.5, 6]
    y = int4.w4a16_projection(torch.ones(1, 33, dtype=torch.float16), packed, scales, torch.tensor([1], dtype=torch.float16), group_size=32)
    assert y.item() == 6.5
    one = int4.dequantize(torch.from_numpy(int4.codes_to_bytes(np.array([[3]], dtype=np.int8))), torch.tensor([[0.1]], dtype=torch.float16), 1, 32)
    assert one.item() == (torch.tensor(0.1, dtype=torch.float16).float() * 3).half().item()


def test_w4a16_matches_upstream():
    for case in load_golden("w4a16"):
        if "quantize_input" in case:
            continue
        k = case["x"].shape[1]
        assert (int4.bytes_to_codes(case["packed"].numpy(), k) == case["codes"].numpy()).all()
        assert torch.equal(int4.dequantize(case["packed"], case["scales"], k, case["group_size"]), case["weight"])
        y = int4.w4a16_projection(case["x"], case["packed"], case["scales"], case["bias"], group_size=case["group_size"])
        assert torch.equal(y, case["y"])
