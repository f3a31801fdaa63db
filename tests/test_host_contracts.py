"""CPU tests of the host side of the library: the INT4 format helpers, the
paged-address helpers, the set-up validator, tolerances and aliasing guards.
The behaviours pinned here are the ones upstream's unit tests pin for the
same-named functions (tests/unit/test_{quantization,paged_address,
rope_vectorized,tolerances,kernel_contracts}.py)."""

from __future__ import annotations

import math

import pytest
import torch

from conftest import load_golden
from cross_dsl_kernels_b200 import contracts, quantization as qz, tolerances
from cross_dsl_kernels_b200.references import (
    PagedAddress, address_for_token, hnd_linear_index, nhd_linear_index, validate_paged_kv_indices)
from cross_dsl_kernels_b200.w4a16 import w4a16_linear
from cross_dsl_kernels_b200 import ops


def test_pack_unpack_roundtrip_and_golden_bytes():
    q = torch.arange(-8, 8, dtype=torch.int8).reshape(2, 8)
    for k in range(1, 9):
        packed = qz.pack_int4(q[:, :k])
        assert torch.equal(qz.unpack_int4(packed, k), q[:, :k])
        if k % 2:
            assert torch.equal(packed[:, -1] >> 4, torch.full((2,), 8, dtype=torch.uint8))
    assert qz.pack_int4(torch.tensor([[-8, 7, 0]], dtype=torch.int8)).tolist() == [[240, 136]]


def test_group_boundary_dequant():
    q = torch.zeros(1, 33, dtype=torch.int8)
    q[0, 0], q[0, 31], q[0, 32] = -8, 7, 3
    scales = torch.tensor([[0.5, 2]], dtype=torch.float16)
    weight = qz.dequantize_int4(qz.pack_int4(q), scales, 33, 32)
    assert weight[0, [0, 31, 32]].tolist() == [-4, 3.5, 6]
    one = qz.dequantize_int4(qz.pack_int4(torch.tensor([[3]], dtype=torch.int8)), torch.tensor([[0.1]], dtype=torch.float16), 1, 32)
    assert one.item() == (torch.tensor([[0.1]], dtype=torch.float16).float() * 3).half().item()


def test_format_helpers_match_upstream_outputs():
    for case in load_golden("w4a16"):
        if "quantize_input" in case:
            packed, scales = qz.quantize_int4(case["quantize_input"], case["group_size"])
            assert torch.equal(packed, case["packed"]) and torch.equal(scales, case["scales"])
            k = case["quantize_input"].shape[1]
        else:
            k = case["x"].shape[1]
            assert torch.equal(qz.pack_int4(case["codes"]), case["packed"])
            assert torch.equal(qz.unpack_int4(case["packed"], k), case["codes"])
        assert torch.equal(qz.dequantize_int4(case["packed"], case["scales"], k, case["group_size"]), case["weight"])


def test_quantizer_zero_groups_and_error_bound():
    g = torch.Generator().manual_seed(26)
    for group in (32, 64, 128, 256):
        for k in (1, 31, 32, 33, 127, 128, 129, 257):
            w = torch.randn(3, k, generator=g).half()
            w[0].zero_()
            packed, scales = qz.quantize_int4(w, group)
            actual = qz.dequantize_int4(packed, scales, k, group)
            assert torch.equal(actual[0], w[0])
            per_value = scales[:, torch.arange(k) // group].float()
            bound = 0.5 * per_value + actual.float().abs() * 0.001 + 1e-6
            assert bool(((actual.float() - w.float()).abs() <= bound).all())


def test_bad_values_and_groups_are_rejected():
    with pytest.raises(ValueError):
        qz.pack_int4(torch.tensor([[8]], dtype=torch.int8))
    for group in (0, 31, 33, True):
        with pytest.raises(ValueError):
            qz.quantize_int4(torch.ones(1, 2), group)
    for value in (float("nan"), float("inf"), 1e30):
        with pytest.raises(ValueError):
            qz.quantize_int4(torch.tensor([[value]]))


def test_w4a16_metadata_contract_and_alias_guard():
    x = torch.ones(2, 33, dtype=torch.float16)
    packed, scales = qz.quantize_int4(torch.ones(5, 33))
    assert qz.validate_w4a16(x, packed, scales, cuda=False) == (2, 33, 5)
    with pytest.raises(ValueError, match="CUDA"):
        qz.validate_w4a16(x, packed, scales)
    with pytest.raises(ValueError, match="overlap"):
        qz.validate_w4a16(x, packed, scales, out=x.flatten()[:10].view(2, 5), cuda=False)
    with pytest.raises(ValueError, match="contiguous"):
        qz.validate_w4a16(x.t().contiguous().t(), packed, scales, cuda=False)
    with pytest.raises(ValueError, match="forward-only"):
        qz.validate_w4a16(x.clone().requires_grad_(), packed, scales, cuda=False)
    with pytest.raises(ValueError):
        qz.validate_w4a16(torch.ones(17, 33, dtype=torch.float16), packed, scales, cuda=False)
    with pytest.raises(ValueError):
        qz.validate_w4a16(x, packed, scales, torch.ones(4, dtype=torch.float16), cuda=False)


def test_w4a16_linear_refuses_other_backends_and_cpu_tensors():
    x = torch.ones(2, 32, dtype=torch.float16)
    packed, scales = qz.quantize_int4(torch.ones(5, 32))
    for backend in ("reference", "triton", "cute", "other"):
        with pytest.raises(ValueError):
            w4a16_linear(x, packed, scales, backend=backend)
    with pytest.raises(ValueError):
        w4a16_linear(x, packed, scales, rows_per_block=2)
    with pytest.raises(ValueError, match="CUDA"):
        w4a16_linear(x, packed, scales)  # no CPU fallback


def test_ops_refuse_cpu_tensors():
    with pytest.raises(ValueError):
        ops.fused_residual_rmsnorm(torch.ones(2, 8), torch.ones(2, 8), torch.ones(8), 1e-6)
    with pytest.raises(ValueError):
        ops.decode_linear(torch.ones(2, 8), torch.ones(8, 4))


def test_page_boundary_and_errors():
    table = [7, 3, 5]
    assert address_for_token(15, 16, table) == PagedAddress(0, 15, 7)
    assert address_for_token(16, 16, table).logical_page == 1
    assert address_for_token(16, 16, table).physical_page == 3
    assert address_for_token(17, 16, table).offset == 1
    with pytest.raises(ValueError):
        address_for_token(0, 0, [1])
    with pytest.raises(ValueError):
        address_for_token(-1, 16, [1])
    with pytest.raises(IndexError):
        address_for_token(32, 16, [1])
    with pytest.raises(ValueError):
        address_for_token(0, 16, [-1])


def test_layout_flattening():
    assert nhd_linear_index(2, 3, 1, 5, page_size=16, num_heads=4, head_dim=8) == (((2 * 16 + 3) * 4 + 1) * 8) + 5
    assert hnd_linear_index(2, 3, 1, 5, page_size=16, num_heads=4, head_dim=8) == (((2 * 4 + 1) * 16 + 3) * 8) + 5


def test_index_validator():
    ok = dict(page_size=8, num_cache_pages=3, max_position=16)
    validate_paged_kv_indices(torch.tensor([0, 9]), torch.tensor([[0, 1], [2, 0]]), torch.tensor([0, 0]), **ok)
    for positions, table, sequences, message in [
        ([0], [[0]], [1], "sequence"),
        ([-1], [[0]], [0], "position"),
        ([16], [[0]], [0], "position"),
        ([0], [[3]], [0], "physical page"),
        ([0, 0], [[0]], [0, 0], "distinct"),
        ([0, 0], [[0], [0]], [0, 1], "distinct"),
    ]:
        with pytest.raises(ValueError, match=message):
            validate_paged_kv_indices(torch.tensor(positions), torch.tensor(table), torch.tensor(sequences), **ok)


def test_fp32_projection_tolerance_policy():
    assert tolerances.fp32_gemv_tolerance(1024)["max_abs_err"] == pytest.approx(2e-4)
    assert tolerances.fp32_gemv_tolerance(4096)["max_abs_err"] == pytest.approx(4e-4)
    assert tolerances.fp32_gemv_tolerance(16)["max_abs_err"] == pytest.approx(2e-4)
    assert tolerances.fp32_gemv_tolerance(4096)["rel_l2_err"] == 1e-5
    assert tolerances.fp32_gemv_status(4096, 3.9e-4, 9e-6)[0] == "PASS"
    assert tolerances.fp32_gemv_status(4096, 4.1e-4, 9e-6)[0] == "FAIL"
    assert tolerances.fp32_gemv_status(4096, 1e-4, 2e-5)[0] == "FAIL"
    with pytest.raises(ValueError):
        tolerances.fp32_gemv_tolerance(0)
    assert math.isclose(tolerances.fp32_gemv_tolerance(16384)["max_abs_err"], 8e-4)


def test_cache_overlap_guard():
    storage = torch.zeros(64)
    a, b, c = storage[:16], storage[16:32], storage[8:24]
    contracts.validate_cache_storage((torch.zeros(4),), a, b)
    with pytest.raises(ValueError, match="overlap"):
        contracts.validate_cache_storage((torch.zeros(4),), a, c)
    with pytest.raises(ValueError, match="overlap"):
        contracts.validate_cache_storage((storage[20:24],), a, b)
    contracts.validate_cache_storage((storage[:0],), a, b)  # empty tensors never overlap


def test_cache_overlap_guard_sees_the_whole_span_of_a_strided_input():
    # q is a column slice of a fused [tokens, 96] QKV matrix: 4 rows of 32 elements, 96 apart.  Its numel
    # (128) covers only the first row and a third; a cache placed over the LAST row must still be refused.
    from cross_dsl_kernels_b200 import contracts
    storage = torch.zeros(4 * 96 + 64)
    qkv = storage[: 4 * 96].view(4, 96)
    q = qkv[:, :32].view(4, 2, 16)
    assert not q.is_contiguous()
    cache_on_last_row = storage[3 * 96: 3 * 96 + 16]
    elsewhere = storage[4 * 96: 4 * 96 + 16]
    other = torch.zeros(16)
    with pytest.raises(ValueError, match="overlap"):
        contracts.validate_cache_storage((q,), cache_on_last_row, other)
    contracts.validate_cache_storage((q,), elsewhere, other)
