"""GPU tests of ``cross_dsl_kernels_b200.compat``: the call shapes of upstream's native modules
(csrc/*/*_ext.cpp) and the rejection list of scripts/verify_gemv_simt.py:95-114."""

from __future__ import annotations

import pytest
import torch

from conftest import rel_l2
from oracle import decode_ops, int4

pytestmark = pytest.mark.gpu


def test_rmsnorm_returns_a_list_of_two_tensors():
    from cross_dsl_kernels_b200 import compat
    g = torch.Generator().manual_seed(1)
    x, r = torch.randn(5, 513, generator=g), torch.randn(5, 513, generator=g)
    w = 1 + 0.1 * torch.randn(513, generator=g)
    for fast in (False, True):
        out = compat.fused_residual_rmsnorm(x.cuda(), r.cuda(), w.cuda(), 1e-5, fast)
        assert isinstance(out, list) and len(out) == 2
        want_y, want_r = decode_ops.residual_rmsnorm(x, r, w, 1e-5)
        assert torch.equal(out[1].cpu(), want_r)
        assert rel_l2(out[0].cpu(), want_y) <= 1e-5


@pytest.mark.parametrize("name", ["decode_gemv", "decode_gemv_warp", "decode_gemv_rows"])
@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_legacy_projection_takes_an_empty_tensor_of_any_dtype_as_no_bias(name, layout):
    from cross_dsl_kernels_b200 import compat
    g = torch.Generator().manual_seed(2)
    x, w_kn, b = torch.randn(3, 257, generator=g), torch.randn(257, 67, generator=g) / 16, torch.randn(67, generator=g)
    w = w_kn if layout == "KN" else w_kn.t().contiguous()
    fn = getattr(compat, name)
    want = x.double() @ w_kn.double()
    for empty in (torch.empty(0, device="cuda"), torch.empty(0, device="cuda", dtype=torch.float16),
                  torch.empty(0, device="cuda", dtype=torch.int64), torch.empty(0)):
        y = fn(x.cuda(), w.cuda(), empty, layout)
        assert rel_l2(y.cpu(), want) <= 1e-5
    y = fn(x.cuda(), w.cuda(), b.cuda(), layout)
    assert rel_l2(y.cpu(), want + b.double()) <= 1e-5


@pytest.mark.parametrize("name", ["decode_gemv_simt_warp", "decode_gemv_simt_rows", "decode_gemm_tiled"])
def test_simt_projection_entry_points_and_their_rejections(name):
    from cross_dsl_kernels_b200 import compat
    fn = getattr(compat, name)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3, 7, generator=g).cuda()
    weight = torch.randn(7, 5, generator=g).cuda()
    bias = torch.randn(5, generator=g).cuda()
    want = x.cpu().double() @ weight.cpu().double()
    assert rel_l2(fn(x, weight).cpu(), want) <= 1e-5                     # defaults: no bias, KN
    assert rel_l2(fn(x, weight, bias).cpu(), want + bias.cpu().double()) <= 1e-5
    assert rel_l2(fn(x, weight.t().contiguous(), None, "NK").cpu(), want) <= 1e-5
    invalid = {
        "x_dtype": (x.half(), weight, bias, "KN"),
        "weight_dtype": (x, weight.half(), bias, "KN"),
        "bias_dtype": (x, weight, bias.half(), "KN"),
        "x_rank": (x.flatten(), weight, bias, "KN"),
        "weight_rank": (x, weight.flatten(), bias, "KN"),
        "k_mismatch": (x, weight[:6].contiguous(), bias, "KN"),
        "layout": (x, weight, bias, "invalid"),
        "x_strided": (torch.randn(3, 14, device="cuda")[:, ::2], weight, bias, "KN"),
        "weight_strided": (x, torch.randn(7, 10, device="cuda")[:, ::2], bias, "KN"),
        "bias_strided": (x, weight, torch.randn(10, device="cuda")[::2], "KN"),
        "bias_shape": (x, weight, bias[:4], "KN"),
        "empty_bias": (x, weight, bias[:0], "KN"),
        "zero_m": (x[:0], weight, bias, "KN"),
        "zero_k": (x[:, :0], weight[:0], bias, "KN"),
        "zero_n": (x, weight[:, :0], None, "KN"),
        "x_cpu": (x.cpu(), weight, bias, "KN"),
        "weight_cpu": (x, weight.cpu(), bias, "KN"),
        "bias_cpu": (x, weight, bias.cpu(), "KN"),
    }
    for label, args in invalid.items():
        with pytest.raises((ValueError, RuntimeError)):
            fn(*args)
            pytest.fail(f"{label} was accepted")


def test_rope_positional_call_with_the_fused_switch():
    from cross_dsl_kernels_b200 import compat
    g = torch.Generator().manual_seed(4)
    tokens, hq, hkv, dim, rd, ps = 3, 4, 2, 66, 34, 7
    q, k, v = (torch.randn(tokens, h, dim, generator=g) for h in (hq, hkv, hkv))
    pos, seq = torch.tensor([0, 7, 8]), torch.tensor([0, 0, 1])
    table = torch.tensor([[2, 0], [1, 3]])
    angle = torch.arange(16.0)[:, None] * (10000.0 ** (-torch.arange(0, rd, 2).float() / rd))[None, :]
    for layout in ("NHD", "HND"):
        shape = (4, ps, hkv, dim) if layout == "NHD" else (4, hkv, ps, dim)
        kc, vc = torch.full(shape, -999.0), torch.full(shape, -999.0)
        want = decode_ops.rope_paged_append(q, k, v, angle.cos(), angle.sin(), pos, table, seq, kc, vc, page_size=ps,
                                            rope_dim=rd, interleaved=True, kv_layout=layout)
        for fused in (False, True):
            kd, vd = torch.full(shape, -999.0).cuda(), torch.full(shape, -999.0).cuda()
            got = compat.rope_gqa_paged_kv_append(q.cuda(), k.cuda(), v.cuda(), angle.cos().cuda(), angle.sin().cuda(),
                                                  pos.cuda(), table.cuda(), seq.cuda(), kd, vd, ps, rd, True, layout, fused)
            assert torch.equal(got.cpu(), want) and torch.equal(kd.cpu(), kc) and torch.equal(vd.cpu(), vc)


def test_w4a16_linear_out_writes_the_callers_tensor():
    from cross_dsl_kernels_b200 import compat, quantization as qz
    g = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 16, (96, 512), generator=g)
    packed = qz.pack_int4((codes - 8).to(torch.int8))
    scales = (0.005 + 0.015 * torch.rand(96, 4, generator=g)).half()
    x = torch.randn(4, 512, generator=g).half()
    y = torch.full((4, 96), float("nan"), dtype=torch.float16, device="cuda")
    assert compat.linear_out(x.cuda(), packed.cuda(), scales.cuda(), scales.cuda(), y, 128, 4, False) is None
    ref = int4.w4a16_projection(x, packed, scales, None, group_size=128)
    assert bool(((y.cpu().double() - ref.double()).abs() <= 0.002 + 0.002 * ref.double().abs()).all())
