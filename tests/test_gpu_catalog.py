"""Upstream's own shape catalogs run through this library's kernels, case by case (by upstream's names).

Each case is built the way upstream's benchmarks/comparison_cases.py:24-125 builds it (seeded CPU draws, FP64 or
CPU-reference expectation, caches full of the sentinel -999, three reversed pages per request) and then goes
through the discipline of benchmarks/compare.py:28-41, 247-258 and benchmarks/gemv_cuda_benchmark.py:97-126:
gate the eager result, capture a CUDA graph, replay it over poisoned outputs and gate again, change the inputs in
place at their fixed addresses, replay and gate against the recomputed expectation."""

from __future__ import annotations

import json

import pytest
import torch

from conftest import GOLDEN, rel_l2
from cross_dsl_kernels_b200.tolerances import fp32_gemv_tolerance
from oracle import decode_ops, int4

pytestmark = pytest.mark.gpu

CATALOG = json.loads((GOLDEN / "shape_catalog.json").read_text())
FP32 = list(enumerate(CATALOG["fp32"]))
W4 = list(enumerate(CATALOG["w4a16"]))


def replay_discipline(call, outputs_of, expectation, mutate):
    """call() -> result; outputs_of(result) -> tensors to poison; expectation(changed) checks a result."""
    from cross_dsl_kernels_b200.timing import capture

    expectation(call(), False)
    captured = []
    graph = capture([call], outputs=captured)
    for t in outputs_of(captured[0]):
        t.fill_(float("nan")) if t.is_floating_point() else None
    graph.replay()
    torch.cuda.synchronize()
    expectation(captured[0], False)
    mutate()
    for t in outputs_of(captured[0]):
        t.fill_(float("nan")) if t.is_floating_point() else None
    graph.replay()
    torch.cuda.synchronize()
    expectation(captured[0], True)


@pytest.mark.parametrize("index,spec", FP32, ids=[s["name"] for _, s in FP32])
def test_fp32_catalog_case(index, spec):
    from cross_dsl_kernels_b200.ops import decode_linear, fused_residual_rmsnorm, rope_gqa_paged_kv_append
    gen = torch.Generator().manual_seed(CATALOG["base_seed"] + index)
    rand = lambda *shape: torch.randn(*shape, generator=gen, dtype=torch.float32)
    if spec["op"] == "rmsnorm":
        rows, hidden = spec["rows"], spec["hidden"]
        x, residual, weight = rand(rows, hidden), rand(rows, hidden), rand(hidden)
        xd, rd, wd = x.cuda(), residual.cuda(), weight.cuda()

        def expect(out, changed):
            xin = xd.cpu()
            r = xin + residual
            inv = torch.rsqrt(r.double().square().mean(-1, keepdim=True) + 1e-5)
            want = (r.double() * inv * weight.double()).float()
            assert torch.equal(out[1].cpu(), r)                                  # residual_out exact
            assert float((out[0].cpu() - want).abs().max()) <= 2e-5 and rel_l2(out[0].cpu(), want) <= 1e-5

        replay_discipline(lambda: fused_residual_rmsnorm(xd, rd, wd, 1e-5), lambda o: o, expect,
                          lambda: xd.mul_(0.5).add_(0.125))
    elif spec["op"] == "gemv":
        m, k, n = spec["m"], spec["k"], spec["n"]
        x, w_kn = rand(m, k), rand(k, n)
        weight = w_kn.t().contiguous() if spec["layout"] == "NK" else w_kn
        bias = rand(n) if spec["bias"] else None
        xd, wd, bd = x.cuda(), weight.cuda(), (bias.cuda() if bias is not None else None)
        tol = fp32_gemv_tolerance(k)

        def expect(out, changed):
            want = xd.cpu().double() @ w_kn.double()
            if bd is not None:
                want = want + bd.cpu().double()
            assert float((out.cpu().double() - want).abs().max()) <= tol["max_abs_err"] * max(1.0, float(want.abs().max()) / 64)
            assert rel_l2(out.cpu(), want) <= tol["rel_l2_err"]

        def mutate():
            xd.mul_(0.5).add_(0.125)
            if bd is not None:
                bd.add_(0.25)

        replay_discipline(lambda: decode_linear(xd, wd, bd, weight_layout=spec["layout"]), lambda o: [o], expect, mutate)
    else:
        tokens, hq, hkv, dim, ps = (spec[key] for key in ("tokens", "q_heads", "kv_heads", "head_dim", "page_size"))
        positions = torch.tensor([ps - 1 + i % 3 for i in range(tokens)])
        sequences = torch.arange(tokens)
        table = torch.arange(tokens * 3).flip(0).reshape(tokens, 3).contiguous()
        trig = rand(ps * 3, spec["rope_dim"] // 2)
        q, k, v = rand(tokens, hq, dim), rand(tokens, hkv, dim), rand(tokens, hkv, dim)
        shape = (tokens * 3 + 1, ps, hkv, dim) if spec["layout"] == "NHD" else (tokens * 3 + 1, hkv, ps, dim)
        kw = dict(page_size=ps, rope_dim=spec["rope_dim"], interleaved=spec["interleaved"], kv_layout=spec["layout"])
        decode_ops.check_paged_indices(positions, table, sequences, page_size=ps, num_cache_pages=shape[0], max_position=trig.shape[0])
        dev = [t.cuda() for t in (q, k, v, trig.cos(), trig.sin(), positions, table, sequences)]
        kc, vc = torch.full(shape, -999.0).cuda(), torch.full(shape, -999.0).cuda()

        def call():
            return rope_gqa_paged_kv_append(*dev, kc, vc, **kw), kc, vc

        def expect(out, changed):
            ck, cv = torch.full(shape, -999.0), torch.full(shape, -999.0)
            want_q = decode_ops.rope_paged_append(dev[0].cpu(), dev[1].cpu(), dev[2].cpu(), trig.cos(), trig.sin(), positions,
                                                  table, sequences, ck, cv, **kw)
            assert torch.equal(out[0].cpu(), want_q)
            assert torch.equal(kc.cpu(), ck) and torch.equal(vc.cpu(), cv)       # written slots AND untouched sentinels

        def mutate():
            for t in dev[:3]:
                t.mul_(0.5).add_(0.125)
            kc.fill_(-999.0)
            vc.fill_(-999.0)

        replay_discipline(call, lambda o: [o[0]], expect, mutate)


@pytest.mark.parametrize("index,spec", W4, ids=[s["name"] for _, s in W4])
def test_w4a16_catalog_case(index, spec):
    from cross_dsl_kernels_b200 import quantization as qz
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    m, k, n, group = (spec[key] for key in ("m", "k", "n", "group_size"))
    gen = torch.Generator().manual_seed(CATALOG["base_seed"] + index)
    x = torch.randn(m, k, generator=gen).half()
    original = torch.randn(n, k, generator=gen).half()
    if spec.get("zero"):
        original.zero_()
    bias = torch.randn(n, generator=gen).half() if spec["bias"] else None
    packed, scales = qz.quantize_int4(original, group)
    xd, pd, sd, bd = x.cuda(), packed.cuda(), scales.cuda(), (bias.cuda() if bias is not None else None)

    def expect(out, changed):
        want = int4.w4a16_projection(xd.cpu(), packed, scales, bd.cpu() if bd is not None else None, group_size=group).double()
        got = out.cpu().double()
        assert bool(((got - want).abs() <= 0.002 + 0.002 * want.abs()).all())
        assert float((got - want).norm()) <= 1e-3 * max(float(want.norm()), 1e-12) or float((got - want).abs().max()) == 0.0

    def mutate():
        xd.mul_(0.5).add_(0.125)
        if bd is not None:
            bd.add_(0.25)

    replay_discipline(lambda: w4a16_linear(xd, pd, sd, bd, group_size=group), lambda o: [o], expect, mutate)
