"""GPU parity of the W4A16 projection.  Gates: |err| <= 0.002 + 0.002 |ref| and
rel-L2 <= 1e-3 against the FP64 product with the FP16-rounded dequantised
weights (upstream benchmarks/w4a16_benchmark.py:33-57), and relative error
<= 2e-3 against the dequantised FP32 matmul."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, rel_l2
from cross_dsl_kernels_b200 import quantization as qz
from oracle import int4

pytestmark = pytest.mark.gpu


def gate(y, x, packed, scales, bias, group):
    ref = int4.w4a16_projection(x, packed, scales, bias, group_size=group)
    err = (y.cpu().double() - ref.double()).abs()
    assert bool((err <= 0.002 + 0.002 * ref.double().abs()).all()), float(err.max())
    assert rel_l2(y.cpu(), ref) <= 1e-3
    dense = int4.w4a16_projection_f32(x, packed, scales, bias, group_size=group)
    assert rel_l2(y.cpu(), dense) <= 2e-3
    return rel_l2(y.cpu(), ref)


def make(m, k, n, group, bias, seed=0):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 16, (n, k), generator=g)
    packed = qz.pack_int4((codes - 8).to(torch.int8))
    scales = (0.005 + 0.015 * torch.rand(n, -(-k // group), generator=g)).half()
    x = torch.randn(m, k, generator=g).half()
    b = (0.02 * torch.randn(n, generator=g)).half() if bias else None
    return x, packed, scales, b


def test_golden_cases():
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    for case in load_golden("w4a16"):
        if "quantize_input" in case:
            continue
        b = case["bias"].cuda() if case["bias"] is not None else None
        y = w4a16_linear(case["x"].cuda(), case["packed"].cuda(), case["scales"].cuda(), b, group_size=case["group_size"])
        err = (y.cpu().double() - case["y"].double()).abs()
        assert bool((err <= 0.002 + 0.002 * case["y"].double().abs()).all())
        assert rel_l2(y.cpu(), case["y"]) <= 1e-3


@pytest.mark.parametrize("m", [1, 16])
@pytest.mark.parametrize("n", [4096, 14336])
def test_baseline_shapes(m, n):
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, _ = make(m, 4096, n, 128, False)
    y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), None, group_size=128)
    worst = gate(y, x, packed, scales, None, 128)
    assert worst <= 3e-4, "FP32 accumulation should land far inside the gate"
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    y2 = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), None, group_size=128, out=out)
    assert y2 is out and torch.equal(y2, y)


@pytest.mark.parametrize("m,k,n,group", [(2, 4096, 4096, 128), (5, 4096, 6144, 64), (8, 4096, 1000, 128), (3, 14336, 520, 128),
                                         (8, 2048, 4100, 32), (1, 4096, 14336, 128), (1, 1024, 24, 256), (4, 4096, 28672 + 8, 128),
                                         (5, 14336, 4096, 128), (7, 3072, 4752 * 2, 64)])
def test_direct_load_tensor_core_kernel(m, k, n, group):
    """M <= 8, K % 1024 == 0: 16 weight columns are the rows of mma.m16n8k16 tiles, the rows of x its columns; eight
    warps split K and walk double-buffered batches.  Ragged N (a last pass that reads clamped columns), more column
    groups than resident CTAs (several passes per CTA), several rounds of loads per pass (K = 14336, with a last
    round of two chunks; K = 3072 with three), one CTA per SM when x is large, bias, all groups."""
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, b = make(m, k, n, group, True, seed=m + n)
    y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), b.cuda(), group_size=group)
    gate(y, x, packed, scales, b, group)
    assert torch.equal(y, w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), b.cuda(), group_size=group)), "deterministic"
    # the same rows inside a taller batch give the same values (while the taller x still fits the kernel's shared memory)
    tall = torch.cat([x, torch.randn(8 - m, k).half()]) if m < 8 and 8 * (2 * k + 16) <= 160 * 1024 else None
    if tall is not None:
        assert torch.equal(w4a16_linear(tall.cuda(), packed.cuda(), scales.cuda(), b.cuda(), group_size=group)[:m], y)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 16])
@pytest.mark.parametrize("group", [32, 64, 128, 256])
def test_every_m_and_group(m, group):
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, b = make(m, 1024, 200, group, True, seed=m * 10 + group)
    y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), b.cuda(), group_size=group)
    gate(y, x, packed, scales, b, group)


@pytest.mark.parametrize("m,k,n", [(1, 33, 5), (2, 1, 1), (3, 257, 9), (16, 31, 7), (4, 96, 17), (16, 6144, 64),
                                   (1, 128, 8), (16, 4096, 6144), (5, 2048, 1001)])
def test_odd_shapes(m, k, n):
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, b = make(m, k, n, 32, True, seed=k)
    y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), b.cuda(), group_size=32)
    gate(y, x, packed, scales, b, 32)


def test_all_sixteen_codes_with_exact_scales():
    """Every code value with power-of-two scales: products and sums are exact, so
    the result must equal the oracle bit for bit (upstream scripts/verify_w4a16.py:30-43)."""
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    n, k = 32, 256
    codes = (torch.arange(n * k).reshape(n, k) % 16).to(torch.int8) - 8
    packed = qz.pack_int4(codes)
    scales = torch.tensor([0.5, 0.25]).repeat(n, 1).half()
    x = (torch.arange(k) % 5 - 2).float().repeat(3, 1).half()
    y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), None, group_size=128)
    assert torch.equal(y.cpu(), int4.w4a16_projection(x, packed, scales, None, group_size=128))


def test_graph_replay_follows_changed_inputs():
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, b = make(16, 1024, 512, 128, True)
    xd, pd, sd, bd = x.cuda(), packed.cuda(), scales.cuda(), b.cuda()
    out = torch.empty(16, 512, dtype=torch.float16, device="cuda")
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        w4a16_linear(xd, pd, sd, bd, out=out)
    side.synchronize()
    gate(out, x, packed, scales, b, 128)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w4a16_linear(xd, pd, sd, bd, out=out)
    x2 = torch.randn(16, 1024, generator=torch.Generator().manual_seed(3)).half()
    xd.copy_(x2); out.fill_(float("nan"))
    graph.replay(); torch.cuda.synchronize()
    gate(out, x2, packed, scales, b, 128)


def test_rejections():
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    x, packed, scales, b = (t.cuda() for t in make(2, 64, 8, 32, True))
    bad = [
        lambda: w4a16_linear(x, packed, scales, b, group_size=48),
        lambda: w4a16_linear(x.float(), packed, scales, b, group_size=32),
        lambda: w4a16_linear(x, packed[:, :16].contiguous(), scales, b, group_size=32),
        lambda: w4a16_linear(x, packed, scales[:, :1].contiguous(), b, group_size=32),
        lambda: w4a16_linear(x, packed, scales, b[:4], group_size=32),
        lambda: w4a16_linear(x, packed, scales, b, group_size=32, out=torch.empty(2, 9, dtype=torch.float16, device="cuda")),
        lambda: w4a16_linear(x, packed, scales, b, group_size=32, out=x.view(-1)[:16].view(2, 8)),
        lambda: w4a16_linear(torch.zeros(17, 64, dtype=torch.float16, device="cuda"), packed, scales, b, group_size=32),
        lambda: w4a16_linear(x, packed, scales, b, group_size=32, rows_per_block=3),
        lambda: w4a16_linear(x.cpu(), packed, scales, b, group_size=32),
    ]
    for call in bad:
        with pytest.raises((ValueError, RuntimeError)):
            call()


@pytest.mark.parametrize("force", ["1", "0"])
def test_both_m16_paths_match_oracle_in_a_fresh_process(force):
    """The library picks the tcgen05 kernel for wide projections and the mma.sync kernel for narrow ones;
    XDK_W4A16_UMMA (read once per process) forces one of them, so each is checked over the same narrow,
    ragged and wide shapes in a child process.  For the tcgen05 kernel this covers the TMEM-resident A
    operand, the UMMA descriptors of x, the four accumulators and full, ragged and multiple strips."""
    import os
    import subprocess
    import sys
    import textwrap
    from conftest import ROOT
    code = textwrap.dedent("""
        import sys, torch
        sys.path.insert(0, %r)
        from cross_dsl_kernels_b200 import workloads as wl
        from cross_dsl_kernels_b200.w4a16 import w4a16_linear
        from oracle import int4
        for (m, k, n, g, bias) in [(16, 256, 8, 128, False), (9, 1024, 200, 64, True), (16, 4096, 4096, 128, False),
                                   (12, 2048, 1001 * 8, 256, True), (16, 4096, 28672, 128, False)]:
            x, packed, scales, b = wl.w4a16_inputs(m, k, n, g, bias, seed=n + m)
            y = w4a16_linear(x.cuda(), packed.cuda(), scales.cuda(), b.cuda() if bias else None, group_size=g)
            ref = int4.w4a16_projection(x, packed, scales, b, group_size=g)
            err = (y.cpu().double() - ref.double()).abs()
            assert bool((err <= 0.002 + 0.002 * ref.double().abs()).all()), (m, k, n, g, float(err.max()))
            assert float((y.cpu().double() - ref.double()).norm() / ref.double().norm()) <= 1e-3
        from cross_dsl_kernels_b200 import _native
        assert _native.fault_flags() == 0
        print("umma ok")
    """ % str(ROOT))
    env = dict(os.environ, XDK_W4A16_UMMA=force)
    done = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "umma ok" in done.stdout, done.stdout + done.stderr


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,k,group", [(64, 4096, 128), (5, 257, 32), (3, 1000, 256), (2, 64, 64), (1, 1, 32)])
def test_device_quantiser_is_bit_identical_to_the_host_function(dtype, n, k, group):
    """xdk_quantize_int4 against quantize_int4 on the CPU (which the golden fixture pins to upstream's own
    output): same packed bytes, same FP16 scales; all-zero groups get scale 1."""
    g = torch.Generator().manual_seed(n * 1000 + k)
    w = (torch.randn(n, k, generator=g) * 0.05).to(dtype)
    if k >= group:
        w[0, :group] = 0  # an all-zero group
    w[-1, -1] = w.abs().max() * 3  # a clear peak at the ragged end
    want_p, want_s = qz.quantize_int4(w, group)
    got_p, got_s = qz.quantize_int4_device(w.cuda(), group)
    assert torch.equal(got_p.cpu(), want_p)
    assert torch.equal(got_s.cpu().view(torch.int16), want_s.view(torch.int16))


def test_device_quantiser_reports_what_the_host_function_raises_on():
    w = torch.randn(4, 256)
    bad = w.clone()
    bad[1, 7] = float("inf")
    with pytest.raises(ValueError, match="finite"):
        qz.quantize_int4_device(bad.cuda(), 128)
    huge = w.clone() * 1e6  # peak / 7 overflows FP16
    with pytest.raises(ValueError, match="FP16"):
        qz.quantize_int4_device(huge.cuda(), 128)
    with pytest.raises(ValueError):
        qz.quantize_int4_device(w, 128)  # a CPU tensor


def test_quantise_then_project_round_trip_on_the_device():
    from cross_dsl_kernels_b200.w4a16 import w4a16_linear
    g = torch.Generator().manual_seed(3)
    w = torch.randn(512, 1024, generator=g) * 0.02
    x = torch.randn(16, 1024, generator=g).half()
    packed, scales = qz.quantize_int4_device(w.cuda(), 128)
    y = w4a16_linear(x.cuda(), packed, scales, None, group_size=128)
    gate(y, x, packed.cpu(), scales.cpu(), None, 128)
