"""GPU parity of the FP32 decode projection.  Gate (upstream
src/crossdsl_kernels/tolerances.py:7-25 against an FP64 product):
max-abs <= 2e-4 * max(1, sqrt(K/1024)) and rel-L2 <= 1e-5."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, rel_l2
from cross_dsl_kernels_b200.tolerances import fp32_gemv_tolerance
from oracle import decode_ops

pytestmark = pytest.mark.gpu


def make(m, k, n, layout, bias, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    w_kn = torch.randn(k, n, generator=g) / k ** 0.5
    b = 0.02 * torch.randn(n, generator=g) if bias else None
    w = w_kn if layout == "KN" else w_kn.t().contiguous()
    return x, w, b, w_kn


def gate(y, x, w_kn, b, k):
    want = x.double() @ w_kn.double()
    if b is not None:
        want = want + b.double()
    tol = fp32_gemv_tolerance(k)
    assert y.dtype == torch.float32 and tuple(y.shape) == tuple(want.shape)
    assert float((y.cpu().double() - want).abs().max()) <= tol["max_abs_err"]
    assert rel_l2(y.cpu(), want) <= tol["rel_l2_err"]


def test_golden_cases_all_split_factors():
    from cross_dsl_kernels_b200.ops import decode_linear
    for case in load_golden("gemv"):
        for split_k in (0, 1, 2, 4, 8):
            b = case["bias"].cuda() if case["bias"] is not None else None
            y = decode_linear(case["x"].cuda(), case["weight"].cuda(), b, weight_layout=case["weight_layout"], split_k=split_k)
            if case["exact"]:
                assert torch.equal(y.cpu(), case["y"]), (case["weight_layout"], split_k)
            else:
                torch.testing.assert_close(y.cpu(), case["y"], rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("layout", ["KN", "NK"])
@pytest.mark.parametrize("m", [1, 4, 16])
@pytest.mark.parametrize("n", [4096, 14336])
def test_baseline_shapes(layout, m, n):
    from cross_dsl_kernels_b200.ops import decode_linear
    k = 4096
    x, w, b, w_kn = make(m, k, n, layout, True)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    oracle = decode_ops.decode_projection(x, w, b, weight_layout=layout)
    for split_k in (0, 1, 2, 4, 8):
        y = decode_linear(xd, wd, bd, weight_layout=layout, split_k=split_k)
        gate(y, x, w_kn, b, k)
        assert rel_l2(y.cpu(), oracle) <= 1e-5
        again = decode_linear(xd, wd, bd, weight_layout=layout, split_k=split_k)
        assert torch.equal(y, again), "a (shape, split_k) pair must be deterministic"
    y = decode_linear(xd, wd, None, weight_layout=layout)
    gate(y, x, w_kn, None, k)


@pytest.mark.parametrize("layout", ["KN", "NK"])
@pytest.mark.parametrize("m,k,n", [(3, 513, 67), (5, 257, 67), (2, 33, 17), (3, 129, 65), (1, 1, 1), (16, 1, 5),
                                   (7, 4096, 100), (17, 300, 130), (33, 64, 40), (2, 5000, 260), (8, 1024, 1028)])
def test_tails_and_odd_sizes(layout, m, k, n):
    from cross_dsl_kernels_b200.ops import decode_linear
    x, w, b, w_kn = make(m, k, n, layout, True, seed=m * 1000 + n)
    for split_k in (0, 1, 2, 8):
        y = decode_linear(x.cuda(), w.cuda(), b.cuda(), weight_layout=layout, split_k=split_k)
        gate(y, x, w_kn, b, k)


@pytest.mark.parametrize("layout", ["KN", "NK"])
def test_unaligned_views(layout):
    from cross_dsl_kernels_b200.ops import decode_linear
    m, k, n = 4, 512, 256
    x, w, b, w_kn = make(m, k, n, layout, True, seed=2)
    bx = torch.zeros(m * k + 1).cuda(); bw = torch.zeros(k * n + 1).cuda(); bb = torch.zeros(n + 1).cuda()
    bx[1:] = x.flatten().cuda(); bw[1:] = w.flatten().cuda(); bb[1:] = b.cuda()
    y = decode_linear(bx[1:].view(m, k), bw[1:].view(*w.shape), bb[1:], weight_layout=layout)
    gate(y, x, w_kn, b, k)


@pytest.mark.parametrize("layout", ["KN", "NK"])
@pytest.mark.parametrize("m,k,n", [(16, 4096, 14336), (8, 4096, 14336), (5, 4100, 12300), (9, 2052, 24580), (16, 8192, 6148)])
def test_tile_stream_path(layout, m, k, n):
    """strict_fp32: 4 < M <= 16 on large matrices takes the persistent CUDA-core tile-stream kernel
    (scratch + finish kernel); sizes off the 32 x 128 tile grid exercise the zero-filled edges."""
    from cross_dsl_kernels_b200.ops import decode_linear
    x, w, b, w_kn = make(m, k, n, layout, True, seed=n)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    y = decode_linear(xd, wd, bd, weight_layout=layout, strict_fp32=True)
    gate(y, x, w_kn, b, k)
    assert torch.equal(y, decode_linear(xd, wd, bd, weight_layout=layout, strict_fp32=True)), "deterministic"
    gate(decode_linear(xd, wd, None, weight_layout=layout, strict_fp32=True), x, w_kn, None, k)


@pytest.mark.parametrize("layout", ["KN", "NK"])
@pytest.mark.parametrize("m,k,n", [
    (16, 4096, 14336),   # 3-4 units of 32 columns per SM: no K split
    (8, 4096, 14336),
    (16, 4096, 4096),    # too narrow for a full strip per SM: K split over clusters of four CTAs
    (16, 4096, 3584),
    (13, 4096, 6144),    # ... of eight
    (16, 4096, 7168),    # ... of two
    (5, 4160, 12300),    # ragged last unit, K a multiple of 64 but not of 256
    (9, 2048, 24580),    # more than four units per SM: several strips
    (16, 8192, 6148),
    (16, 1024, 4096),    # the smallest matrix the path takes
    (16, 4096, 28672),
    (16, 14336, 4096),   # the MLP-down projection: long K over a cluster
    (16, 4096, 1792),    # column shards of a multi-GPU run: cluster split, alone or with the lane-quarter split on top
    (16, 4096, 2368),
    (12, 8192, 2048),
    (16, 8192, 1056),
    (16, 14336, 512),
    (16, 4096, 1024),
    (7, 16384, 1000),    # ragged last unit with the cluster split
])
def test_tensor_core_path(layout, m, k, n):
    """The default for 4 < M <= 16 and K % 64 == 0: tcgen05 kind::tf32 MMAs on operands split into two
    TF32 halves (hi.hi + hi.lo + lo.hi), FP32 accumulation.  Same gate as every other projection kernel:
    max abs error <= 2e-4 * max(1, sqrt(K / 1024)) and relative L2 error <= 1e-5 against the FP64 product."""
    from cross_dsl_kernels_b200.ops import decode_linear
    x, w, b, w_kn = make(m, k, n, layout, True, seed=n + m)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    y = decode_linear(xd, wd, bd, weight_layout=layout)
    gate(y, x, w_kn, b, k)
    assert torch.equal(y, decode_linear(xd, wd, bd, weight_layout=layout)), "deterministic"
    gate(decode_linear(xd, wd, None, weight_layout=layout), x, w_kn, None, k)
    # rows of x past M never reach the output: the same rows inside a taller batch give the same values
    if m < 16:
        tall = torch.cat([x, torch.randn(16 - m, k)]).cuda()
        assert torch.equal(decode_linear(tall, wd, bd, weight_layout=layout)[:m], y)


@pytest.mark.parametrize("strict,bound", [(True, 2e-6), (False, 1e-5)])
def test_linearity_at_full_size(strict, bound):
    """y(a*x1 + x2) == a*y(x1) + y(x2) up to rounding: a size-independent property."""
    from cross_dsl_kernels_b200.ops import decode_linear
    g = torch.Generator().manual_seed(4)
    k, n = 4096, 14336
    w = (torch.randn(k, n, generator=g) / 64).cuda()
    x1, x2 = torch.randn(16, k, generator=g).cuda(), torch.randn(16, k, generator=g).cuda()
    lhs = decode_linear(2.0 * x1 + x2, w, strict_fp32=strict)
    rhs = 2.0 * decode_linear(x1, w, strict_fp32=strict) + decode_linear(x2, w, strict_fp32=strict)
    assert rel_l2(lhs.cpu(), rhs.cpu()) <= bound


def test_graph_replay_follows_changed_inputs_on_side_stream():
    from cross_dsl_kernels_b200.ops import decode_linear
    x, w, b, w_kn = make(4, 1024, 512, "KN", True)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y = decode_linear(xd, wd, bd, split_k=4)
    side.synchronize()
    gate(y, x, w_kn, b, 1024)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gy = decode_linear(xd, wd, bd, split_k=4)
    x2 = torch.randn(4, 1024, generator=torch.Generator().manual_seed(8))
    xd.copy_(x2); gy.fill_(float("nan"))
    graph.replay(); torch.cuda.synchronize()
    gate(gy, x2, w_kn, b, 1024)


@pytest.mark.parametrize("layout", ["KN", "NK"])
@pytest.mark.parametrize("k", [14336, 16384, 32768])
def test_tensor_core_path_at_large_k(layout, k):
    """The split-TF32 accumulation error grows with the number of products an accumulator sums, so the gate is
    checked at the largest K the tensor-core path takes (16384), at the MLP-down projection of the model the
    decode-layer chain is shaped on (14336), and beyond the cap (32768 runs on FP32 FMAs)."""
    from cross_dsl_kernels_b200.ops import decode_linear
    m, n = 16, 4096
    x, w, b, w_kn = make(m, k, n, layout, True, seed=k)
    y = decode_linear(x.cuda(), w.cuda(), b.cuda(), weight_layout=layout)
    gate(y, x, w_kn, b, k)
    import ctypes
    from cross_dsl_kernels_b200 import _native
    plan = (ctypes.c_int32 * 5)()
    assert (_native.lib().xdk_gemv_tc_plan(m, k, n, int(layout == "NK"), plan) > 0) == (k <= 16384)


def test_tensor_core_path_on_same_sign_and_wide_range_operands():
    """All-positive operands (post-activation inputs) expose a one-sided truncation bias that zero-mean data hide;
    a wide exponent spread exercises the lo halves.  Same gate."""
    from cross_dsl_kernels_b200.ops import decode_linear
    g = torch.Generator().manual_seed(11)
    m, k, n = 16, 4096, 4096
    x = torch.rand(m, k, generator=g) + 0.1
    w_kn = (torch.rand(k, n, generator=g) + 0.1) / k
    y = decode_linear(x.cuda(), w_kn.cuda())
    gate(y, x, w_kn, None, k)
    x2 = torch.randn(m, k, generator=g) * torch.exp2(torch.randint(-12, 12, (m, k), generator=g).float())
    w2 = torch.randn(k, n, generator=g) * torch.exp2(torch.randint(-12, 12, (k, n), generator=g).float()) / k ** 0.5
    want = x2.double() @ w2.double()
    y2 = decode_linear(x2.cuda(), w2.cuda())
    assert rel_l2(y2.cpu(), want) <= 1e-5


def test_rejections():
    from cross_dsl_kernels_b200.ops import decode_linear
    x, w, b, _ = make(2, 64, 32, "KN", True)
    x, w, b = x.cuda(), w.cuda(), b.cuda()
    bad = [
        lambda: decode_linear(x, w, b, weight_layout="XX"),
        lambda: decode_linear(x, w.t().contiguous(), b),
        lambda: decode_linear(x, w, b[:8]),
        lambda: decode_linear(x, w, b.half()),
        lambda: decode_linear(x.half(), w, b),
        lambda: decode_linear(x, w.half(), b),
        lambda: decode_linear(x[0], w, b),
        lambda: decode_linear(x, w.t(), b, weight_layout="NK"),
        lambda: decode_linear(x, w, b, split_k=3),
        lambda: decode_linear(x.cpu(), w, b),
        lambda: decode_linear(x, w, b.cpu()),
        lambda: decode_linear(x, w, torch.empty(0, device="cuda")),
    ]
    for call in bad:
        with pytest.raises((ValueError, RuntimeError)):
            call()
