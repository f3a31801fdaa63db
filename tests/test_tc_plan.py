"""Launch plan of the tensor-core FP32 projection (xdk_gemv_tc_plan): which shapes it takes and with what grid,
K split, ring depth and shared memory.  Pure host arithmetic inside the library: runs without a GPU (the SM
count then defaults to the B200's 148)."""

from __future__ import annotations

import ctypes

import pytest

SMS = 148
MAX_DYNAMIC_SMEM = 227 * 1024
STEP_BYTES = 32 * 1024  # one 64-k step of 128 columns of FP32 weights


def plan(m, k, n, nk=0):
    from cross_dsl_kernels_b200 import _native
    out = (ctypes.c_int32 * 5)(-1, -1, -1, -1, -1)
    took = _native.lib().xdk_gemv_tc_plan(m, k, n, nk, out)
    return took, list(out)


@pytest.mark.parametrize("m,k,n,nk", [
    (4, 4096, 14336, 0),     # M <= 4: the cluster kernels already run at the HBM rate
    (17, 4096, 14336, 0),    # M > 16 is tiled by rows elsewhere
    (16, 4100, 14336, 0),    # K not a multiple of the 64-k step
    (16, 4096, 14334, 0),    # KN rows must be 16-byte multiples for TMA
    (16, 4096, 512, 0),      # too small to pay for the pipeline set-up (K*N < 4M)
])
def test_shapes_the_path_declines(m, k, n, nk):
    took, out = plan(m, k, n, nk)
    assert took == 0 and out == [-1] * 5, "a declined shape leaves the output untouched"


def test_null_output_is_an_argument_error():
    from cross_dsl_kernels_b200 import _native
    assert _native.lib().xdk_gemv_tc_plan(16, 4096, 4096, 0, None) == -1


@pytest.mark.parametrize("nk", [0, 1])
@pytest.mark.parametrize("k", [64, 192, 1024, 4096, 8192, 12352, 14336])
@pytest.mark.parametrize("n", [512, 1024, 1792, 3584, 4096, 4100, 6144, 7168, 12300, 14336, 24580, 28672, 131072])
def test_plan_invariants(k, n, nk):
    # a CTA never sums more than 4096 k (accuracy of the truncating accumulation): longer rows need a cluster split
    admissible = [p for p in (1, 2, 4, 8) if k % (64 * p) == 0 and k // p <= 4096 and (p == 1 or k // p >= 256)]
    if k * n < (4 << 20) or not admissible:
        assert plan(16, k, n, nk)[0] == 0
        return
    parts, (ctas, split, ring, smem, units) = plan(16, k, n, nk)
    assert parts in admissible
    assert units == -(-n // 32)
    assert ctas % parts == 0 and ctas <= SMS, "whole clusters, one CTA per SM"
    assert ctas // parts <= units, "never more clusters than 32-column units"
    # both K splits leave every CTA and every TMEM lane quarter a whole number of 64-k steps
    assert split in (1, 2) and k % (64 * parts * split) == 0
    assert parts == 1 or k // parts >= 256
    assert 3 <= ring <= 8
    assert smem <= MAX_DYNAMIC_SMEM
    fixed = smem - ring * STEP_BYTES
    # x buffers grow with the lane-quarter split: 2 x (hi image + lo image + raw rows) of 16 S rows x 64 k FP32;
    # then the partial sums of this CTA and an inbox per further CTA of the cluster; then the barriers
    assert fixed == 2 * split * (2 * 4096 + 4096) + 8192 * parts + 512
    assert smem + STEP_BYTES > 220 * 1024 or ring == 8, "the ring takes whatever the other buffers leave"


def test_wide_projections_keep_one_cta_per_strip():
    assert plan(16, 4096, 14336) == (1, [148, 1, 5, 5 * STEP_BYTES + 2 * 12288 + 8192 + 512, 448])
    assert plan(16, 4096, 28672)[0] == 1 and plan(16, 4096, 131072, 1)[0] == 1
    assert plan(16, 64, 65536)[1][:2] == [148, 1]


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 3584), (14336, 4096), (4096, 1792), (4096, 6144), (4096, 1024), (8192, 1056)])
def test_narrow_projections_split_k_over_a_cluster(k, n):
    """With too few 32-column units to give every SM a four-unit strip, the CTAs of a cluster share each strip
    along K, and the busiest CTA walks fewer 64-k steps than it would alone."""
    parts, (ctas, split, ring, smem, units) = plan(16, k, n, 0)
    assert parts >= 2
    clusters = ctas // parts
    per_cluster = -(-units // clusters)
    steps = -(-per_cluster // (4 // split)) * (k // parts // split // 64)
    alone = -(-(-(-units // min(SMS, units))) // 4) * (k // 64)
    assert steps * 2 <= alone
