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
@pytest.mark.parametrize("k", [64, 192, 1024, 4096, 8192, 12352])
@pytest.mark.parametrize("n", [4096, 4100, 6144, 7168, 12300, 14336, 24580, 28672, 131072])
def test_plan_invariants(k, n, nk):
    if k * n < (4 << 20):
        assert plan(16, k, n, nk)[0] == 0
        return
    took, (ctas, split, ring, smem, units) = plan(16, k, n, nk)
    assert took == 1
    assert units == -(-n // 32)
    assert ctas == min(SMS, units), "one persistent CTA per SM, never more CTAs than 32-column units"
    per_cta = -(-units // ctas)
    # K is split over the TMEM lane quarters only as far as every k range stays a whole number of 64-k steps
    want = 4 if per_cta == 1 else (2 if per_cta == 2 else 1)
    while want > 1 and k % (64 * want):
        want //= 2
    assert split == want and k % (64 * split) == 0
    assert 3 <= ring <= 8
    assert smem <= MAX_DYNAMIC_SMEM
    fixed = smem - ring * STEP_BYTES
    # x buffers grow with the split: 2 x (hi image + lo image + raw rows) of 16 S rows x 64 k FP32, + partials + barriers
    assert fixed == 2 * split * (2 * 4096 + 4096) + 8192 + 512
    assert smem + STEP_BYTES > 220 * 1024 or ring == 8, "the ring takes whatever the x buffers leave"


def test_headline_shapes():
    assert plan(16, 4096, 14336)[1][:3] == [148, 1, 5]
    assert plan(16, 4096, 4096)[1][:3] == [128, 4, 3]
    assert plan(16, 4096, 6144, 1)[1][:3] == [148, 2, 5]


@pytest.mark.parametrize("k,n,parts", [(4096, 1792, 2), (4096, 2368, 2), (4096, 1024, 4), (8192, 1056, 4), (4096, 2400, 1),
                                       (256, 16384, 1)])
def test_narrow_projections_split_k_over_a_cluster(k, n, parts):
    """Fewer 32-column units than half (a quarter) of the SMs: two (four) CTAs share every unit along K, so the
    plan reports parts x units CTAs."""
    took, (ctas, split, ring, smem, units) = plan(16, k, n, 0)
    assert took == 1
    assert units == -(-n // 32)
    assert ctas == min(SMS, units) * parts
    assert (k // parts) % (64 * split) == 0
    assert smem <= MAX_DYNAMIC_SMEM
