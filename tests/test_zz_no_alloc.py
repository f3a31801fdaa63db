"""The allocation-free projection entry point, xdk_gemv_f32_static_scratch.

Some hosts cannot allocate device memory around a kernel call (a decode loop that runs with the
allocator closed, a plugin boundary that only passes inputs and outputs), so this entry point keeps
its partial sums in an array inside the library.  The test drives it straight through the C ABI and
demands the same bits as xdk_gemv_f32 given caller-provided scratch -- twice in a row with different
activations, because the built-in array still holds the first call's partial sums when the second
one starts.  This file sorts last so that a run stopping at the first failure has already run
everything else.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _project(fn_name, x, w, b, y, nk, scratch=None):
    from cross_dsl_kernels_b200 import _native
    lib = _native.lib()
    m, k = x.shape
    n = y.shape[1]
    stream = _native.stream_ptr(x.device)
    if fn_name == "static":
        status = lib.xdk_gemv_f32_static_scratch(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), m, k, n, int(nk), stream)
    else:
        status = lib.xdk_gemv_f32(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), m, k, n, int(nk), 0,
                                  scratch.data_ptr(), scratch.numel(), stream)
    _native.check(status, fn_name)


@pytest.mark.parametrize("nk", [False, True])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(nk):
    from cross_dsl_kernels_b200 import _native
    m, k, n = 16, 4096, 14336
    g = torch.Generator().manual_seed(21)
    w = (torch.randn(n, k, generator=g) / 64 if nk else torch.randn(k, n, generator=g) / 64).cuda()
    b = (0.02 * torch.randn(n, generator=g)).cuda()
    need = _native.lib().xdk_gemv_scratch_bytes(m, k, n, int(nk))
    assert 0 < need <= 160 * 2 * 16 * 128 * 4
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    for call in range(2):
        x = torch.randn(m, k, generator=g).cuda()
        want = torch.full((m, n), float("nan"), device="cuda")
        got = torch.full((m, n), float("nan"), device="cuda")
        _project("caller", x, w, b, want, nk, scratch)
        _project("static", x, w, b, got, nk)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all(), f"call {call}"
        assert torch.equal(got, want), f"call {call}: the built-in scratch must give the caller-scratch bits"
        reference = x.double() @ (w.double().t() if nk else w.double()) + b.double()
        assert float((got.double() - reference).abs().max()) <= 4e-4  # the projection's own gate at K = 4096


@pytest.mark.parametrize("nk", [False, True])
def test_static_scratch_on_a_small_matrix_runs_the_tile_stream_kernel_too(nk):
    """Below K*N = 48M xdk_gemv_f32 itself would pick the cluster kernels (another summation order); the
    allocation-free entry point runs the tile-stream kernel at every size.  So on a small matrix it is held to the
    projection's gate against an FP64 product, and to giving the same bits twice -- not to equality with xdk_gemv_f32."""
    m, k, n = 9, 1024, 640
    g = torch.Generator().manual_seed(22)
    w = (torch.randn(n, k, generator=g) / 32 if nk else torch.randn(k, n, generator=g) / 32).cuda()
    b = (0.02 * torch.randn(n, generator=g)).cuda()
    x = torch.randn(m, k, generator=g).cuda()
    reference = x.double() @ (w.double().t() if nk else w.double()) + b.double()
    results = []
    for _ in range(2):
        got = torch.full((m, n), float("nan"), device="cuda")
        _project("static", x, w, b, got, nk)
        torch.cuda.synchronize()
        assert float((got.double() - reference).abs().max()) <= 2e-4
        assert float((got.double() - reference).norm() / reference.norm()) <= 1e-5
        results.append(got)
    assert torch.equal(results[0], results[1])


def test_static_scratch_rejects_what_it_cannot_hold():
    from cross_dsl_kernels_b200 import _native
    lib = _native.lib()
    x = torch.zeros(16, 64, device="cuda")
    w = torch.zeros(64, 128, device="cuda")
    y = torch.zeros(16, 128, device="cuda")
    stream = _native.stream_ptr(x.device)
    # M outside the tile-stream kernel's range, then an unaligned activation pointer
    assert lib.xdk_gemv_f32_static_scratch(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 4, 64, 128, 0, stream) == -1
    assert lib.xdk_gemv_f32_static_scratch(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 17, 64, 128, 0, stream) == -1
    assert lib.xdk_gemv_f32_static_scratch(x.data_ptr() + 4, w.data_ptr(), None, y.data_ptr(), 8, 60, 128, 0, stream) == -1
    assert lib.xdk_gemv_f32_static_scratch(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 8, 1 << 30, 128, 0, stream) == -4


def test_no_device_side_wait_ever_gave_up():
    """Runs after the whole GPU suite: none of the time-bounded mbarrier waits in the TMA-fed kernels
    may have expired in this process."""
    from cross_dsl_kernels_b200 import _native
    torch.cuda.synchronize()
    assert _native.fault_flags() == 0
