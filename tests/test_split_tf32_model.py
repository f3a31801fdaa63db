"""CPU model of the arithmetic of the tensor-core FP32 projection (csrc/gemv_tc.cu): operands split into two
TF32 numbers, products hi.hi + hi.lo + lo.hi, FP32 accumulation that truncates (the pessimistic assumption for
the tensor core), k blocks of 8 dealt round-robin over several accumulators that are added in FP32 at the end.
It pins the design decisions the kernel relies on: the split is exact, one accumulator would break the
projection's 1e-5 relative-L2 gate at K = 4096, sixteen keep a wide margin (the GPU measures 2.35e-6)."""

from __future__ import annotations

import numpy as np

HI_MASK = np.uint32(0xFFFFE000)  # sign, exponent and the 10 mantissa bits TF32 keeps


def split(a: np.ndarray):
    hi = (a.view(np.uint32) & HI_MASK).view(np.float32)
    lo = a - hi  # exact in FP32: at most 13 significant bits remain
    lo_seen = (lo.view(np.uint32) & HI_MASK).view(np.float32)  # the tensor core ignores the low 13 bits of lo too
    return hi, lo, lo_seen


def truncate_to_f32(v: np.ndarray) -> np.ndarray:
    f = v.astype(np.float32)
    over = np.abs(f.astype(np.float64)) > np.abs(v)
    f[over] = np.nextafter(f[over], np.float32(0))
    return f


def model(x, w, accumulators: int) -> np.ndarray:
    xh, _, xl = split(x)
    wh, _, wl = split(w)
    m, k = x.shape
    acc = np.zeros((accumulators, m, w.shape[1]), np.float32)
    for i, k0 in enumerate(range(0, k, 8)):
        sl = slice(k0, k0 + 8)
        f = np.float64
        part = xh[:, sl].astype(f) @ wh[sl].astype(f) + xh[:, sl].astype(f) @ wl[sl].astype(f) + xl[:, sl].astype(f) @ wh[sl].astype(f)
        a = i % accumulators
        acc[a] = truncate_to_f32(acc[a].astype(f) + part)
    y = acc[0]
    for a in range(1, accumulators):
        y = (y + acc[a]).astype(np.float32)
    return y


def rel_l2(y, ref) -> float:
    return float(np.linalg.norm(y.astype(np.float64) - ref) / np.linalg.norm(ref))


def test_the_split_is_exact_and_tf32_representable():
    rng = np.random.default_rng(1)
    a = (rng.standard_normal(4096) * np.exp(rng.uniform(-20, 20, 4096))).astype(np.float32)
    hi, lo, lo_seen = split(a)
    assert np.array_equal((hi.astype(np.float64) + lo.astype(np.float64)).astype(np.float32), a)
    assert not np.any(hi.view(np.uint32) & ~HI_MASK)
    nz = a != 0
    assert np.all(np.abs(lo[nz]) <= np.abs(a[nz]) * 2.0 ** -10)          # lo carries the bits below TF32's mantissa
    assert np.all(np.abs(lo - lo_seen)[nz] <= np.abs(a[nz]) * 2.0 ** -20)  # what the hardware drops from lo


def test_accumulator_count_decides_the_gate():
    rng = np.random.default_rng(0)
    m, k, n = 16, 4096, 48
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / 64).astype(np.float32)
    ref = x.astype(np.float64) @ w.astype(np.float64)
    one, sixteen = rel_l2(model(x, w, 1), ref), rel_l2(model(x, w, 16), ref)
    assert one > 1e-5, "a single truncating accumulator would fail the projection's gate"
    assert sixteen < 2.5e-6, "sixteen accumulators leave a 4x margin even if every addition truncates"
    plain_tf32 = rel_l2((split(x)[0].astype(np.float64) @ split(w)[0].astype(np.float64)).astype(np.float32), ref)
    assert plain_tf32 > 1e-4, "without the lo terms TF32 is two orders of magnitude outside the gate"
