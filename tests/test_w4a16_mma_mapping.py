"""CPU model of the operand mapping of the direct-load W4A16 tensor-core kernel (w4a16_mma_kernel in csrc/w4a16.cu).

The kernel feeds mma.m16n8k16 with the operands swapped -- 16 weight columns are the MMA's rows, the rows of x its
columns -- and lets a fragment slot stand for whatever k the exact unpack happens to put there: word w of a lane's
16-byte vector (8 codes, first k = kw) unpacks to the half2 pairs (kw+0, kw+4) (kw+1, kw+5) (kw+2, kw+6) (kw+3, kw+7);
the first two pairs are the A registers of one MMA, the last two of the next, and x is staged in shared memory with
every 8 k permuted to (0, 4, 1, 5, 2, 6, 3, 7) so that one 16-byte read yields the matching B registers.  This file
restates that index arithmetic in numpy on top of an emulator of the PTX fragment layouts and checks that the eight
warps' partial sums add up to x @ W^T for every output the kernel stores.  No GPU, no rounding questions: integer data.
"""

from __future__ import annotations

import numpy as np
import pytest

WARPS = 8


def mma_m16n8k16(a_regs, b_regs, acc):
    """One warp-wide MMA from per-lane registers, by the PTX fragment layouts (row-major A, column-major B).

    a_regs[lane] = 4 registers of 2 values, b_regs[lane] = 2 registers of 2 values, acc[lane] = 4 values (updated)."""
    a = np.zeros((16, 16))
    b = np.zeros((16, 8))
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        (a[g, 2 * t], a[g, 2 * t + 1]) = a_regs[lane][0]
        (a[g + 8, 2 * t], a[g + 8, 2 * t + 1]) = a_regs[lane][1]
        (a[g, 2 * t + 8], a[g, 2 * t + 9]) = a_regs[lane][2]
        (a[g + 8, 2 * t + 8], a[g + 8, 2 * t + 9]) = a_regs[lane][3]
        (b[2 * t, g], b[2 * t + 1, g]) = b_regs[lane][0]
        (b[2 * t + 8, g], b[2 * t + 9, g]) = b_regs[lane][1]
    d = a @ b
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        acc[lane][0] += d[g, 2 * t]
        acc[lane][1] += d[g, 2 * t + 1]
        acc[lane][2] += d[g + 8, 2 * t]
        acc[lane][3] += d[g + 8, 2 * t + 1]


def unpack_pairs(wrow, kw):
    """What dequant8 makes of the word that starts at k = kw: four pairs, in its order."""
    return [(wrow[kw + i], wrow[kw + i + 4]) for i in range(4)]


def staged_x_row(xrow):
    """A row of x as the kernel stages it: every 8 k permuted to (0, 4, 1, 5, 2, 6, 3, 7)."""
    out = np.empty_like(xrow)
    for u in range(0, len(xrow), 8):
        out[u:u + 8] = xrow[u:u + 8][[0, 4, 1, 5, 2, 6, 3, 7]]
    return out


@pytest.mark.parametrize("m,k,n", [(8, 1024, 16), (3, 2048, 16), (1, 3072, 13)])
def test_fragment_slots_follow_the_unpack(m, k, n):
    rng = np.random.default_rng(m * 1000 + k)
    w = rng.integers(-8, 8, size=(16, k)).astype(np.float64)  # one pass = 16 weight columns
    w[n:] = 99.0                                                # columns past N: their sums are never stored
    x = rng.integers(-3, 4, size=(m, k)).astype(np.float64)
    xs = [staged_x_row(x[r]) for r in range(m)]
    k_warp = k // WARPS
    chunks = k_warp // 128
    total = np.zeros((32, 4))
    for warp in range(WARPS):
        acc0 = [[0.0] * 4 for _ in range(32)]
        acc1 = [[0.0] * 4 for _ in range(32)]
        for chunk in range(chunks):
            for word in range(4):
                a_first, a_second, b_first, b_second = [], [], [], []
                for lane in range(32):
                    col, q = lane >> 2, lane & 3
                    kw = warp * k_warp + chunk * 128 + q * 32 + word * 8   # first k of this lane's word
                    lo, hi = unpack_pairs(w[col], kw), unpack_pairs(w[col + 8], kw)
                    a_first.append([lo[0], hi[0], lo[1], hi[1]])
                    a_second.append([lo[2], hi[2], lo[3], hi[3]])
                    xrow = xs[col if col < m else 0]                        # lanes past M read row 0
                    xv = [tuple(xrow[kw + 2 * i: kw + 2 * i + 2]) for i in range(4)]  # one 16-byte read = 4 registers
                    b_first.append([xv[0], xv[1]])
                    b_second.append([xv[2], xv[3]])
                mma_m16n8k16(a_first, b_first, acc0)
                mma_m16n8k16(a_second, b_second, acc1)
        total += np.array(acc0) + np.array(acc1)
    want = x @ w.T
    for lane in range(32):
        col, q = lane >> 2, lane & 3
        for e in range(4):
            c, row = (e >> 1) * 8 + col, q * 2 + (e & 1)
            if row < m and c < n:  # exactly what the kernel stores
                assert total[lane][e] == want[row, c], (lane, e)
