"""GPU tests of the two ops after the path: paged decode attention over the cache the append writes, and SwiGLU.
Upstream has neither, so the expectation is the oracle's own FP32 restatement (parity unpinned); tolerances:
FP32 rel-L2 <= 1e-5, 16-bit outputs <= 2 ulp / rel-L2 <= 2e-3."""

from __future__ import annotations

import pytest
import torch

from conftest import rel_l2, ulp_distance16  # noqa: F401
from oracle import attention as oracle_attention
from oracle import decode_ops

pytestmark = pytest.mark.gpu


def check(got, want, dtype):
    """rel-L2, and every element within about one unit of the output type at the result's top magnitude (values that
    cancel to nearly zero have no meaningful ulp distance)."""
    rel, top = {torch.float32: (1e-5, 2e-6), torch.float16: (1e-3, 2e-3), torch.bfloat16: (5e-3, 1e-2)}[dtype]
    assert rel_l2(got, want) <= rel
    assert float((got.double() - want.double()).abs().max()) <= top * float(want.double().abs().max())


def make_cache(tokens, q_heads, kv_heads, dim, page_size, max_pos, layout, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = -(-max_pos // page_size)
    pages = tokens * pages_per_seq + 1
    positions = torch.randint(0, max_pos, (tokens,), generator=g)
    positions[0] = 0                      # a context of one token
    positions[-1] = max_pos - 1           # and the longest one
    table = torch.randperm(pages - 1, generator=g).reshape(tokens, pages_per_seq)
    shape = (pages, page_size, kv_heads, dim) if layout == "NHD" else (pages, kv_heads, page_size, dim)
    kc = torch.randn(shape, generator=g).to(dtype)
    vc = torch.randn(shape, generator=g).to(dtype)
    q = torch.randn(tokens, q_heads, dim, generator=g).to(dtype)
    return q, kc, vc, positions, table, torch.arange(tokens)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("q_heads,kv_heads,dim,page_size,max_pos", [
    (32, 8, 128, 16, 1500),   # the decode layer's head geometry
    (8, 8, 64, 7, 300),       # no grouping, odd page size
    (16, 2, 256, 32, 700),    # eight query heads per KV head
    (4, 2, 128, 16, 40),      # contexts shorter than one tile
])
def test_attention_matches_the_fp32_restatement(dtype, layout, q_heads, kv_heads, dim, page_size, max_pos):
    from cross_dsl_kernels_b200.ops import paged_decode_attention
    tokens = 5
    q, kc, vc, pos, table, seq = make_cache(tokens, q_heads, kv_heads, dim, page_size, max_pos, layout, dtype, seed=dim + max_pos)
    want = oracle_attention.paged_decode_attention(q, kc, vc, pos, table, seq, page_size=page_size, kv_layout=layout)
    for hint in (0, max_pos):
        got = paged_decode_attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), table.cuda(), seq.cuda(), page_size=page_size,
                                     kv_layout=layout, context_hint=hint).cpu()
        check(got, want, dtype)
    again = paged_decode_attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), table.cuda(), seq.cuda(), page_size=page_size,
                                   kv_layout=layout).cpu()
    assert torch.equal(again, paged_decode_attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), table.cuda(), seq.cuda(),
                                                     page_size=page_size, kv_layout=layout).cpu()), "deterministic"


def test_attention_reads_what_the_append_wrote():
    """Append (rotation + cache write) followed by the attention read, both on the GPU, against the oracle's append
    followed by the oracle's attention: the two kernels agree on every address."""
    from cross_dsl_kernels_b200.ops import paged_decode_attention, rope_gqa_paged_kv_append
    tokens, hq, hkv, dim, ps, ctx = 4, 8, 2, 128, 16, 200
    q, kc, vc, pos, table, seq = make_cache(tokens, hq, hkv, dim, ps, ctx, "NHD", torch.float16, seed=9)
    g = torch.Generator().manual_seed(10)
    k_new, v_new = torch.randn(tokens, hkv, dim, generator=g).half(), torch.randn(tokens, hkv, dim, generator=g).half()
    angle = torch.arange(float(ctx))[:, None] * (10000.0 ** (-torch.arange(0, dim, 2).float() / dim))[None, :]
    kd, vd = kc.cuda(), vc.cuda()
    q_rot = rope_gqa_paged_kv_append(q.cuda(), k_new.cuda(), v_new.cuda(), angle.cos().cuda(), angle.sin().cuda(), pos.cuda(),
                                     table.cuda(), seq.cuda(), kd, vd, page_size=ps, rope_dim=dim, interleaved=False)
    got = paged_decode_attention(q_rot, kd, vd, pos.cuda(), table.cuda(), seq.cuda(), page_size=ps).cpu()
    q_ref = decode_ops.rope_paged_append(q, k_new, v_new, angle.cos(), angle.sin(), pos, table, seq, kc, vc, page_size=ps,
                                         rope_dim=dim, interleaved=False)
    want = oracle_attention.paged_decode_attention(q_ref, kc, vc, pos, table, seq, page_size=ps)
    check(got, want, torch.float16)


def test_attention_rejections():
    from cross_dsl_kernels_b200.ops import paged_decode_attention
    q, kc, vc, pos, table, seq = (t.cuda() for t in make_cache(3, 8, 2, 128, 16, 64, "NHD", torch.float16, seed=1))
    bad = [
        lambda: paged_decode_attention(q, kc, vc.float(), pos, table, seq, page_size=16),
        lambda: paged_decode_attention(q, kc, vc, pos.int(), table, seq, page_size=16),
        lambda: paged_decode_attention(q, kc, vc, pos, table, seq, page_size=8),           # cache shape says 16
        lambda: paged_decode_attention(q[:, :6].contiguous(), kc, vc, pos, table, seq, page_size=16),   # 6 / 2 = 3 heads per group
        lambda: paged_decode_attention(q, kc, vc, pos, table, seq, page_size=16, kv_layout="XYZ"),
        lambda: paged_decode_attention(q.cpu(), kc, vc, pos, table, seq, page_size=16),
    ]
    for call in bad:
        with pytest.raises((ValueError, RuntimeError)):
            call()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,width", [(16, 14336), (3, 513), (1, 8)])
def test_swiglu(dtype, rows, width):
    from cross_dsl_kernels_b200.ops import swiglu
    g = torch.Generator().manual_seed(rows + width)
    x = (2 * torch.randn(rows, 2 * width, generator=g)).to(dtype)
    want = oracle_attention.swiglu(x)
    got = swiglu(x.cuda()).cpu()
    if dtype == torch.float32:
        assert rel_l2(got, want) <= 1e-6
    else:
        assert ulp_distance16(got, want) <= 1
    wide = torch.zeros(rows, 2 * width + 16, dtype=dtype)
    wide[:, : 2 * width] = x
    assert torch.equal(swiglu(wide.cuda()[:, : 2 * width]).cpu(), got), "rows a fixed number of elements apart"


def _one_rank_out(matrix, col0):
    """The descriptor a rank of a one-rank "arena" would pass: columns [col0, ...) of its own wider matrix."""
    from cross_dsl_kernels_b200 import _native
    out = _native.PeerOutStruct()
    out.ptr[0] = matrix.data_ptr()
    out.world, out.ld, out.col0 = 1, matrix.shape[1], col0
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_attention_and_swiglu_store_into_a_slice_of_a_wider_matrix(dtype):
    """The peer form of both ops (a rank's heads / columns inside the full-width matrix every rank assembles), with one
    rank: same values as the plain call, nothing written outside the slice."""
    from cross_dsl_kernels_b200.ops import paged_decode_attention, swiglu
    tokens, q_heads, kv_heads, dim, ps = 5, 8, 2, 128, 16
    q, kc, vc, pos, table, seq = make_cache(tokens, q_heads, kv_heads, dim, ps, 600, "NHD", dtype, seed=3)
    args = (q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), table.cuda(), seq.cuda())
    plain = paged_decode_attention(*args, page_size=ps)
    hidden = 3 * q_heads * dim  # the matrix of three such ranks; this one is the middle one
    full = torch.full((tokens, hidden), -7.0, dtype=dtype, device="cuda")
    assert paged_decode_attention(*args, page_size=ps, peer_out=_one_rank_out(full, q_heads * dim)) is None
    torch.cuda.synchronize()
    assert torch.equal(full[:, q_heads * dim: 2 * q_heads * dim], plain.view(tokens, q_heads * dim))
    assert bool((full[:, : q_heads * dim] == -7.0).all()) and bool((full[:, 2 * q_heads * dim:] == -7.0).all())
    with pytest.raises(ValueError):
        paged_decode_attention(*args, page_size=ps, peer_out=_one_rank_out(full, hidden - 8))

    for width in (512, 513):  # vector and scalar store paths
        g = torch.Generator().manual_seed(width)
        x = torch.randn(tokens, 2 * width, generator=g).to(dtype).cuda()
        want = swiglu(x)
        act = torch.full((tokens, 3 * width + 8), -7.0, dtype=dtype, device="cuda")
        assert swiglu(x, peer_out=_one_rank_out(act, width)) is None
        torch.cuda.synchronize()
        assert torch.equal(act[:, width: 2 * width], want)
        assert bool((act[:, :width] == -7.0).all()) and bool((act[:, 2 * width:] == -7.0).all())
