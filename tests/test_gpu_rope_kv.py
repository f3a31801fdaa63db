"""GPU parity of fused RoPE + paged K/V append: everything bit-exact against
the CPU oracle and the upstream golden outputs -- rotated Q, every K and V byte
written, and every cache slot that must stay untouched."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden, rebuild_cache
from oracle import decode_ops

pytestmark = pytest.mark.gpu

NAMES = ("q", "k", "v", "cos", "sin", "positions", "page_table", "sequence_ids")


def run_gpu(case, k_cache, v_cache):
    from cross_dsl_kernels_b200.ops import rope_gqa_paged_kv_append
    args = [case[n].cuda() for n in NAMES]
    return rope_gqa_paged_kv_append(*args, k_cache, v_cache, page_size=case["page_size"], rope_dim=case["rope_dim"],
                                    interleaved=case["interleaved"], kv_layout=case["kv_layout"])


def test_golden_cases_bit_exact():
    for case in load_golden("rope_kv"):
        k_cache = torch.full(case["cache_shape"], -999.0, dtype=case["k"].dtype, device="cuda")
        v_cache = torch.full_like(k_cache, -999.0)
        q_out = run_gpu(case, k_cache, v_cache)
        assert torch.equal(q_out.cpu(), case["q_out"])
        assert torch.equal(k_cache.cpu(), rebuild_cache(case, "k"))
        assert torch.equal(v_cache.cpu(), rebuild_cache(case, "v"))


def build_case(tokens, hq, hkv, dim, rd, ps, pages_per_seq, layout, interleaved, dtype, seed=0, max_pos=None):
    g = torch.Generator().manual_seed(seed)
    n_pages = tokens * pages_per_seq
    max_pos = max_pos or ps * pages_per_seq
    inv_freq = 10000.0 ** (-torch.arange(0, rd, 2).float() / rd)
    angle = torch.arange(max_pos).float()[:, None] * inv_freq[None, :]
    case = dict(
        q=torch.randn(tokens, hq, dim, generator=g).to(dtype),
        k=torch.randn(tokens, hkv, dim, generator=g).to(dtype),
        v=torch.randn(tokens, hkv, dim, generator=g).to(dtype),
        cos=angle.cos(), sin=angle.sin(),
        positions=torch.randint(0, max_pos, (tokens,), generator=g),
        page_table=torch.randperm(n_pages, generator=g).reshape(tokens, pages_per_seq),
        sequence_ids=torch.arange(tokens),
        page_size=ps, rope_dim=rd, interleaved=interleaved, kv_layout=layout,
        cache_shape=(n_pages, ps, hkv, dim) if layout == "NHD" else (n_pages, hkv, ps, dim))
    decode_ops.check_paged_indices(case["positions"], case["page_table"], case["sequence_ids"], page_size=ps,
                                   num_cache_pages=n_pages, max_position=max_pos)
    return case


def compare_with_oracle(case):
    dtype = case["k"].dtype
    k_ref = torch.full(case["cache_shape"], -999.0, dtype=dtype)
    v_ref = torch.full(case["cache_shape"], -999.0, dtype=dtype)
    q_ref = decode_ops.rope_paged_append(*[case[n] for n in NAMES], k_ref, v_ref, page_size=case["page_size"],
                                         rope_dim=case["rope_dim"], interleaved=case["interleaved"], kv_layout=case["kv_layout"])
    k_cache = torch.full(case["cache_shape"], -999.0, dtype=dtype, device="cuda")
    v_cache = torch.full_like(k_cache, -999.0)
    q_out = run_gpu(case, k_cache, v_cache)
    assert torch.equal(q_out.cpu(), q_ref), "rotated Q must be bit-exact"
    assert torch.equal(k_cache.cpu(), k_ref), "K cache (written and untouched slots) must be bit-exact"
    assert torch.equal(v_cache.cpu(), v_ref), "V cache must be bit-exact"
    # written slots hold no sentinel; count them
    written = int((k_cache != -999.0).sum())
    assert written == case["k"].numel()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["NHD", "HND"])
@pytest.mark.parametrize("rd", [64, 128])
def test_baseline_config(dtype, layout, rd):
    """16 decode tokens, 32 Q / 8 KV heads, head_dim 128, page 16, 4096 pages,
    positions uniform in [0, 4096), block tables from one random permutation."""
    compare_with_oracle(build_case(16, 32, 8, 128, rd, 16, 256, layout, False, dtype))


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("spec", [
    # tokens, hq, hkv, dim, rope_dim, page_size, pages_per_seq, layout, dtype
    (5, 6, 2, 10, 8, 8, 3, "NHD", torch.float32),
    (5, 6, 2, 10, 10, 8, 3, "HND", torch.float32),
    (4, 4, 4, 66, 22, 7, 5, "HND", torch.float32),
    (4, 4, 4, 66, 66, 7, 5, "NHD", torch.bfloat16),
    (7, 8, 1, 64, 32, 16, 4, "NHD", torch.float16),
    (3, 16, 4, 128, 128, 1, 9, "HND", torch.bfloat16),
    (9, 2, 2, 256, 96, 32, 2, "NHD", torch.float32),
    (1, 1, 1, 2, 2, 3, 2, "NHD", torch.float32),
    (16, 32, 8, 128, 64, 16, 512, "NHD", torch.float16),
])
def test_shapes_layouts_dtypes(spec, interleaved):
    tokens, hq, hkv, dim, rd, ps, pps, layout, dtype = spec
    compare_with_oracle(build_case(tokens, hq, hkv, dim, rd, ps, pps, layout, interleaved, dtype, seed=tokens + dim))


def test_wider_trig_table_and_shared_sequences():
    """cos/sin may have more columns than rope_dim/2; several tokens may belong to one sequence."""
    case = build_case(6, 8, 2, 64, 32, 8, 4, "NHD", False, torch.float32, seed=11)
    wide = torch.randn(case["cos"].shape[0], 40, generator=torch.Generator().manual_seed(1))
    case["cos"], case["sin"] = wide.cos(), wide.sin()
    case["sequence_ids"] = torch.tensor([0, 0, 0, 1, 1, 2])
    case["positions"] = torch.tensor([0, 7, 8, 31, 3, 16])
    compare_with_oracle(case)


def test_unaligned_views_take_scalar_path():
    case = build_case(4, 8, 2, 64, 32, 8, 4, "NHD", False, torch.bfloat16, seed=12)
    from cross_dsl_kernels_b200.ops import rope_gqa_paged_kv_append
    dtype = case["k"].dtype
    def shifted(t):
        buf = torch.zeros(t.numel() + 1, dtype=t.dtype, device="cuda")
        buf[1:] = t.flatten().cuda()
        return buf[1:].view(t.shape)
    q, k, v = shifted(case["q"]), shifted(case["k"]), shifted(case["v"])
    k_cache = shifted(torch.full(case["cache_shape"], -999.0, dtype=dtype))
    v_cache = shifted(torch.full(case["cache_shape"], -999.0, dtype=dtype))
    q_out = rope_gqa_paged_kv_append(q, k, v, *[case[n].cuda() for n in NAMES[3:]], k_cache, v_cache,
                                     page_size=8, rope_dim=32, interleaved=False, kv_layout="NHD")
    k_ref = torch.full(case["cache_shape"], -999.0, dtype=dtype); v_ref = k_ref.clone()
    q_ref = decode_ops.rope_paged_append(*[case[n] for n in NAMES], k_ref, v_ref, page_size=8, rope_dim=32, interleaved=False)
    assert torch.equal(q_out.cpu(), q_ref) and torch.equal(k_cache.cpu(), k_ref) and torch.equal(v_cache.cpu(), v_ref)


def test_append_then_append_is_idempotent_and_graph_safe():
    case = build_case(16, 32, 8, 128, 64, 16, 8, "HND", False, torch.bfloat16, seed=13)
    k_cache = torch.full(case["cache_shape"], -999.0, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.full_like(k_cache, -999.0)
    q1 = run_gpu(case, k_cache, v_cache)
    snap_k, snap_v = k_cache.clone(), v_cache.clone()
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        q2 = run_gpu(case, k_cache, v_cache)
    side.synchronize()
    assert torch.equal(q1, q2) and torch.equal(k_cache, snap_k) and torch.equal(v_cache, snap_v)
    from cross_dsl_kernels_b200.ops import rope_gqa_paged_kv_append
    args = [case[n].cuda() for n in NAMES]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gq = rope_gqa_paged_kv_append(*args, k_cache, v_cache, page_size=16, rope_dim=64, interleaved=False, kv_layout="HND")
    k_cache.fill_(-999.0); v_cache.fill_(-999.0); gq.fill_(float("nan"))
    graph.replay(); torch.cuda.synchronize()
    assert torch.equal(gq, q1) and torch.equal(k_cache, snap_k) and torch.equal(v_cache, snap_v)


def test_rejections():
    from cross_dsl_kernels_b200.ops import rope_gqa_paged_kv_append
    case = build_case(4, 8, 2, 64, 32, 8, 4, "NHD", False, torch.float32, seed=14)
    a = {n: case[n].cuda() for n in NAMES}
    kc = torch.full(case["cache_shape"], -999.0, device="cuda"); vc = kc.clone()
    kw = dict(page_size=8, rope_dim=32, interleaved=False, kv_layout="NHD")
    def call(**over):
        args = dict(a); cache = dict(k_cache=kc, v_cache=vc); kws = dict(kw)
        for key, val in over.items():
            (args if key in args else cache if key in cache else kws)[key] = val
        return rope_gqa_paged_kv_append(*[args[n] for n in NAMES], cache["k_cache"], cache["v_cache"], **kws)
    call()
    bad = [
        dict(v_cache=kc),                                  # caches alias each other
        dict(k_cache=a["q"].view(-1)[: 4 * 8 * 2 * 8].view(4, 8, 2, 8)),  # cache aliases an input / wrong dims
        dict(q=a["q"][:, :7].contiguous()),                # 7 Q heads over 2 KV heads
        dict(rope_dim=33), dict(rope_dim=0), dict(rope_dim=66), dict(page_size=0), dict(page_size=4),
        dict(kv_layout="DHN"), dict(kv_layout="HND"),
        dict(positions=a["positions"].int()), dict(cos=a["cos"][:, :8].contiguous()),
        dict(k=a["k"].half()), dict(v=a["v"][:3]), dict(sin=a["sin"][:5]),
        dict(q=a["q"].cpu()), dict(sequence_ids=a["sequence_ids"][:2]),
    ]
    for over in bad:
        with pytest.raises((ValueError, RuntimeError)):
            call(**over)
