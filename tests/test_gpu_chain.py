"""GPU parity of the decode-layer chain, stage by stage: every launch is checked
against the CPU oracle applied to the GPU's own input of that stage, with the
gate of that op (norm <= 1 FP16 ulp and residual exact; W4A16 |err| <= 0.002 +
0.002 |ref|; RoPE + append bit-exact)."""

from __future__ import annotations

import pytest
import torch

from conftest import rel_l2, ulp_distance16
from oracle import decode_ops, int4

pytestmark = pytest.mark.gpu


def w4_gate(y, ref):
    err = (y.double() - ref.double()).abs()
    assert bool((err <= 0.002 + 0.002 * ref.double().abs()).all()), float(err.max())
    assert rel_l2(y, ref) <= 1e-3


@pytest.mark.parametrize("small", [True, False])
def test_chain_stages_match_oracle(small):
    from cross_dsl_kernels_b200.chain import ChainConfig, DecodeLayerChain
    cfg = ChainConfig(hidden=1024, q_heads=8, kv_heads=2, mlp=1536, context=256) if small else ChainConfig()
    chain = DecodeLayerChain(cfg, layers=1)
    out = {k: v.cpu() for k, v in chain.step(0).items()}
    host = chain.host_weights(0)
    d, hq, hkv, t = cfg.head_dim, cfg.q_heads, cfg.kv_heads, cfg.tokens

    n1, r1 = decode_ops.residual_rmsnorm(chain.h, chain.res, host["w1"], cfg.eps)
    assert torch.equal(out["r1"], r1) and ulp_distance16(out["n1"], n1) <= 1

    qkv = int4.w4a16_projection(out["n1"], host["qkv_packed"], host["qkv_scales"], None, group_size=cfg.group)
    w4_gate(out["qkv"], qkv)

    q = out["qkv"][:, : hq * d].reshape(t, hq, d)
    k = out["qkv"][:, hq * d: (hq + hkv) * d].reshape(t, hkv, d)
    v = out["qkv"][:, (hq + hkv) * d:].reshape(t, hkv, d)
    shape = tuple(chain.k_cache.shape)
    k_ref = torch.full(shape, -999.0, dtype=torch.float16)
    v_ref = torch.full(shape, -999.0, dtype=torch.float16)
    q_ref = decode_ops.rope_paged_append(q, k, v, chain.cos, chain.sin, chain.positions, chain.page_table,
                                         chain.sequence_ids, k_ref, v_ref, page_size=cfg.page_size, rope_dim=d,
                                         interleaved=False)
    assert torch.equal(out["q_rot"], q_ref)
    assert torch.equal(chain.k_cache.cpu(), k_ref) and torch.equal(chain.v_cache.cpu(), v_ref)

    n2, r2 = decode_ops.residual_rmsnorm(out["attn"], out["r1"], host["w2"], cfg.eps)
    assert torch.equal(out["r2"], r2) and ulp_distance16(out["n2"], n2) <= 1

    up = int4.w4a16_projection(out["n2"], host["up_packed"], host["up_scales"], None, group_size=cfg.group)
    w4_gate(out["up_all"], up)


def test_chain_graph_replay_is_stable():
    from cross_dsl_kernels_b200.chain import ChainConfig, DecodeLayerChain
    chain = DecodeLayerChain(ChainConfig(hidden=1024, q_heads=8, kv_heads=2, mlp=1536, context=256), layers=2)
    eager = chain.run_layers()["up_all"].clone()
    stream = torch.cuda.Stream(); stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        captured = chain.run_layers()["up_all"]
    captured.fill_(float("nan"))
    graph.replay(); torch.cuda.synchronize()
    assert torch.equal(captured, eager)


def test_unshard_columns_kernel():
    from cross_dsl_kernels_b200.chain import unshard_columns, unshard_reference
    for world, rows, cols, dtype in [(2, 16, 2048, torch.float16), (8, 16, 3584, torch.float16), (4, 3, 5, torch.float32),
                                     (3, 7, 9, torch.uint8)]:
        g = torch.arange(world * rows * cols).reshape(world, rows, cols).to(dtype).cuda()
        out = torch.empty(rows, world * cols, dtype=dtype, device="cuda")
        assert torch.equal(unshard_columns(g, out), unshard_reference(g))
