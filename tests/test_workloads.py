"""The algorithmic byte models behind every reported GB/s figure, pinned to the numbers the
roofline targets are quoted on (upstream's logical_bytes formulas: benchmarks/comparison_cases.py:42,
59, 113-117 and benchmarks/rmsnorm_bf16.py:74), plus the split-K slicing rule the kernels implement."""

from __future__ import annotations

import torch

from cross_dsl_kernels_b200 import workloads as wl
from cross_dsl_kernels_b200.chain import ChainConfig, qkv_shard_rows, upgate_shard_rows
from oracle import decode_ops


def test_rmsnorm_bytes():
    assert wl.rmsnorm_bytes(256, 4096, torch.float32) == 16_793_600
    assert wl.rmsnorm_bytes(4096, 4096, torch.float32) == 268_451_840
    assert wl.rmsnorm_bytes(256, 4096, torch.bfloat16) == 8_396_800
    assert wl.rmsnorm_bytes(4096, 4096, torch.bfloat16) == 134_225_920


def test_projection_bytes():
    assert wl.projection_bytes(1, 4096, 4096, bias=False) == 67_141_632
    assert wl.projection_bytes(16, 4096, 4096, bias=False) == 67_633_152
    assert wl.projection_bytes(1, 4096, 14336, bias=False) == 234_954_752
    assert wl.projection_bytes(16, 4096, 14336, bias=False) == 236_060_672
    assert wl.projection_bytes(1, 4096, 14336, bias=True) - wl.projection_bytes(1, 4096, 14336, bias=False) == 57_344


def test_rope_bytes():
    assert wl.rope_bytes(16, 32, 8, 128, 64, torch.float32) == 790_912
    assert wl.rope_bytes(16, 32, 8, 128, 128, torch.float32) == 795_008
    assert wl.rope_bytes(16, 32, 8, 128, 64, torch.bfloat16) == 397_696
    assert wl.rope_bytes(16, 32, 8, 128, 128, torch.bfloat16) == 401_792


def test_w4a16_bytes_and_chain_total():
    assert wl.w4a16_bytes(1, 4096, 4096) == 8_667_136
    assert wl.w4a16_bytes(16, 4096, 4096) == 8_912_896
    assert wl.w4a16_bytes(1, 4096, 14336) == 30_314_496
    assert wl.w4a16_bytes(16, 4096, 14336) == 30_867_456
    assert ChainConfig().algorithmic_bytes() == 76_374_400


def test_rope_workload_is_a_valid_batch():
    case = wl.rope_inputs()
    assert tuple(case["page_table"].shape) == (16, 256) and case["cache_shape"] == (4096, 16, 8, 128)
    assert case["page_table"].unique().numel() == 4096, "block tables come from one permutation: no shared page"
    decode_ops.check_paged_indices(case["positions"], case["page_table"], case["sequence_ids"], page_size=16,
                                   num_cache_pages=4096, max_position=4096)


def test_shards_partition_the_columns_for_every_world_size():
    cfg = ChainConfig()
    for world in (1, 2, 4, 8):
        qkv = torch.cat([qkv_shard_rows(cfg, r, world) for r in range(world)])
        up = torch.cat([upgate_shard_rows(cfg, r, world) for r in range(world)])
        assert sorted(qkv.tolist()) == list(range(cfg.qkv_cols))
        assert up.tolist() == list(range(2 * cfg.mlp))
        d = cfg.head_dim
        for r in range(world):  # a rank's K and V rows are the heads it appends to its own cache shard
            rows = qkv_shard_rows(cfg, r, world)
            hq, hkv = cfg.q_heads // world, cfg.kv_heads // world
            assert rows[hq * d].item() == cfg.q_heads * d + r * hkv * d
            assert rows[(hq + hkv) * d].item() == (cfg.q_heads + cfg.kv_heads) * d + r * hkv * d


def test_paired_up_gate_shards_keep_a_column_and_its_gate_on_one_rank():
    """For the layer that applies SwiGLU every rank owns a block of up columns and the same block of gate columns,
    stored [up_r | gate_r]: the activation of those columns needs no other rank."""
    cfg = ChainConfig()
    for world in (1, 2, 4, 8):
        width = cfg.mlp // world
        seen = []
        for r in range(world):
            rows = upgate_shard_rows(cfg, r, world, paired=True)
            assert rows.numel() == 2 * width
            up, gate = rows[:width], rows[width:]
            assert torch.equal(gate, up + cfg.mlp), "row j of the gate half gates row j of the up half"
            assert up[0].item() == r * width and up[-1].item() == (r + 1) * width - 1
            seen += rows.tolist()
        assert sorted(seen) == list(range(2 * cfg.mlp))
