"""Host logic of the multi-GPU path on CPU: two gloo ranks each compute their
column shard of the chain's two projections with the CPU oracle, all-gather the
shards rank-major and un-shard them; the result must equal the unsharded
projection (QKV up to the documented column order, up+gate exactly in place)."""

from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ok):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cross_dsl_kernels_b200.chain import (ChainConfig, _quantised, qkv_shard_rows, unshard_reference,
                                                  upgate_shard_rows)
        from oracle import int4
        cfg = ChainConfig(tokens=4, hidden=256, q_heads=4, kv_heads=2, head_dim=32, mlp=192, context=64)
        gen = torch.Generator().manual_seed(0)  # same weights on every rank
        qkv_p, qkv_s = _quantised(cfg.qkv_cols, cfg.hidden, cfg.group, gen)
        up_p, up_s = _quantised(2 * cfg.mlp, cfg.hidden, cfg.group, gen)
        x = torch.randn(cfg.tokens, cfg.hidden, generator=gen).half()
        for packed, scales, rows_fn in ((qkv_p, qkv_s, qkv_shard_rows), (up_p, up_s, upgate_shard_rows)):
            rows = rows_fn(cfg, rank, world)
            shard = int4.w4a16_projection(x, packed[rows].contiguous(), scales[rows].contiguous(), group_size=cfg.group)
            parts = [torch.empty_like(shard) for _ in range(world)]
            dist.all_gather(parts, shard)  # rank-major, like all_gather_into_tensor on the GPU path
            gathered = torch.stack(parts)
            full = int4.w4a16_projection(x, packed, scales, group_size=cfg.group)
            order = torch.cat([rows_fn(cfg, r, world) for r in range(world)])
            assert sorted(order.tolist()) == list(range(packed.shape[0])), "shards must partition the columns"
            assert torch.equal(unshard_reference(gathered), full[:, order])
        # KV heads: rank r appends exactly heads [r*Hkv/g, (r+1)*Hkv/g) -- the K/V part of its QKV rows
        d, hkv = cfg.head_dim, cfg.kv_heads // world
        rows = qkv_shard_rows(cfg, rank, world)
        k_rows = rows[cfg.q_heads // world * d: cfg.q_heads // world * d + hkv * d]
        assert k_rows[0].item() == cfg.q_heads * d + rank * hkv * d
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_column_sharding_with_two_gloo_ranks():
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_worker, args=(world, _free_port(), ok), nprocs=world, join=True)
    assert list(ok) == [1] * world


def _replay_count_worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cross_dsl_kernels_b200.timing import lockstep_replays
        # the ranks measured different times for the same 20 steps; both must replay the graph equally often
        out[rank] = lockstep_replays(7.0 if rank == 0 else 9.5, 20, device="cpu")
        out[world + rank] = lockstep_replays(1e-9 * (rank + 1), 20, device="cpu")  # absurdly fast: capped
    finally:
        dist.destroy_process_group()


def test_ranks_agree_on_the_number_of_graph_replays():
    """A step graph with collectives inside must be replayed the same number of times on every rank; the
    count follows the slowest rank's step time (about one second of load), and is bounded."""
    world = 2
    out = mp.get_context("spawn").Array("i", [0] * (2 * world))
    mp.spawn(_replay_count_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[0] == out[1] == int(1000.0 / (9.5 / 20))
    assert out[2] == out[3] == 5000


def test_replay_count_without_a_process_group():
    from cross_dsl_kernels_b200.timing import lockstep_replays
    assert lockstep_replays(10.0, 20, device="cpu") == 2000
    assert lockstep_replays(1e6, 2, device="cpu") == 1


# ---- host side of the peer-mapped path: agreement checks and failures made on the host (no GPU involved)


def _peer_host_worker(rank: int, world: int, port: int, ok):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from cross_dsl_kernels_b200.peer import agree, exchange_handles
        # 1. well-formed handles come back rank-major on every rank
        handles = exchange_handles(bytes([rank]) * 64)
        assert handles == [bytes([r]) * 64 for r in range(world)]
        # 2. a rank that contributes a truncated handle (a dropped or mangled message) makes EVERY rank refuse
        try:
            exchange_handles(bytes([rank]) * (64 if rank == 0 else 10))
            raise AssertionError("a 10-byte handle was accepted")
        except ValueError as err:
            assert "ranks [1]" in str(err)
        # 3. ranks that disagree on the arena size or the carving are stopped before any kernel runs
        agree("a value all ranks share", 4096)
        try:
            agree("the arena size", 4096 + rank)
            raise AssertionError("a size mismatch was accepted")
        except ValueError:
            pass
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_peer_arena_host_agreement_with_two_gloo_ranks():
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_peer_host_worker, args=(world, _free_port(), ok), nprocs=world, join=True)
    assert list(ok) == [1] * world


def _leaver_worker(rank: int, world: int, port: int, ok):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from cross_dsl_kernels_b200.peer import agree
    agree("the first step", 1)
    if rank == 1:
        ok[rank] = 1
        return  # leaves between steps without joining the next exchange (a rank that died on the host)
    try:
        agree("the step the other rank never joins", 2)
    except Exception:  # the short process-group timeout turns the missing rank into an error, not a hang
        ok[rank] = 1


def test_a_rank_that_leaves_is_an_error_not_a_hang():
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_leaver_worker, args=(world, _free_port(), ok), nprocs=world, join=True)
    assert list(ok) == [1] * world
