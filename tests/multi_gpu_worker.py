"""One rank of the multi-GPU parity run started by tests/test_gpu_multi.py (not a test module itself).

Checks, on real GPUs with one process per GPU:
  1. a column-sharded FP32 projection whose epilogue stores into every rank's peer-mapped matrix, against the FP64
     product, for the CUDA-core (M = 1, 4) and tensor-core (M = 16) kernels and both weight layouts;
  2. the same shards exchanged with NCCL all-gather + the re-layout kernel (the comparison arm);
  3. one sharded decode layer (peer exchange, and NCCL) against the same layer run unsharded on this GPU;
  4. a flag-barrier wait that runs out: only rank 0 enters a barrier nobody else joins, with a 2 ms budget; the
     kernel must return, report the missing ranks, and leave the context usable.
"""

from __future__ import annotations

import os
import pathlib
import sys

import torch
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def rel_l2(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-12))


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from cross_dsl_kernels_b200 import _native
    from cross_dsl_kernels_b200.chain import ChainConfig, DecodeLayerChain, unshard_columns
    from cross_dsl_kernels_b200.ops import decode_linear
    from cross_dsl_kernels_b200.peer import PeerArena
    from cross_dsl_kernels_b200.tolerances import fp32_gemv_tolerance

    # ---- 1 + 2: sharded projections
    k, n = 4096, 4096 * world
    arena = PeerArena(3 * 16 * n * 4 + 4096)
    site = arena.new_site()
    for m in (1, 4, 16):
        full = arena.matrix(m, n, torch.float32) if m != 4 else arena.matrix(m, n, torch.float32)
        for layout in ("KN", "NK"):
            g = torch.Generator(device="cuda").manual_seed(100 + m)  # the same stream on every rank
            x = torch.randn(m, k, generator=g, device="cuda")
            w = torch.randn(k, n, generator=g, device="cuda") / k ** 0.5
            b = 0.02 * torch.randn(n, generator=g, device="cuda")
            lo, hi = rank * n // world, (rank + 1) * n // world
            w_shard = w[:, lo:hi].contiguous() if layout == "KN" else w.t()[lo:hi].contiguous()
            want = x.double() @ w.double() + b.double()
            tol = fp32_gemv_tolerance(k)
            full.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            assert decode_linear(x, w_shard, b[lo:hi].contiguous(), weight_layout=layout, peer_out=full.out_for(lo)) is None
            arena.barrier(site)
            torch.cuda.synchronize()
            got = full.local
            assert float((got.double() - want).abs().max()) <= tol["max_abs_err"], (m, layout, "peer max abs")
            assert rel_l2(got, want) <= tol["rel_l2_err"], (m, layout, "peer rel l2")
            # comparison arm: NCCL all-gather + re-layout
            y = decode_linear(x, w_shard, b[lo:hi].contiguous(), weight_layout=layout)
            gathered = torch.empty(world, m, n // world, device="cuda")
            dist.all_gather_into_tensor(gathered, y)
            out = unshard_columns(gathered, torch.empty(m, n, device="cuda"))
            assert torch.equal(out, got), (m, layout, "peer store and NCCL gather disagree")
            dist.barrier()
    assert arena.fault_flags() == 0

    # ---- 3: one decode layer, sharded against unsharded
    cfg = ChainConfig()
    whole = DecodeLayerChain(cfg, layers=2, rank=0, world=1, seed=0)
    ref = whole.run_layers()
    torch.cuda.synchronize()
    for exchange in ("peer", "nccl"):
        for dependent in (False, True):
            chain = DecodeLayerChain(cfg, layers=2, rank=rank, world=world, seed=0, exchange=exchange,
                                     dependent_launch=dependent)
            out = chain.run_layers()
            torch.cuda.synchronize()
            dist.barrier()
            assert rel_l2(out["attn"].float(), ref["attn"].float()) <= 2e-3, (exchange, dependent, "rotated q")
            assert rel_l2(out["up_all"].float(), ref["up_all"].float()) <= 2e-3, (exchange, dependent, "up+gate")
            hkv = cfg.kv_heads // world
            want_k = whole.k_cache[:, :, rank * hkv:(rank + 1) * hkv]
            assert rel_l2(chain.k_cache.float(), want_k.float()) <= 2e-3, (exchange, dependent, "k cache shard")
            if chain.arena is not None:
                assert chain.arena.fault_flags() == 0
                dist.barrier()
                chain.arena.close()

    # ---- 3b: the layer with the attention read and SwiGLU: attention sharded by KV head against the rank's own cache
    # shard, up and gate columns paired on a rank, both results assembled on every rank through peer stores
    del whole, ref
    small = ChainConfig(context=2048)
    whole = DecodeLayerChain(small, layers=2, rank=0, world=1, seed=0, attention=True)
    ref = whole.run_layers()
    torch.cuda.synchronize()
    for dependent in (False, True):
        chain = DecodeLayerChain(small, layers=2, rank=rank, world=world, seed=0, exchange="peer", dependent_launch=dependent,
                                 attention=True)
        out = chain.run_layers()
        torch.cuda.synchronize()
        dist.barrier()
        assert torch.isfinite(out["attn"]).all() and torch.isfinite(out["act"]).all()
        assert rel_l2(out["attn"].float(), ref["attn"].float()) <= 2e-3, (dependent, "attention output")
        assert rel_l2(out["act"].float(), ref["act"].float()) <= 3e-3, (dependent, "SwiGLU activation")
        assert rel_l2(out["n2"].float(), ref["n2"].float()) <= 2e-3, (dependent, "second norm")
        assert chain.arena.fault_flags() == 0
        dist.barrier()
        chain.arena.close()
    del whole, ref

    # ---- 4: a barrier nobody else joins runs out of time, reports it, and the context stays usable
    lonely = arena.new_site()
    dist.barrier()
    if rank == 0:
        arena.barrier(lonely, timeout_us=2000)
        torch.cuda.synchronize()
        missing = arena.fault_flags()
        assert missing == sum(1 << p for p in range(1, world)), hex(missing)
        t = torch.ones(8, device="cuda") * 2
        assert float(t.sum()) == 16.0
    dist.barrier()
    assert _native.fault_flags() == 0
    torch.cuda.synchronize()
    dist.barrier()
    arena.close()
    print(f"rank {rank}: multi-GPU parity ok", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
