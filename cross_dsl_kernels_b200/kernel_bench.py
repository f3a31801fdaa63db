"""Per-kernel CUDA-graph medians for the decode ops at their headline shapes.

Each row times one op at one shape: a CUDA graph of back-to-back calls that
rotate over enough distinct buffer sets to defeat the L2 (see timing.py),
replayed and event-timed; ``gbps`` is the op's algorithmic bytes over the
per-call median.  Used by bench.py and usable on its own:

    python -m cross_dsl_kernels_b200.kernel_bench [rmsnorm|gemv|rope|w4a16] ...

Every ``bench_*`` function takes an optional ``check(stage, outputs)``: the
caller's gate, run on the eager result, on a replay with poisoned outputs and
on a replay after the inputs changed in place (timing.graph_median_us).  The
functions hand the gate what it needs to recompute the expected result: call 0
always runs on the seeded inputs of workloads.py, and the in-place change is
"negate the activations".  ``dependent=True`` launches every call as a
programmatic dependent of the call before it (rows named ``*_pdl``): the calls
are independent of one another, so this shows what the op costs inside a chain
whose kernels overlap their set-up with the predecessor's tail.
"""

from __future__ import annotations

import json
import sys

import torch

from . import _native
from . import workloads as wl
from .ops import decode_linear, fused_residual_rmsnorm, paged_decode_attention, rope_gqa_paged_kv_append, swiglu
from .timing import graph_median_us, rotation_for
from .w4a16 import w4a16_linear

NOMINAL_HBM_GBPS = 8000.0


def _row(name: str, nbytes: int, timing: dict, sets: int, peak_gbps: float | None, **extra) -> dict:
    us = timing["median_us"]
    gbps = nbytes / us * 1e-3
    row = {"kernel": name, "us": round(us, 3), "bytes": nbytes, "gbps": round(gbps, 1),
           "frac_of_8tbs": round(gbps / NOMINAL_HBM_GBPS, 4), "buffer_sets": sets,
           "p10_us": round(timing["p10_us"], 3), "p90_us": round(timing["p90_us"], 3), "gated": timing["gated"]}
    if peak_gbps:
        row["frac_of_measured"] = round(gbps / peak_gbps, 4)
    row.update(extra)
    return row


def _calls_per_graph(sets: int) -> int:
    return sets * max(1, -(-20 // sets))  # at least 20 calls, whole rotations


def bench_noop(replays=20, dependent=False) -> dict:
    """An empty kernel as a graph node: the floor under every per-call figure of this table."""
    lib = _native.lib()
    flags = _native.XDK_DEPENDENT_LAUNCH if dependent else 0

    def call():
        _native.check(lib.xdk_noop(flags, _native.stream_ptr(torch.device("cuda", torch.cuda.current_device()))), "xdk_noop")

    t = graph_median_us([call] * 40, replays)
    return {"kernel": "empty_kernel_graph_node" + ("_pdl" if dependent else ""), "us": round(t["median_us"], 3),
            "p10_us": round(t["p10_us"], 3), "p90_us": round(t["p90_us"], 3), "bytes": 0, "gated": False}


def bench_rmsnorm(rows: int, hidden: int, dtype, peak=None, replays=20, check=None, dependent=False) -> dict:
    nbytes = wl.rmsnorm_bytes(rows, hidden, dtype)
    sets = rotation_for(nbytes)
    x, r, w = (t.cuda() for t in wl.rmsnorm_inputs(rows, hidden, dtype))
    data = [(x.roll(s, 0), r.roll(s, 0), w) if s else (x, r, w) for s in range(sets)]
    n = _calls_per_graph(sets)
    calls = [(lambda d=data[i % sets]: fused_residual_rmsnorm(d[0], d[1], d[2], 1e-6, dependent_launch=dependent)) for i in range(n)]
    t = graph_median_us(calls, replays, check=check, mutate=lambda: x.neg_())
    name = f"rmsnorm_{str(dtype).split('.')[-1]}_{rows}x{hidden}" + ("_pdl" if dependent else "")
    return _row(name, nbytes, t, sets, peak)


def bench_gemv(m: int, k: int, n: int, layout: str, split_k: int = 0, bias=True, peak=None, replays=20,
               strict_fp32: bool = False, check=None, dependent=False) -> dict:
    nbytes = wl.projection_bytes(m, k, n, bias)
    sets = rotation_for(nbytes, cap=8)
    x, w, b = wl.projection_inputs(m, k, n, layout, bias)
    xd, bd = x.cuda(), (b.cuda() if bias else None)
    ws = [w.cuda()] + [torch.empty_like(w, device="cuda").normal_(0, k ** -0.5) for _ in range(sets - 1)]
    ncalls = _calls_per_graph(sets)
    calls = [(lambda wt=ws[i % sets]: decode_linear(xd, wt, bd, weight_layout=layout, split_k=split_k, strict_fp32=strict_fp32,
                                                    dependent_launch=dependent)) for i in range(ncalls)]
    t = graph_median_us(calls, replays, check=check, mutate=lambda: xd.neg_())
    name = (f"gemv_f32_{layout}_m{m}_k{k}_n{n}_s{split_k}" + ("_strict" if strict_fp32 else "") + ("_pdl" if dependent else ""))
    return _row(name, nbytes, t, sets, peak, split_k=split_k)


def bench_rope(dtype, layout: str, rope_dim: int, peak=None, replays=20, check=None, dependent=False, **shape) -> dict:
    case = wl.rope_inputs(rope_dim=rope_dim, layout=layout, dtype=dtype, **shape)
    tokens, hq, dim = case["q"].shape
    hkv = case["k"].shape[1]
    nbytes = wl.rope_bytes(tokens, hq, hkv, dim, rope_dim, dtype)
    sets = 8
    dev = {key: (val.cuda() if torch.is_tensor(val) else val) for key, val in case.items()}
    kc = torch.full(case["cache_shape"], -999.0, dtype=dtype, device="cuda")
    vc = torch.full_like(kc, -999.0)
    qs = [dev["q"]] + [dev["q"].roll(s, 0) for s in range(1, sets)]

    def run(q):
        q_out = rope_gqa_paged_kv_append(q, dev["k"], dev["v"], dev["cos"], dev["sin"], dev["positions"], dev["page_table"],
                                         dev["sequence_ids"], kc, vc, page_size=case["page_size"], rope_dim=rope_dim,
                                         interleaved=False, kv_layout=layout, dependent_launch=dependent)
        return q_out, kc, vc  # the caches are outputs too (the gate checks the written slots and the sentinels)

    calls = [(lambda q=qs[i % sets]: run(q)) for i in range(24)]

    def mutate():
        for key in ("q", "k", "v"):
            dev[key].neg_()

    def poison(outputs):  # rotated Q is rewritten whole; the caches go back to the sentinel the gate counts
        for q_out, _, _ in outputs:
            q_out.fill_(float("nan"))
        kc.fill_(-999.0)
        vc.fill_(-999.0)

    t = graph_median_us(calls, replays, check=check, mutate=mutate, poison=poison)
    name = f"rope_kv_{str(dtype).split('.')[-1]}_{layout}_rd{rope_dim}_t{tokens}" + ("_pdl" if dependent else "")
    return _row(name, nbytes, t, sets, peak)


def bench_w4a16(m: int, k: int, n: int, group: int = 128, peak=None, replays=20, check=None, dependent=False) -> dict:
    nbytes = wl.w4a16_bytes(m, k, n, group)
    sets = rotation_for(nbytes, cap=48)
    x, packed, scales, _ = wl.w4a16_inputs(m, k, n, group)
    xd, sd = x.cuda(), scales.cuda()
    ps = [packed.cuda()] + [torch.randint(0, 256, packed.shape, dtype=torch.uint8, device="cuda") for _ in range(sets - 1)]
    ss = [sd] + [sd.clone() for _ in range(sets - 1)]
    outs = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in range(sets)]
    ncalls = _calls_per_graph(sets)
    calls = [(lambda i=i: w4a16_linear(xd, ps[i % sets], ss[i % sets], None, group_size=group, out=outs[i % sets],
                                       dependent_launch=dependent)) for i in range(ncalls)]
    t = graph_median_us(calls, replays, check=check, mutate=lambda: xd.neg_())
    return _row(f"w4a16_m{m}_k{k}_n{n}_g{group}" + ("_pdl" if dependent else ""), nbytes, t, sets, peak)


def bench_attention(context: int, tokens: int = 16, q_heads: int = 32, kv_heads: int = 8, head_dim: int = 128, page_size: int = 16,
                    dtype=torch.float16, peak=None, replays=20, check=None, dependent=False) -> dict:
    """Decode attention of ``tokens`` sequences, each ``context`` positions long, over one shared paged cache.  The
    rotating sets are disjoint page ranges of that cache (one page table per set), so every call reads K and V
    that the L2 has not seen for a whole rotation.  ``check(stage, (out, q, k_cache, v_cache, positions, table, ids))``
    sees call 0."""
    pages_per_seq = -(-context // page_size)
    nbytes = 2 * tokens * context * kv_heads * head_dim * dtype.itemsize + 2 * tokens * q_heads * head_dim * dtype.itemsize
    sets = rotation_for(nbytes, cap=48)
    g = torch.Generator(device="cuda").manual_seed(context)
    pages = sets * tokens * pages_per_seq
    kc = torch.randn(pages, page_size, kv_heads, head_dim, generator=g, device="cuda", dtype=dtype)
    vc = torch.randn(pages, page_size, kv_heads, head_dim, generator=g, device="cuda", dtype=dtype)
    q = torch.randn(tokens, q_heads, head_dim, generator=g, device="cuda", dtype=dtype)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(context)).reshape(sets, tokens, pages_per_seq).cuda()
    tables = [order[i].contiguous() for i in range(sets)]
    positions = torch.full((tokens,), context - 1, dtype=torch.int64, device="cuda")
    ids = torch.arange(tokens, dtype=torch.int64, device="cuda")
    ncalls = _calls_per_graph(sets)
    calls = [(lambda i=i: (paged_decode_attention(q, kc, vc, positions, tables[i % sets], ids, page_size=page_size,
                                                  dependent_launch=dependent), q, kc, vc, positions, tables[i % sets], ids))
             for i in range(ncalls)]
    t = graph_median_us(calls, replays, check=check, mutate=lambda: q.neg_(), poison=lambda outs: [o[0].fill_(float("nan")) for o in outs])
    name = f"paged_decode_attention_{str(dtype).split('.')[-1]}_t{tokens}_hq{q_heads}_hkv{kv_heads}_d{head_dim}_ctx{context}"
    return _row(name + ("_pdl" if dependent else ""), nbytes, t, sets, peak)


def bench_swiglu(rows: int, width: int, dtype=torch.float16, peak=None, replays=20, check=None, dependent=False) -> dict:
    nbytes = 3 * rows * width * dtype.itemsize
    sets = rotation_for(nbytes, cap=48)
    g = torch.Generator(device="cuda").manual_seed(width)
    ins = [torch.randn(rows, 2 * width, generator=g, device="cuda", dtype=dtype) for _ in range(sets)]
    ncalls = _calls_per_graph(sets)
    calls = [(lambda i=i: (swiglu(ins[i % sets], dependent_launch=dependent), ins[i % sets])) for i in range(ncalls)]
    t = graph_median_us(calls, replays, check=check, mutate=lambda: ins[0].neg_(), poison=lambda outs: [o[0].fill_(float("nan")) for o in outs])
    return _row(f"swiglu_{str(dtype).split('.')[-1]}_{rows}x{width}" + ("_pdl" if dependent else ""), nbytes, t, sets, peak)


def bench_chain(rank: int = 0, world: int = 1, layers: int = 4, peak=None, replays=20, group=None, exchange: str = "peer",
                dependent: bool = False, check=None, attention: bool = False) -> dict:
    """Decode-layer chain: ``layers`` layers with distinct weights (more than L2 in total) in one
    CUDA graph; reports the per-layer median.  With world > 1 every rank must call this.
    ``check(chain, outputs_of_last_layer)`` (optional) is run on the eager result before timing."""
    from .chain import ChainConfig, DecodeLayerChain
    from .timing import capture, replay_times_ms
    import statistics

    cfg = ChainConfig()
    chain = DecodeLayerChain(cfg, layers=layers, rank=rank, world=world, group=group, exchange=exchange,
                             dependent_launch=dependent, attention=attention)
    if check is not None:
        out = chain.run_layers()
        torch.cuda.synchronize()
        check(chain, out)
    graph = capture([chain.run_layers])
    times = replay_times_ms(graph, replays, 3)
    us = statistics.median(times) * 1e3 / layers
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([us], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        us = float(t.item())
    nbytes = cfg.algorithmic_bytes()
    if attention:  # K and V rows of every context position (position + 1 of them per sequence), q in, out, SwiGLU in and out
        ctx = int((chain.positions + 1).sum())
        nbytes += 2 * ctx * cfg.kv_heads * cfg.head_dim * 2 + 2 * cfg.tokens * cfg.hidden * 2 + 3 * cfg.tokens * cfg.mlp * 2
    name = (f"decode_layer_chain_fp16_t{cfg.tokens}_h{cfg.hidden}_ctx{cfg.context}" + ("_attention_swiglu" if attention else "")
            + ("_pdl" if dependent else ""))
    row = {"kernel": name, "us": round(us, 3),
           "bytes": nbytes, "gbps": round(nbytes / us * 1e-3, 1), "frac_of_8tbs": round(nbytes / us * 1e-3 / (NOMINAL_HBM_GBPS * world), 4),
           "n_gpus": world, "layers_in_graph": layers, "launches_per_layer": chain.launches_per_layer,
           "exchange": exchange if world > 1 else "none", "dependent_launch": dependent, "gated": check is not None}
    if peak:
        row["frac_of_measured"] = round(nbytes / us * 1e-3 / (peak * world), 4)
    del graph
    if chain.arena is not None:
        torch.cuda.synchronize()
        import torch.distributed as dist
        dist.barrier(group=group)
        chain.arena.close()
    return row


def table(which=("rmsnorm", "gemv", "rope", "w4a16"), peak=None, split_sweep=True) -> list[dict]:
    """The ungated table (command-line use); bench.py builds the gated one row by row."""
    rows = [bench_noop()]
    if "rmsnorm" in which:
        for dtype in (torch.float32, torch.bfloat16):
            for r in (256, 4096):
                rows.append(bench_rmsnorm(r, 4096, dtype, peak))
    if "gemv" in which:
        for layout in ("KN", "NK"):
            for n in (4096, 14336):
                for m in (1, 4, 16):
                    for s in ((0, 1, 2, 4, 8) if split_sweep else (0,)):
                        rows.append(bench_gemv(m, 4096, n, layout, s, True, peak))
                if n == 14336:  # the strict-FP32 alternative of the tensor-core path, for comparison
                    rows.append(bench_gemv(16, 4096, n, layout, 0, True, peak, strict_fp32=True))
    if "rope" in which:
        for dtype in (torch.float32, torch.bfloat16):
            for layout in ("NHD", "HND"):
                for rd in (64, 128):
                    rows.append(bench_rope(dtype, layout, rd, peak))
    if "w4a16" in which:
        for n in (4096, 14336):
            for m in (1, 16):
                rows.append(bench_w4a16(m, 4096, n, 128, peak))
    if "chain" in which:
        rows.append(bench_chain(peak=peak))
    return rows


def one(argv: list[str]) -> dict:
    """``--one rmsnorm ROWS HIDDEN f32|bf16|f16`` | ``--one gemv M K N KN|NK SPLIT [strict]`` |
    ``--one rope f32|bf16 NHD|HND ROPE_DIM`` | ``--one w4a16 M K N GROUP`` | ``--one attention CONTEXT [TOKENS]`` |
    ``--one swiglu ROWS WIDTH``; few replays (for profilers)."""
    dtypes = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
    op, rest = argv[0], argv[1:]
    if op == "rmsnorm":
        return bench_rmsnorm(int(rest[0]), int(rest[1]), dtypes[rest[2]], replays=3)
    if op == "gemv":
        return bench_gemv(int(rest[0]), int(rest[1]), int(rest[2]), rest[3], int(rest[4]), replays=3,
                          strict_fp32=len(rest) > 5 and rest[5] == "strict")
    if op == "rope":
        return bench_rope(dtypes[rest[0]], rest[1], int(rest[2]), replays=3)
    if op == "w4a16":
        return bench_w4a16(int(rest[0]), int(rest[1]), int(rest[2]), int(rest[3]), replays=3)
    if op == "attention":
        return bench_attention(int(rest[0]), tokens=int(rest[1]) if len(rest) > 1 else 16, replays=3)
    if op == "swiglu":
        return bench_swiglu(int(rest[0]), int(rest[1]), replays=3)
    raise SystemExit(one.__doc__)


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[1] == "--one":
        print(json.dumps(one(sys.argv[2:])))
        raise SystemExit(0)
    chosen = tuple(sys.argv[1:]) or ("rmsnorm", "gemv", "rope", "w4a16", "chain")
    for row in table(chosen):
        print(json.dumps(row))
