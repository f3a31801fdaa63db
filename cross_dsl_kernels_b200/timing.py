"""CUDA-graph timing: the "per-call median" metric.

A graph holding ``len(calls)`` back-to-back launches is replayed several times;
each replay is timed with CUDA events on the capturing stream and the median
replay time is divided by the number of calls (the method of upstream's
benchmarks/common.py:129-153).  Callers pass one closure per call so that
consecutive calls can use different buffer sets: when the sets together exceed
the 126 MB L2, every call streams from HBM instead of hitting lines the
previous call left behind.
"""

from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Callable, Sequence

import torch

L2_BYTES = 126 * 1024 * 1024


def rotation_for(working_set_bytes: int, target_bytes: int = 3 * L2_BYTES, cap: int = 64) -> int:
    """How many distinct buffer sets make consecutive calls miss L2."""
    return max(1, min(cap, -(-target_bytes // max(1, working_set_bytes))))


def capture(calls: Sequence[Callable[[], object]], stream: torch.cuda.Stream | None = None, outputs: list | None = None
            ) -> torch.cuda.CUDAGraph:
    """Warm the calls up, then capture them back to back into one graph.  ``outputs`` (optional list) receives
    what each captured call returned: tensors in the graph's private pool that every replay rewrites."""
    stream = stream or torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for fn in calls:  # warm-up outside capture: loads modules, sizes allocator pools
            fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for fn in calls:
            out = fn()
            if outputs is not None:
                outputs.append(out)
    return graph


def replay_times_ms(graph: torch.cuda.CUDAGraph, replays: int = 20, warmup: int = 3) -> list[float]:
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return times


def _poison(obj) -> None:
    if torch.is_tensor(obj):
        if obj.is_floating_point():
            obj.fill_(float("nan"))
    elif isinstance(obj, (tuple, list)):
        for item in obj:
            _poison(item)


def graph_median_us(calls: Sequence[Callable[[], object]], replays: int = 20, warmup: int = 3,
                    check: Callable[[str, object], None] | None = None, mutate: Callable[[], None] | None = None,
                    poison: Callable[[list], None] | None = None) -> dict:
    """Per-call median of a graph of back-to-back calls.

    ``check(stage, output_of_call_0)`` (optional) is the gate, and it raises on a mismatch.  It runs three times:
    ``"eager"`` on the first call's result before anything is timed; ``"poisoned"`` on the captured output of call 0
    after a replay whose output buffers were filled with NaN first (a replay that silently does nothing fails);
    ``"changed"`` after ``mutate()`` has changed the INPUT contents of call 0 in place at their fixed addresses and
    the graph was replayed again (a graph that baked values in instead of addresses fails).  ``mutate`` is then
    called a second time and must restore the inputs.  ``poison(outputs)`` replaces the default (NaN into every
    floating-point output) for ops whose outputs are not all freshly written, such as a cache that keeps a sentinel.  This is the discipline of upstream's
    benchmarks/compare.py:28-41, 247-258 and benchmarks/gemv_cuda_benchmark.py:97-126."""
    if check is not None:
        first = calls[0]()
        torch.cuda.synchronize()
        check("eager", first)
    outputs: list = []
    graph = capture(calls, outputs=outputs)
    if check is not None:
        poison = poison or _poison
        poison(outputs)
        graph.replay()
        torch.cuda.synchronize()
        check("poisoned", outputs[0])
        if mutate is not None:
            mutate()
            poison(outputs)
            graph.replay()
            torch.cuda.synchronize()
            check("changed", outputs[0])
            mutate()
    times = replay_times_ms(graph, replays, warmup)
    per_call = [t * 1e3 / len(calls) for t in times]
    ordered = sorted(per_call)
    return {
        "median_us": statistics.median(per_call),
        "p10_us": ordered[max(0, int(0.1 * len(ordered)) - 0)],
        "p90_us": ordered[min(len(ordered) - 1, int(0.9 * len(ordered)))],
        "min_us": ordered[0],
        "calls_per_graph": len(calls),
        "replays": replays,
        "gated": check is not None,
    }


def lockstep_replays(local_ms: float, steps: int, *, device="cuda", group=None, target_ms: float = 1000.0,
                     cap: int = 5000) -> int:
    """How many extra replays of a step graph give about ``target_ms`` of load -- the SAME number on every rank.

    A step graph that holds collectives must be replayed equally often by all ranks: a rank that stops early
    leaves the others waiting in a collective for ever.  So the count is derived from the slowest rank's
    measured time for ``steps`` replays (MAX all-reduce), never from a rank's own wall clock."""
    import torch.distributed as dist

    ms = torch.tensor([float(local_ms)], device=device, dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
    per_step = max(float(ms.item()), 1e-3) / max(1, steps)
    return int(min(float(cap), max(1.0, target_ms / per_step)))


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0, period_ms: int = 100):
        # nvidia-smi numbers GPUs by PCI order, CUDA by CUDA_VISIBLE_DEVICES: address the GPU by its UUID
        # (a read-only query), falling back to the ordinal when the UUID cannot be had
        ident = str(device_index)
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            pass
        self.cmd = ["nvidia-smi", f"--id={ident}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                    "-lms", str(period_ms)]
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self

        def pump():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 7:
                    self.rows.append(parts)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=5)

    def summary(self) -> dict:
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in self.rows:
            try:
                clocks.append(float(row[0]))
                max_clock = float(row[1])
            except ValueError:
                continue
            for name, flag in zip(names, row[3:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }
