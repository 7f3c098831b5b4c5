"""Device-side timing of one operator call.

Protocol of the reference timer (tilebench/core/timer.py:208-284): `warmup` untimed calls, then
`repeat` timed calls, each preceded — outside the timed region — by a write of 2x the L2 size so
the call starts cold; with `use_cuda_graph` the call is captured once and the replay is timed
(capture failure falls back to eager, as in timer.py:129-143).  The reference sums kernel
durations with the Proton profiler.  Here the timed quantity is a CUDA-event pair on the launching
stream: in graph mode the two events are event-record NODES of the captured graph, directly before
and after the operator's kernels, so the host-side launch gap stays outside the measurement; in
eager mode the pair brackets the Python call and very short operators carry a few microseconds of
launch gap.  `report_benchmark_batched` amortises that gap for roofline numbers by timing
back-to-back calls on rotating buffers whose combined footprint exceeds L2.
"""
from __future__ import annotations

import statistics
from typing import Any, Callable, Sequence

import torch

from tilebench_b200.hardware import B200_L2_BYTES, last_level_cache_bytes

DEFAULT_WARMUP = 1
DEFAULT_REPEAT = 3

_flush_buf: torch.Tensor | None = None
_flush_bytes_override: int | None = None


def set_flush_bytes(nbytes: int | None) -> None:
    """Override the size of the eviction buffer (None = 2x the last-level cache).  The reference's published B200
    rows were taken with a fixed 64 MB buffer, half of that GPU's L2 (docs/developer_guide.md:432-433); this
    switch reproduces that protocol for side-by-side tables."""
    global _flush_bytes_override
    _flush_bytes_override = int(nbytes) if nbytes else None


def effective_use_cuda_graph(requested: bool) -> bool:
    return bool(requested)


def timing_mode(requested: bool, timer: str = "events") -> dict[str, Any]:
    eff = effective_use_cuda_graph(requested)
    return {"requested_use_cuda_graph": bool(requested), "effective_use_cuda_graph": eff,
            "timing_execution_mode": "graph" if eff else "eager", "timing_note": None,
            "timer": "kernel_time_sum" if timer == "kernel" else "cuda_events"}


def flush_buffer_bytes() -> int:
    """2x the last-level cache (B200: 2 x 126.5 MB = 253 MB), unless set_flush_bytes() overrides it."""
    if _flush_bytes_override:
        return _flush_bytes_override
    return 2 * (last_level_cache_bytes() or B200_L2_BYTES)


def flush_l2_cache() -> None:
    """Evict L2 by writing a buffer twice its size (enqueued on the current stream, no sync)."""
    global _flush_buf
    numel = flush_buffer_bytes() // 4
    if _flush_buf is None or _flush_buf.numel() != numel:
        _flush_buf = torch.empty(numel, device="cuda", dtype=torch.float32)
    _flush_buf.fill_(1.0)


def _prepare_runner(f: Callable, args: Sequence, kwargs: dict, use_cuda_graph: bool):
    """Returns (runner, mode, events).  Graph mode: 3 eager calls on a side stream, then capture with an
    event-record node on either side of the call; `events` is that pair, or None when the events have to
    be recorded around the runner by the caller."""
    if not use_cuda_graph:
        return (lambda: f(*args, **kwargs)), "eager", None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                f(*args, **kwargs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        try:
            ev0 = torch.cuda.Event(enable_timing=True, external=True)
            ev1 = torch.cuda.Event(enable_timing=True, external=True)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                ev0.record()
                f(*args, **kwargs)
                ev1.record()
            graph.replay()
            torch.cuda.synchronize()
            ev0.elapsed_time(ev1)                      # raises if the events did not become timing nodes
            return graph.replay, "graph", (ev0, ev1)
        except Exception:
            torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            f(*args, **kwargs)
        return graph.replay, "graph", None
    except Exception:
        torch.cuda.synchronize()
        return (lambda: f(*args, **kwargs)), "eager", None


def _kernel_time_ms(runner: Callable) -> float:
    """Summed device time of the kernels `runner` launches, from the CUPTI activity records torch.profiler
    collects — the quantity the reference's Proton-based timer reports (tilebench/core/timer.py:208-284), free
    of launch gaps and of the cost of event records."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        runner()
        torch.cuda.synchronize()
    total_us = 0.0
    for evt in prof.events():
        if "memcpy" in evt.name.lower() or "memset" in evt.name.lower():
            continue
        total_us += float(getattr(evt, "device_time_total", 0.0) or getattr(evt, "cuda_time_total", 0.0) or 0.0)
    if total_us <= 0.0:
        raise RuntimeError("the profiler recorded no kernel time")
    return total_us / 1e3


def report_benchmark(f: Callable, args: Sequence = (), kwargs: dict | None = None, *, warmup: int = DEFAULT_WARMUP,
                     repeat: int = DEFAULT_REPEAT, use_cuda_graph: bool = False, flush_l2: bool = True,
                     timer: str = "events", **_ignored) -> dict[str, Any]:
    """Time `f(*args, **kwargs)`; returns {"mean", "median", "min", "max", "samples", "mode", "timer"} in ms.
    timer="events": a CUDA-event pair around the call (event-record nodes inside the graph in graph mode).
    timer="kernel": summed kernel durations from the profiler's activity records (what Proton gives the
    reference); falls back to events, and says so, if the profiler yields nothing."""
    kwargs = kwargs or {}
    do_flush = flush_l2
    for _ in range(max(0, warmup)):
        if do_flush:
            flush_l2_cache()
        f(*args, **kwargs)
    torch.cuda.synchronize()
    runner, mode, graph_events = _prepare_runner(f, args, kwargs, use_cuda_graph)
    samples = []
    if timer == "kernel":
        try:
            for _ in range(max(1, repeat)):
                if do_flush:
                    flush_l2_cache()
                torch.cuda.synchronize()
                samples.append(_kernel_time_ms(runner))
            return {"mean": statistics.fmean(samples), "median": statistics.median(samples), "min": min(samples),
                    "max": max(samples), "samples": samples, "mode": mode, "timer": "kernel_time_sum"}
        except Exception:
            samples = []
            torch.cuda.synchronize()
    for _ in range(max(1, repeat)):
        if do_flush:
            flush_l2_cache()
        if graph_events is not None:
            runner()
            torch.cuda.current_stream().synchronize()
            samples.append(graph_events[0].elapsed_time(graph_events[1]))
            continue
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end))
    return {"mean": statistics.fmean(samples), "median": statistics.median(samples), "min": min(samples),
            "max": max(samples), "samples": samples, "mode": mode, "timer": "cuda_events"}


def report_benchmark_batched(launchers: Sequence[Callable[[], Any]], *, warmup: int = 3, repeat: int = 20) -> dict[str, Any]:
    """Time back-to-back calls of `launchers` (one per rotating buffer set; together the sets must
    exceed L2 so no call finds its inputs cached).  One event pair brackets a full rotation; the
    per-call time is rotation time / len(launchers)."""
    n = len(launchers)
    for _ in range(max(0, warmup)):
        for fn in launchers:
            fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(max(1, repeat)):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for fn in launchers:
            fn()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end) / n)
    return {"mean": statistics.fmean(samples), "median": statistics.median(samples), "min": min(samples),
            "max": max(samples), "samples": samples, "mode": f"batched x{n}"}
