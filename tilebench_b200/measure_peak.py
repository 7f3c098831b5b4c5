"""Measured roofline denominators of the GPU this runs on: HBM copy bandwidth and the library GEMM rate of
every tensor-core input type the path uses.

    python -m tilebench_b200.measure_peak [--kinds bf16,fp16,tf32,fp8_e4m3fn,int8] [--size 8192]
                                          [--sustained-s 4] [--write] [--json PATH]

The reference takes its own denominators the same way (scripts/measure_peak.py:134-256: device copies for
HBM, torch.matmul for fp32/bf16/fp16, torch._scaled_mm for e4m3 with unit scales, torch._int_mm for int8).
Here every GEMM kind is measured twice — as a burst (best of a few back-to-back calls on a cool board: the
denominator for a kernel timed alone) and as a loop of `--sustained-s` seconds (the board settles at its
power cap: the denominator for a kernel timed inside a long step) — with the SM clock and the clock-event
reasons sampled during the loop, so a throttled or clock-locked measurement can be told from a good one.
`--write` stores the result in the `measured` block of data/peak_performance/B200.json, which
core/metrics.py reads for the pct_measured_* columns; bench.py calls `measure()` live for the types the
driver's own peak file lacks (fp8, int8).  These are library kernels used as yardsticks, never on the path.
"""
from __future__ import annotations

import argparse
import datetime
import json
import sys
import time

KINDS = ("bf16", "fp16", "tf32", "fp8_e4m3fn", "int8")


def _gemm_call(kind: str, size: int, device):
    """A zero-argument launcher of one size^3 library GEMM of `kind`, and its operation count."""
    import torch
    n = size
    if kind in ("bf16", "fp16"):
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        a, b = torch.randn(n, n, device=device, dtype=dt), torch.randn(n, n, device=device, dtype=dt)
        out = torch.empty(n, n, device=device, dtype=dt)
        return (lambda: torch.matmul(a, b, out=out)), 2.0 * n ** 3
    if kind == "tf32":
        a, b = torch.randn(n, n, device=device), torch.randn(n, n, device=device)
        out = torch.empty(n, n, device=device)

        def run():
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                torch.matmul(a, b, out=out)
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
        return run, 2.0 * n ** 3
    if kind == "fp8_e4m3fn":
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()         # column-major, as _scaled_mm wants
        one = torch.tensor(1.0, device=device)
        return (lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)), 2.0 * n ** 3
    if kind == "int8":
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        return (lambda: torch._int_mm(a, b)), 2.0 * n ** 3
    raise ValueError(f"unknown kind {kind!r}; choose from {KINDS}")


def _event_ms(torch, fn, calls: int) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(calls):
        fn()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / calls


def measure_gemm(kind: str, size: int = 8192, burst_reps: int = 10, sustained_s: float = 4.0, sampler=None, device=None) -> dict:
    """{"tflops": burst, "tflops_sustained": ..., "clocks": {...}} for one kind (TOPS for int8)."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    fn, ops = _gemm_call(kind, size, device)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    burst_ms = min(_event_ms(torch, fn, 1) for _ in range(burst_reps))
    out = {"kind": kind, "size": size, "tflops": ops / burst_ms / 1e9, "burst_ms": burst_ms}
    if sustained_s > 0:
        since = sampler.mark() if sampler else 0
        if sampler:
            sampler.busy(True)
        batch = max(1, int(0.25e3 / burst_ms))                   # about a quarter of a second per event pair
        t0, total_ms, calls = time.perf_counter(), 0.0, 0
        while time.perf_counter() - t0 < sustained_s:
            total_ms += _event_ms(torch, fn, batch) * batch
            calls += batch
        if sampler:
            sampler.busy(False)
            out["clocks"] = sampler.snapshot(since)
        out["tflops_sustained"] = ops * calls / total_ms / 1e9
        out["sustained_s"] = total_ms / 1e3
    return out


def measure_hbm_copy(nbytes: int = 2 << 30, reps: int = 10, device=None) -> dict:
    """STREAM-style copy: read + written bytes / best time of `reps` copies of `nbytes`."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    a = torch.empty(nbytes, dtype=torch.uint8, device=device).fill_(1)
    b = torch.empty_like(a)
    for _ in range(3):
        b.copy_(a)
    torch.cuda.synchronize()
    ms = min(_event_ms(torch, lambda: b.copy_(a), 1) for _ in range(reps))
    return {"hbm_GBs": 2.0 * nbytes / ms / 1e6, "copy_bytes": nbytes, "ms": ms}


def measure(kinds=KINDS, size: int = 8192, sustained_s: float = 4.0, hbm: bool = True) -> dict:
    """All requested denominators of the current device, with provenance."""
    import torch
    from tilebench_b200.clocks import ClockSampler
    index = torch.cuda.current_device()
    sampler = ClockSampler(index, period_s=0.05).start()
    res = {"gpu": torch.cuda.get_device_name(index), "torch": torch.__version__,
           "when": datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ"),
           "how": f"library GEMM {size}^3: best of 10 single calls (burst) and a {sustained_s:g} s loop (sustained); "
                  "bf16/fp16/tf32 torch.matmul, e4m3 torch._scaled_mm with unit scales, int8 torch._int_mm",
           "gemm": {}}
    if hbm:
        res["hbm"] = measure_hbm_copy()
    # all bursts first, on a board that is still cool; then the loops that take it to its power cap
    for kind in kinds:
        try:
            res["gemm"][kind] = measure_gemm(kind, size, sustained_s=0.0)
        except Exception as e:                                  # a kind this torch build lacks must not lose the others
            res["gemm"][kind] = {"kind": kind, "error": f"{type(e).__name__}: {e}"}
    for kind in kinds:
        if "error" in res["gemm"][kind] or sustained_s <= 0:
            continue
        loop = measure_gemm(kind, size, burst_reps=1, sustained_s=sustained_s, sampler=sampler)
        res["gemm"][kind].update({k: loop[k] for k in ("tflops_sustained", "sustained_s", "clocks") if k in loop})
    sampler.stop()
    return res


def merge_into_peak_file(result: dict, path=None) -> dict:
    """Folds a measure() result into the `measured` block of the peak file (burst under "tflops", the loop
    under "tflops_sustained"); returns the new block."""
    from tilebench_b200.paths import PEAK_PERFORMANCE_ROOT
    path = path or (PEAK_PERFORMANCE_ROOT / "B200.json")
    with open(path) as f:
        cfg = json.load(f)
    block = cfg.setdefault("measured", {})
    if "hbm" in result:
        block["hbm_GBs"] = round(result["hbm"]["hbm_GBs"], 1)
    for kind, r in result.get("gemm", {}).items():
        if "tflops" not in r:
            continue
        block.setdefault("tflops", {})[kind] = round(r["tflops"], 1)
        if "tflops_sustained" in r:
            block.setdefault("tflops_sustained", {})[kind] = round(r["tflops_sustained"], 1)
        if r.get("clocks"):
            block.setdefault("clocks", {})[kind] = r["clocks"]
    block["note"] = f"measured by tilebench_b200.measure_peak on {result.get('gpu')} at {result.get('when')} (torch {result.get('torch')}); {result.get('how')}"
    with open(path, "w") as f:
        json.dump(cfg, f, indent=2)
        f.write("\n")
    return block


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--kinds", default=",".join(KINDS))
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--sustained-s", type=float, default=4.0)
    ap.add_argument("--write", action="store_true", help="store the result in data/peak_performance/B200.json")
    ap.add_argument("--json", default=None, help="also write the full result to this file")
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("measure_peak needs a GPU", file=sys.stderr)
        return 2
    res = measure(tuple(k for k in args.kinds.split(",") if k), args.size, args.sustained_s)
    text = json.dumps(res, indent=2)
    print(text)
    if args.json:
        with open(args.json, "w") as f:
            f.write(text + "\n")
    if args.write:
        merge_into_peak_file(res)
    return 0


if __name__ == "__main__":
    sys.exit(main())
