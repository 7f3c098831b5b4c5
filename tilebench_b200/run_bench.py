"""Command-line runner: one operator, every case, torch baseline + the cuda backend.

    python -m tilebench_b200.run_bench --gpu B200 --operator dequant_int4_group
    python -m tilebench_b200.run_bench --gpu B200 --operator gemm_w4a16 --case-indices 0,3 --cpu-baseline

Same surface and result layout as the reference CLI (scripts/run_bench.py:199-447, tilebench/paths.py:111-136):
the raw timing JSON at results/<gpu>/logs/time_measurement_logs/<op>_<mode>_<backends>.json (where the reference's
scripts/visualize.py looks for it), the provenance sidecar under the same name in results/<gpu>/logs/provenance/,
a summary CSV at results/<gpu>/csv/<op>_<mode>.csv with
`params, dtype, torch_ms, cuda_ms, speedup_cuda`, extended here by the derived columns the north star
asks for (GB/s or TFLOPS and the fraction of the HBM / tensor roofline, against the datasheet table and
against the peaks measured on the box).  An empty result set never overwrites existing logs.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import sys
from pathlib import Path

import yaml

from tilebench_b200 import provenance
from tilebench_b200.backends import MODES, backend_tag, parse_backends
from tilebench_b200.core.metrics import compute_derived, load_peak_config
from tilebench_b200.paths import list_operators, operator_config, results_csv_dir, results_logs_dir

_BACKEND_LABEL = {"cuda": "CUDA"}
_SPEEDUP_CODE = {"cuda": "cu"}


def log_name(operator: str, mode: str, backends) -> str:
    """<operator>_<mode>_<backend tag>.json: one name for the timing log and its provenance sidecar."""
    if mode not in MODES:
        raise ValueError(f"unknown mode {mode!r}; choose from {', '.join(MODES)}")
    return f"{operator}_{mode}_{backend_tag(backends)}.json"


def timing_log_path(gpu: str, operator: str, mode: str, backends) -> Path:
    return results_logs_dir(gpu) / "time_measurement_logs" / log_name(operator, mode, backends)


def provenance_log_path(gpu: str, operator: str, mode: str, backends) -> Path:
    return results_logs_dir(gpu) / "provenance" / log_name(operator, mode, backends)


def fmt_params(row: dict) -> str:
    return ", ".join(f"{k}={row['params'][k]}" for k in sorted(row["params"]))


def _jsonable(o):
    if isinstance(o, float) and (math.isnan(o) or math.isinf(o)):
        return None
    if isinstance(o, dict):
        return {k: _jsonable(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_jsonable(v) for v in o]
    return o


def build_overrides(args) -> dict:
    ov = {}
    if args.warmup is not None:
        ov["warmup"] = args.warmup
    if args.repeat is not None:
        ov["repeat"] = args.repeat
    if args.no_cuda_graph:
        ov["use_cuda_graph"] = False
    if args.no_flush_l2:
        ov["flush_l2"] = False
    if args.autotune:
        ov["autotune"] = True
    if args.cpu_baseline:
        ov["cpu_baseline"] = True
    if args.seed is not None:
        ov["seed"] = args.seed
    if args.timer:
        ov["timer"] = args.timer
    if args.case_indices:
        ov["case_indices"] = [int(x) for x in args.case_indices.split(",") if x.strip()]
    return ov


def write_outputs(gpu: str, operator: str, mode: str, active, results, prov, out_root: Path | None = None):
    """Timing JSON + provenance sidecar + summary CSV.  Returns the three paths."""
    metrics_cfg = yaml.safe_load(open(operator_config(operator))).get("metrics", {})
    peak = load_peak_config(gpu)
    logs = (out_root / gpu / "logs") if out_root else results_logs_dir(gpu)
    csvd = (out_root / gpu / "csv") if out_root else results_csv_dir(gpu)
    timing = logs / "time_measurement_logs" / log_name(operator, mode, active)
    sidecar = logs / "provenance" / log_name(operator, mode, active)
    for d in (timing.parent, sidecar.parent, csvd):
        d.mkdir(parents=True, exist_ok=True)
    csv_path = csvd / f"{operator}_{mode}.csv"
    for r in results:
        r["derived"] = compute_derived(r, metrics_cfg, peak)
    timing.write_text(json.dumps(_jsonable(results), indent=1))
    sidecar.write_text(json.dumps(prov, indent=1))
    with open(csv_path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["params", "dtype", "torch_ms"] + [f"{b}_ms" for b in active] + [f"speedup_{b}" for b in active]
                   + ["cuda_GBs", "cuda_tflops", "cuda_pct_peak_bw", "cuda_pct_measured_bw", "cuda_pct_peak_tflops",
                      "cuda_pct_measured_tflops", "cpu_ms"])
        for r in results:
            d = r["derived"].get("cuda", {})
            def g(k):
                return f"{d[k]:.2f}" if k in d else ""
            w.writerow([fmt_params(r), r["dtype"], f"{r['torch_ms']:.4f}"] + [f"{r[f'{b}_ms']:.4f}" for b in active]
                       + [f"{r[f'speedup_{b}']:.2f}" for b in active]
                       + [g("bandwidth_GBs"), g("tflops"), g("pct_peak_bw"), g("pct_measured_bw"), g("pct_peak_tflops"),
                          g("pct_measured_tflops"), f"{r['cpu_ms']:.3f}" if "cpu_ms" in r else ""])
    return timing, sidecar, csv_path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--gpu", default="B200", help="result namespace results/<gpu>/ and peak table data/peak_performance/<gpu>.json")
    ap.add_argument("--operator", required=True, choices=list_operators())
    ap.add_argument("--tile-language", default=None, help="comma-separated backends (cuda); torch always runs")
    ap.add_argument("--warmup", type=int)
    ap.add_argument("--repeat", type=int)
    ap.add_argument("--autotune", action="store_true", help="kept for layout parity: the cuda backend has a static config table")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--no-flush-l2", action="store_true")
    ap.add_argument("--flush-mb", type=float, default=None,
                    help="size of the L2 eviction buffer in MB (default: 2x L2; 64 reproduces the reference's published B200 protocol)")
    ap.add_argument("--timer", choices=["events", "kernel"], default=None,
                    help="events: CUDA-event pair (default); kernel: summed kernel durations from the profiler, as the reference's Proton timer reports")
    ap.add_argument("--cpu-baseline", action="store_true", help="also time the PyTorch reference on the host CPU cores")
    ap.add_argument("--case-indices", default=None)
    ap.add_argument("--seed", type=int)
    ap.add_argument("--output-root", default=None, help="write under this directory instead of results/")
    args = ap.parse_args(argv)

    from tilebench_b200.core.engine import run_benchmark_suite
    if args.flush_mb:
        from tilebench_b200.core import timer
        timer.set_flush_bytes(int(args.flush_mb * (1 << 20)))
    active = parse_backends(args.tile_language)
    mode = MODES[1] if args.autotune else MODES[0]
    prov = provenance.collect(args.gpu)
    prov["flush_mb"] = args.flush_mb
    results = run_benchmark_suite(args.operator, build_overrides(args), active)
    if not results:
        print("No case produced a result; existing logs are left untouched.", file=sys.stderr)
        return 1
    timing, sidecar, csv_path = write_outputs(args.gpu, args.operator, mode, active, results, prov,
                                              Path(args.output_root) if args.output_root else None)
    width = max(len(fmt_params(r)) for r in results)
    print(f"\n{'Params':<{width}} | {'Dtype':>10} | {'Torch(ms)':>10} | {'CUDA(ms)':>10} | {'Speedup':>8} | ok")
    for r in results:
        print(f"{fmt_params(r):<{width}} | {r['dtype']:>10} | {r['torch_ms']:10.4f} | {r['cuda_ms']:10.4f} | "
              f"{r['speedup_cuda']:8.2f} | {r['cuda_ok']}{'' if r['cuda_ok'] else '  ' + str(r['cuda_err'])[:80]}")
    print(f"Timing log      -> {timing}\nProvenance      -> {sidecar}\nSummary CSV     -> {csv_path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
