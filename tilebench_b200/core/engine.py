"""Benchmark engine: for every case of an operator, generate seeded inputs, run the PyTorch
reference, then verify-and-time each selected backend.

The control flow and the result keys follow the reference engine (tilebench/core/engine.py:103-498):
the reference output comes from `impl_torch.run`; a backend is run once, synchronised and verified
with the operator's tolerances, and *only if verified* timed; any exception becomes
`<backend>_ok=False, <backend>_err=str(e), <backend>_ms=nan` and the run continues; `block_size`
and `autotune` reach `run()` only when its signature names them.  Differences: the only backend
is `cuda`, inputs are seeded, and an optional `cpu_baseline` times the same reference on host
cores (a reported baseline, never a fallback).
"""
from __future__ import annotations

import importlib
import inspect
import os
import time

import torch
import yaml

from tilebench_b200.backends import GPU_BACKENDS, canonical_backends
from tilebench_b200.core.dtypes import resolve_dtype
from tilebench_b200.core.timer import DEFAULT_REPEAT, DEFAULT_WARMUP, report_benchmark, timing_mode
from tilebench_b200.core.verifier import config_tolerance, verify
from tilebench_b200.data.tensors import SEED0, expand_cases, get_generator, infer_problem_size
from tilebench_b200.hardware import detect_arch
from tilebench_b200.paths import list_operators, operator_config

HAS_CUDA = torch.cuda.is_available()
DEFAULT_ENABLED_BACKENDS = GPU_BACKENDS
OPERATOR_PACKAGE = "tilebench_b200.benchmarks.operators"


def _sync():
    if HAS_CUDA:
        torch.cuda.synchronize()


def _run_kwargs(fn, block_size, autotune):
    sig = inspect.signature(fn).parameters
    kw = {}
    if "block_size" in sig:
        kw["block_size"] = block_size
    if "autotune" in sig:
        kw["autotune"] = autotune
    return kw


def _to_cpu(x):
    return x.cpu() if isinstance(x, torch.Tensor) else x


def time_cpu_reference(run, inputs, repeat: int = 3) -> dict:
    """Wall-clock ms of the PyTorch reference on host cores (all threads), 1 warm-up + `repeat`."""
    cpu_inputs = tuple(_to_cpu(x) for x in inputs)
    torch.set_num_threads(os.cpu_count() or 1)
    run(*cpu_inputs)
    samples = []
    for _ in range(max(1, repeat)):
        t0 = time.perf_counter()
        run(*cpu_inputs)
        samples.append((time.perf_counter() - t0) * 1e3)
    return {"mean": sum(samples) / len(samples), "samples": samples, "cores": torch.get_num_threads()}


def run_benchmark_suite(operator_name, benchmark_overrides=None, enabled_backends=None, logs_dir=None):
    """Run every case of `operator_name`; returns one result dict per case."""
    with open(operator_config(operator_name)) as f:
        config = yaml.safe_load(f)

    enabled = set(DEFAULT_ENABLED_BACKENDS if enabled_backends is None else canonical_backends(enabled_backends))
    impl_torch = importlib.import_module(f"{OPERATOR_PACKAGE}.{operator_name}.impl_torch")
    impl_cuda = None
    if "cuda" in enabled:
        try:
            impl_cuda = importlib.import_module(f"{OPERATOR_PACKAGE}.{operator_name}.impl_cuda")
        except ImportError as e:
            print(f"  cuda import skipped: {e}")
    else:
        print("  cuda not selected (--tile-language)")

    generate_inputs = get_generator(operator_name)
    bench_cfg = dict(config.get("benchmark", {}))
    bench_cfg.update(benchmark_overrides or {})
    warmup = int(bench_cfg.get("warmup", DEFAULT_WARMUP))
    repeat = int(bench_cfg.get("repeat", DEFAULT_REPEAT))
    autotune = bool(bench_cfg.get("autotune", False))
    use_cuda_graph = bool(bench_cfg.get("use_cuda_graph", False))
    flush = bool(bench_cfg.get("flush_l2", False))
    cpu_baseline = bool(bench_cfg.get("cpu_baseline", False))
    timer_kind = str(bench_cfg.get("timer", "events"))
    verify_atol, verify_rtol = config_tolerance(config.get("verify", {}), detect_arch() if HAS_CUDA else None)
    timing = timing_mode(use_cuda_graph, str(bench_cfg.get("timer", "events"))) if HAS_CUDA else None

    cases = expand_cases(operator_name, config)
    case_indices = bench_cfg.get("case_indices")
    if case_indices is not None:
        for idx in case_indices:
            if idx < 0 or idx >= len(cases):
                raise ValueError(f"case index {idx} out of range for {len(cases)} generated cases")
        cases = [cases[i] for i in case_indices]
    op_index = list_operators().index(operator_name) if operator_name in list_operators() else 0

    def _bench(fn, args, kw=None):
        return report_benchmark(fn, args, kwargs=kw or {}, warmup=warmup, repeat=repeat,
                                use_cuda_graph=use_cuda_graph, flush_l2=flush, timer=timer_kind)

    results = []
    for case_idx, case in enumerate(cases):
        params = {k: v for k, v in case.items() if k not in ("dtype", "block_size")}
        dtype_str = case.get("dtype", "fp32")
        dtype = resolve_dtype(dtype_str)
        block_size = case.get("block_size", 1024)
        seed = int(bench_cfg.get("seed", SEED0)) + 1000 * op_index + case_idx
        print(f"Running case: {params}, dtype={dtype_str}, seed={seed}")

        try:
            inputs = generate_inputs(**params, dtype=dtype, seed=seed)
        except (RuntimeError, TypeError, ValueError) as e:
            print(f"  Skipped: input generation failed ({type(e).__name__}: {e})")
            continue
        try:
            ref_output = impl_torch.run(*inputs)
            _sync()
        except (RuntimeError, TypeError, ValueError) as e:
            print(f"  Skipped: torch reference failed ({type(e).__name__}: {e})")
            continue

        torch_stats = _bench(impl_torch.run, inputs) if HAS_CUDA else None
        torch_ms = torch_stats["mean"] if torch_stats else float("nan")

        cuda_cfg = None
        if impl_cuda is None or not HAS_CUDA:
            cuda_ok, cuda_ms, cuda_stats = False, float("nan"), None
            cuda_err = ("cuda backend requires an NVIDIA GPU" if impl_cuda is not None
                        else "cuda not selected or import failed")
            print(f"  cuda skipped ({cuda_err})")
        else:
            try:
                kw = _run_kwargs(impl_cuda.run, block_size, autotune)
                out = impl_cuda.run(*inputs, **kw)
                _sync()
                cuda_ok, cuda_err = verify(out, ref_output, atol=verify_atol, rtol=verify_rtol)
                cuda_cfg = getattr(impl_cuda, "get_last_config", lambda: None)() if autotune else None
                if not cuda_ok:
                    print(f"  cuda verification FAILED: {cuda_err}")
                cuda_stats = _bench(impl_cuda.run, inputs, kw) if cuda_ok else None
                cuda_ms = cuda_stats["mean"] if cuda_stats is not None else float("nan")
            except Exception as e:
                cuda_ok, cuda_err, cuda_ms, cuda_stats = False, str(e), float("nan"), None
                print(f"  cuda execution FAILED: {cuda_err}")

        row = {
            "params": params,
            "problem_size": infer_problem_size(operator_name, params),
            "dtype": dtype_str,
            "seed": seed,
            "torch_ms": torch_ms,
            "torch_stats": torch_stats,
            "cuda_ms": cuda_ms,
            "cuda_stats": cuda_stats or {},
            "cuda_ok": cuda_ok,
            "cuda_err": cuda_err,
            "cuda_autotune_cfg": cuda_cfg,
            "speedup_cuda": torch_ms / cuda_ms if cuda_ms > 0 else 0.0,
            "timing": timing,
        }
        if cpu_baseline:
            try:
                cpu = time_cpu_reference(impl_torch.run, inputs, repeat=min(repeat, 3))
                row.update(cpu_ms=cpu["mean"], cpu_stats=cpu)
            except Exception as e:
                row.update(cpu_ms=float("nan"), cpu_stats={"err": str(e)})
        results.append(row)
    return results
