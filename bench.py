#!/usr/bin/env python
"""Headline benchmark of the B200 `cuda` backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sections all|none]

Headline workload: per-channel int8 dequantisation, int8 [65536, 4096] x fp32 row scale -> bf16
(805,568,512 algorithmic bytes per pass; HBM-bound).  One step = one pass over the matrix.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank dequantises its own
65536-row shard (weak scaling, no data-path collective); the time is the max over ranks.

One JSON line is printed by rank 0.  Beyond the contract keys it carries
  roofline      achieved algorithmic GB/s of the dominant kernel / measured HBM peak
  e2e           the same metric through the host-buffer entry point (tilebench_b200.host_api) with pinned
                HOST tensors: H2D of w and scale, kernel, D2H of the result, all inside the timed region,
                pipelined over row chunks so that upload, kernel and download overlap
  cpu_baseline  the path's PyTorch reference formula on this host's cores, all threads (rank 0, N = 1)
  peaks         the roofline denominators in force: the driver-measured HBM / bf16 figures and the fp8 / int8
                library-GEMM rates measured live by tilebench_b200.measure_peak
  multi_gpu     (N > 1) BASELINE config 4, the N-partitioned W4A16 GEMM, timed before anything else heats the
                boards: compute-only, NCCL gather, push-kernel gather and fused gather, each beside the time
                of the whole problem on rank 0's GPU alone taken in the same process
  sections      the other workloads of the path (int4 dequant, W4A16 GEMM, FP8 block-scaled GEMM,
                the reference's own GEMM operators) with absolute rate and roofline fraction each
`--impl reference` times the path's PyTorch reference on the host CPU cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# stdout carries exactly one JSON line: main() points file descriptor 1 at stderr for the rest of the run, so
# whatever a library prints (NCCL's banner and NCCL_DEBUG output included) ends up on stderr untouched

ROWS, COLS = 65536, 4096
CFG4 = (4096, 8192, 57344)                        # M, K, N of BASELINE config 4 (N-partitioned W4A16 GEMM)
ALG_BYTES = ROWS * COLS * 3 + ROWS * 4            # int8 in + bf16 out + fp32 scales = 805,568,512
METRIC = "dequant_int8_channel_hbm_GBps"
UNIT = "GB/s"
WORKLOAD = "dequant_int8_channel rows=65536 cols=4096 int8->bf16 (BASELINE config 1, largest size)"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes per launch of tb200_k_dequant_int8_rowwise_bf16_wide on the headline workload, from one ncu
# capture of this workload (dram__bytes_read.sum + dram__bytes_write.sum): 268.73 MB read + 484.93 MB written.
# Less than the algorithmic bytes because the tail of the output is still in L2 when the kernel ends.
NCU_DRAM_BYTES_PER_LAUNCH = 753_666_304


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one for the same N."""
    return {"workload": WORKLOAD, "per_gpu_rows": ROWS, "cols": COLS,
            "l2": "805 MB touched per step, larger than the 126 MB L2; no flush needed",
            "parallelism": f"row shards x{world}, no collective"}


def load_peaks():
    """Driver-measured denominators (HBM copy, cuBLAS bf16 burst / sustained), else the stated fallback."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        peaks = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                 "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    else:
        peaks = {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
                 "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    src = f"cuBLAS bf16 8192^3, driver-{peaks['source']}" if peaks["source"] == "measured" else "fallback figure"
    peaks["tflops"] = {k: {"burst": peaks["bf16_tflops"], "sustained": peaks["bf16_tflops_sustained"], "source": src}
                       for k in ("bf16", "fp16")}
    return peaks


def fill_tensor_fractions(rows, peaks):
    """frac_of_tensor_peak (burst) and frac_of_sustained_peak of every tensor-bound row, from the measured
    library-GEMM rate of the row's input type."""
    for r in rows:
        kind = r.get("peak_kind")
        if not kind:
            continue
        scale = r.pop("peak_scale", 1)
        pk = peaks["tflops"].get(kind)
        if pk:
            r.update(frac_of_tensor_peak=r["TFLOPs"] / (scale * pk["burst"]), frac_of_sustained_peak=r["TFLOPs"] / (scale * pk["sustained"]),
                     tensor_peak=f"{'%d x ' % scale if scale != 1 else ''}{kind}: {pk['burst']:.0f} burst / {pk['sustained']:.0f} sustained TFLOPS, {pk['source']}")
        else:
            r.update(frac_of_tensor_peak=None, tensor_peak=f"{kind}: no measured peak available")
    return rows


def add_live_peaks(peaks, kinds=("fp8_e4m3fn", "int8", "tf32"), sustained_s=1.5, live=True):
    """The tensor-core denominators the driver's file lacks, measured now on this GPU with the library GEMMs
    (tilebench_b200.measure_peak: torch._scaled_mm e4m3, torch._int_mm, TF32 matmul; burst and a short loop).
    A kind that cannot be measured falls back to the block committed in data/peak_performance/B200.json."""
    from tilebench_b200 import measure_peak
    from tilebench_b200.core.metrics import load_peak_config
    committed = (load_peak_config("B200").get("measured") or {})
    for kind in kinds:
        try:
            if not live:
                raise RuntimeError("live probe switched off")
            r = measure_peak.measure_gemm(kind, 8192, sustained_s=sustained_s)
            peaks["tflops"][kind] = {"burst": r["tflops"], "sustained": r["tflops_sustained"],
                                     "source": f"library GEMM 8192^3 measured in this run ({kind})"}
        except Exception as e:
            burst = (committed.get("tflops") or {}).get(kind)
            if burst:
                peaks["tflops"][kind] = {"burst": burst, "sustained": (committed.get("tflops_sustained") or {}).get(kind, burst),
                                         "source": f"committed measure_peak block ({e})"}
    return peaks


from tilebench_b200.clocks import ClockSampler  # noqa: E402  (NVML polling of SM clock and throttle reasons)


# ------------------------------------------------------------------------------------------------
# reference arm: the path's PyTorch reference on host cores
# ------------------------------------------------------------------------------------------------

def cpu_sample_inputs(sample_rows: int):
    import torch
    g = torch.Generator().manual_seed(20261125)
    w = torch.randint(-127, 128, (sample_rows, COLS), dtype=torch.int8, generator=g)
    scale = torch.randn(sample_rows, generator=g).abs() * 0.02 + 1e-4
    return w, scale


def time_cpu_reference(rows: int, warmup: int, steps: int):
    """(GB/s, seconds per step, threads) of oracle/torch_ref.dequant_int8_channel — the reference's PyTorch
    formula on CPU tensors with every host thread — over `rows` rows of the headline workload."""
    from oracle import torch_ref
    cores = torch_ref.use_all_cores()
    w, scale = cpu_sample_inputs(rows)
    for _ in range(warmup):
        torch_ref.dequant_int8_channel(w, scale)
    t0 = time.perf_counter()
    for _ in range(steps):
        torch_ref.dequant_int8_channel(w, scale)
    dt = (time.perf_counter() - t0) / steps
    return (rows * COLS * 3 + rows * 4) / dt / 1e9, dt, cores


def run_reference(args):
    """Times oracle/torch_ref.dequant_int8_channel (the reference formula on CPU tensors, all host
    threads) on the whole headline workload, one pass over all 65536 rows per step (about 0.15 s)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import torch_ref
    cores = torch_ref.use_all_cores()
    sample_rows = ROWS
    w, scale = cpu_sample_inputs(sample_rows)
    sample_bytes = sample_rows * COLS * 3 + sample_rows * 4
    for _ in range(args.warmup):
        torch_ref.dequant_int8_channel(w, scale)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch_ref.dequant_int8_channel(w, scale)
    dt = (time.perf_counter() - t0) / args.steps
    value = sample_bytes / dt / 1e9
    sample = f"all {ROWS} rows per step ({sample_bytes} algorithmic bytes), torch CPU, {cores} threads"
    print(file=args.out, *[json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })])


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def event_time_ms(torch, fn, iters: int) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / iters


def time_rotating(torch, make_call, sets: int, warmup: int, iters: int) -> float:
    """ms per call over back-to-back calls that rotate through `sets` independent buffer sets
    (their combined footprint exceeds L2, so no call finds its operands cached).

    One rotation is captured into a CUDA graph and the replay is timed, so the figure is device time: kernels
    of 5-40 us would otherwise be paced by how fast the host can launch them (which differs from box to box).
    If capture fails the rotation is launched eagerly."""
    calls = [make_call(i) for i in range(sets)]
    for _ in range(warmup):
        for c in calls:
            c()
    torch.cuda.synchronize()

    def rotation():
        for c in calls:
            c()
    runner = rotation
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            rotation()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            rotation()
        graph.replay()
        torch.cuda.synchronize()
        runner = graph.replay
    except Exception:
        torch.cuda.synchronize()
    return event_time_ms(torch, runner, iters) / sets


def sections(torch, dev, peaks, world, rank, steps, warmup):
    """Absolute rate and roofline fraction of the other workloads of the path."""
    from tilebench_b200 import native, npart
    from tilebench_b200.data import tensors
    ext = native.load()
    out = []
    L2 = 132_644_864
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def hbm_row(name, nbytes, ms, launches=1, note=None):
        gbs = nbytes / (ms * 1e-3) / 1e9
        r = {"name": name, "ms": ms, "GBps": gbs, "bound": "hbm", "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
             "algorithmic_bytes": nbytes, "launches_per_call": launches}
        if note:
            r["note"] = note
        return r

    def tensor_row(name, flops, ms, kind, nbytes=None, launches=1, note=None, scale=1):
        """`kind` names the measured library-GEMM rate that bounds the row (bf16, fp16, tf32, fp8_e4m3fn, int8);
        `scale` multiplies it (aggregate rows over several GPUs)."""
        tf = flops / (ms * 1e-3) / 1e12
        r = {"name": name, "ms": ms, "TFLOPs": tf, "bound": "tensor", "launches_per_call": launches, "peak_kind": kind,
             "peak_scale": scale}
        if nbytes:
            r["GBps"] = nbytes / (ms * 1e-3) / 1e9
            r["frac_of_hbm_peak"] = r["GBps"] / peaks["hbm_gbs"]
        if note:
            r["note"] = note
        return r

    iters = max(5, min(steps, 20))
    # ---- config 0: int4 group dequant 4096 x 4096 (42.2 MB per call; 8 rotating sets = 338 MB) ----
    N, K = 4096, 4096
    sets = 8
    wps = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(sets)]
    scs = [(torch.randn(N, K // 128, device=dev, generator=gen).abs() * 0.01 + 1e-3).half() for _ in range(sets)]
    outs = [torch.empty(N, K, dtype=torch.float16, device=dev) for _ in range(sets)]
    ms = time_rotating(torch, lambda i: (lambda: ext.dequant_int4_group(wps[i], scs[i], outs[i], 128, 8)), sets, warmup, iters)
    out.append(hbm_row("dequant_int4_group N=4096 K=4096 g128", N * K // 2 + N * (K // 128) * 2 + N * K * 2, ms,
                       note="8 rotating buffer sets (338 MB > L2)"))
    del wps, scs, outs
    # yardstick for that size: a plain device copy moving the same 42.2 MB per call (21.1 MB read + 21.1 MB written) under
    # the same protocol — what a streaming kernel of this length can reach at all, launch ramp and tail included
    half = (N * K // 2 + N * (K // 128) * 2 + N * K * 2) // 2
    srcs = [torch.empty(half, dtype=torch.uint8, device=dev).fill_(i) for i in range(sets)]
    dsts = [torch.empty(half, dtype=torch.uint8, device=dev) for _ in range(sets)]
    ms = time_rotating(torch, lambda i: (lambda: dsts[i].copy_(srcs[i])), sets, warmup, iters)
    out.append(hbm_row("yardstick: device copy of 42.2 MB per call (torch copy_)", 2 * half, ms, note="library copy kernel, same rotating protocol; not a kernel of this package"))
    del srcs, dsts

    # ---- config 1 smaller sizes ----
    for rows, sets in ((256, 64), (4096, 8)):
        ws = [torch.randint(-127, 128, (rows, COLS), dtype=torch.int8, device=dev, generator=gen) for _ in range(sets)]
        ss = [torch.randn(rows, device=dev, generator=gen).abs() * 0.02 + 1e-4 for _ in range(sets)]
        os_ = [torch.empty(rows, COLS, dtype=torch.bfloat16, device=dev) for _ in range(sets)]
        ms = time_rotating(torch, lambda i: (lambda: ext.dequant_int8_rowwise(ws[i], ss[i], os_[i], False, 1.0)), sets, warmup, iters)
        out.append(hbm_row(f"dequant_int8_channel rows={rows} cols=4096", rows * COLS * 3 + rows * 4, ms,
                           note=f"{sets} rotating buffer sets"))
        del ws, ss, os_

    # ---- config 2: W4A16 GEMM K=4096 N=14336 ----
    K, N = 4096, 14336
    for M in (1, 16, 128, 4096):
        nbytes = M * K * 2 + N * K // 2 + N * (K // 128) * 2 + M * N * 2
        sets = max(2, -(-2 * L2 // nbytes))
        a = [torch.randn(M, K, device=dev, generator=gen).half() for _ in range(sets)]
        wp = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(sets)]
        sc = [(torch.randn(N, K // 128, device=dev, generator=gen).abs() * 0.01 + 1e-3).half() for _ in range(sets)]
        o = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(sets)]
        wsb = ext.gemm_w4a16_workspace_bytes(M, N, K)
        ws = torch.empty(max(wsb // 4, 1), dtype=torch.float32, device=dev)
        ms = time_rotating(torch, lambda i: (lambda: ext.gemm_w4a16(a[i], wp[i], sc[i], o[i], 128, 8, 0, ws)), sets, warmup, iters)
        flops = 2 * M * N * K
        launches = 2 if wsb else 1
        if M <= 16:
            r = hbm_row(f"gemm_w4a16 M={M} K=4096 N=14336", nbytes, ms, launches, note=f"{sets} rotating sets; split-K workspace {wsb} B")
            r["TFLOPs"] = flops / (ms * 1e-3) / 1e12
        else:
            r = tensor_row(f"gemm_w4a16 M={M} K=4096 N=14336", flops, ms, "fp16", nbytes, launches, note=f"{sets} rotating sets")
        out.append(r)
        del a, wp, sc, o, ws

    # ---- config 3: FP8 block-scaled GEMM, square ----
    for S in (1024, 4096, 8192, 16384):
        nbytes = 2 * S * S + S * (S // 128) * 4 + (S // 128) ** 2 * 4 + 2 * S * S
        sets = max(1, min(8, -(-2 * L2 // nbytes)))
        ins = []
        for _ in range(sets):
            aq, sa = tensors.quantize_fp8_blockwise(torch.randn(S, S, device=dev, generator=gen), 1, 128)
            bq, sb = tensors.quantize_fp8_blockwise(torch.randn(S, S, device=dev, generator=gen), 128, 128)
            ins.append((aq, sa, bq, sb, torch.empty(S, S, dtype=torch.bfloat16, device=dev)))
        ms = time_rotating(torch, lambda i: (lambda: ext.gemm_fp8_blockscaled(*ins[i])), sets, warmup, max(3, iters // (1 if S < 16384 else 4)))
        out.append(tensor_row(f"gemm_fp8_blockscaled S={S}", 2 * S ** 3, ms, "fp8_e4m3fn", nbytes, note=f"{sets} rotating sets"))
        del ins

    # ---- the reference's own GEMM operators on the path, at the largest case of their grids ----
    # matmul_int8: a int8 [2048, 20480] x b uint8 [5120, 2048] (four 2-bit weights per byte) -> int32
    M, N, K = 2048, 2048, 20480
    nbytes = M * K + K * N // 4 + 4 * M * N
    sets = max(2, -(-2 * L2 // nbytes))
    ai = [torch.randint(-64, 65, (M, K), dtype=torch.int8, device=dev, generator=gen) for _ in range(sets)]
    bi = [torch.randint(0, 256, (K // 4, N), dtype=torch.uint8, device=dev, generator=gen) for _ in range(sets)]
    oi = [torch.empty(M, N, dtype=torch.int32, device=dev) for _ in range(sets)]
    ms = time_rotating(torch, lambda i: (lambda: ext.matmul_int8_packed2(ai[i], bi[i], oi[i])), sets, warmup, iters)
    out.append(tensor_row("matmul_int8 M=2048 N=2048 K=20480", 2 * M * N * K, ms, "int8", nbytes,
                          note=f"{sets} rotating sets; TOPS reported as TFLOPs"))
    del ai, bi, oi
    # matmul_fp32_fp16_fp8: a [4096, 16384] x b [16384, 4096], both row-major
    M, N, K = 4096, 4096, 16384
    for dt, label, kind in ((torch.float16, "fp16", "fp16"), (torch.float32, "fp32 (TF32)", "tf32"), (torch.float8_e4m3fn, "e4m3", "fp8_e4m3fn")):
        esize = torch.empty((), dtype=dt).element_size()
        nbytes = (M * K + K * N + M * N) * esize
        sets = max(2, -(-2 * L2 // nbytes))
        scale = K ** -0.5
        ap = [(torch.randn(M, K, device=dev, generator=gen) * scale).to(dt) for _ in range(sets)]
        bp = [(torch.randn(K, N, device=dev, generator=gen) * scale).to(dt) for _ in range(sets)]
        op = [torch.empty(M, N, dtype=dt, device=dev) for _ in range(sets)]
        ms = time_rotating(torch, lambda i: (lambda: ext.matmul_plain(ap[i], bp[i], op[i])), sets, warmup, iters)
        out.append(tensor_row(f"matmul_fp32_fp16_fp8 {label} M=4096 N=4096 K=16384", 2 * M * N * K, ms, kind, nbytes, note=f"{sets} rotating sets"))
        del ap, bp, op

    # ---- config 4 on one GPU: the whole N = 57344 problem (the multi-rank timings live in `multi_gpu`) ----
    if world == 1:
        M, K, N = CFG4
        a = torch.randn(M, K, device=dev, generator=gen).half()
        wp = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=gen)
        sc = (torch.randn(N, K // 128, device=dev, generator=gen).abs() * 0.01 + 1e-3).half()
        o = torch.empty(M, N, dtype=torch.float16, device=dev)
        for _ in range(warmup):
            ext.gemm_w4a16(a, wp, sc, o, 128, 8, 0, None)
        torch.cuda.synchronize()
        ms = event_time_ms(torch, lambda: ext.gemm_w4a16(a, wp, sc, o, 128, 8, 0, None), max(3, iters // 2))
        out.append(tensor_row("gemm_w4a16_npart M=4096 K=8192 N=57344 world=1 gather=none", 2 * M * N * K, ms, "fp16",
                              note="705 MB touched per call (larger than L2); output preallocated"))
        del a, wp, sc, o
    return out


def multi_gpu_config4(torch, dist, dev, world, rank, sampler, peaks, repeats=10, warmup=3):
    """BASELINE config 4 over `world` ranks: M=4096, K=8192, N=57344 split evenly, activations replicated.

    Runs before anything else has heated the boards.  First rank 0 times the WHOLE problem (all 57344 weight
    rows) on its own GPU while the others wait, so every speed-up below is taken inside one process and one
    thermal state.  Then every mode is timed `repeats` times: a barrier, then one event-timed call per rank;
    a repeat's time is the max over ranks, the reported time the median over repeats (min beside it).
    `ms_x_mhz` = ms x median SM clock of rank 0's GPU during that mode: a clock-independent cost figure."""
    from tilebench_b200 import native, npart
    ext = native.load()
    M, K, N = CFG4
    flops = 2 * M * N * K
    lo, hi = npart.partition(N, world, rank)
    n_local = hi - lo
    shared = torch.Generator(device=dev).manual_seed(99)               # same stream on every rank: replicated inputs
    a = torch.randn(M, K, device=dev, generator=shared).half()
    wp_full = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=shared)
    sc_full = (torch.randn(N, K // 128, device=dev, generator=shared).abs() * 0.01 + 1e-3).half()
    wp, sc = wp_full[lo:hi].contiguous(), sc_full[lo:hi].contiguous()

    def timed(call):
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        call()
        s1.record()
        s1.synchronize()
        return s0.elapsed_time(s1)

    def summary(samples, since):
        med = statistics.median(samples)
        clk = sampler.snapshot(since)
        return {"ms": med, "ms_min": min(samples), "TFLOPs": flops / med / 1e9, "repeats": len(samples),
                "sm_mhz": clk["sm_mhz"], "ms_x_mhz": med * clk["sm_mhz"] if clk["sm_mhz"] else None}

    # ---- the whole problem on one GPU (rank 0), same kernel, same process ----
    single = None
    sampler.busy(True)
    if rank == 0:
        o = torch.empty(M, N, dtype=torch.float16, device=dev)
        for _ in range(warmup):
            ext.gemm_w4a16(a, wp_full, sc_full, o, 128, 8, 0, None)
        torch.cuda.synchronize()
        since = sampler.mark()
        single = summary([timed(lambda: ext.gemm_w4a16(a, wp_full, sc_full, o, 128, 8, 0, None)) for _ in range(repeats)], since)
        del o
    del wp_full, sc_full
    torch.cuda.empty_cache()
    dist.barrier()

    out_local = torch.empty(M, n_local, dtype=torch.float16, device=dev)
    modes = {}
    for name, gather in (("compute_only", False), ("gather_fused", "fused"), ("gather_push", "push"), ("gather_nccl", "nccl")):
        def call():
            return npart.gemm_w4a16_partitioned(a, wp, sc, 128, 8, gather=gather, out_local=out_local)
        for _ in range(warmup):
            call()
        torch.cuda.synchronize()
        since = sampler.mark()
        mine = []
        for _ in range(repeats):
            dist.barrier()
            torch.cuda.synchronize()
            mine.append(timed(call))
        t = torch.tensor(mine, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)                        # per repeat: the slowest rank
        modes[name] = summary([float(x) for x in t.tolist()], since)
    sampler.busy(False)
    res = {"workload": f"gemm_w4a16_npart M={M} K={K} N={N} split over {world} ranks ({n_local} weight rows each), fp16 activations replicated",
           "timing": f"median of {repeats} repeats, each the max over ranks of one CUDA-event-timed call after a barrier; {warmup} warm-up calls per mode",
           "single_gpu_whole_problem": single, "world": world, "modes": modes,
           "gathered_bytes_per_rank": M * (N - n_local) * 2}
    if rank == 0 and single:
        for name, m in modes.items():
            m["speedup_vs_single_gpu"] = single["ms"] / m["ms"]
            if m.get("ms_x_mhz") and single.get("ms_x_mhz"):
                m["speedup_clock_normalised"] = single["ms_x_mhz"] / m["ms_x_mhz"]
            m["frac_of_tensor_peak"] = m["TFLOPs"] / (world * peaks["tflops"]["fp16"]["burst"])
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks (WORLD_SIZE is 1)")
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from tilebench_b200 import native
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    ext = native.load()          # raises if the CUDA extension is missing: there is no fallback
    native.require_b200()
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    sampler.start()
    native.clear_device_status()

    multi = None
    if world > 1 and args.sections != "none":
        try:
            multi = multi_gpu_config4(torch, dist, dev, world, rank, sampler, peaks)
        except Exception as e:      # must not lose the headline
            multi = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()

    # inputs resident in HBM before the timed region (seeded per rank)
    g = torch.Generator(device=dev).manual_seed(20261125 + rank)
    w = torch.randint(-127, 128, (ROWS, COLS), dtype=torch.int8, device=dev, generator=g)
    scale = torch.randn(ROWS, device=dev, generator=g).abs() * 0.02 + 1e-4
    out = torch.empty(ROWS, COLS, dtype=torch.bfloat16, device=dev)

    def step():
        ext.dequant_int8_rowwise(w, scale, out, False, 1.0)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    # the K timed steps are K kernel launches replayed as one CUDA graph (host launch cost stays out of a device
    # measurement); if capture is not possible they are launched one by one
    run_steps, launch_mode = (lambda: [step() for _ in range(args.steps)]), "eager launches"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.steps):
                step()
        graph.replay()                                   # one untimed replay: graph upload
        torch.cuda.synchronize()
        run_steps, launch_mode = graph.replay, f"one CUDA graph of {args.steps} kernel launches"
    except Exception:
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.busy(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    run_steps()
    end.record()
    end.synchronize()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed_ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * ALG_BYTES / (ms_per_step * 1e-3) / 1e9
    per_gpu = ALG_BYTES / (ms_per_step * 1e-3) / 1e9

    # spot check of the timed output against the package's PyTorch reference on the same device
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_torch
    assert torch.equal(out[:1024], impl_torch.run(w[:1024], scale[:1024])), "headline kernel output differs from reference"

    # ---- end to end through the operator entry point with host buffers ----
    hw = torch.empty((ROWS, COLS), dtype=torch.int8).pin_memory()
    hw.copy_(w.cpu())
    hs = scale.cpu().pin_memory()
    hout = torch.empty((ROWS, COLS), dtype=torch.bfloat16).pin_memory()

    from tilebench_b200 import host_api

    def e2e_step():
        # host tensors in, host tensor out: upload, kernel and download of row chunks pipelined over three streams
        host_api.dequant_int8_channel_host(hw, hs, hout, device=dev)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e2e_ms = event_time_ms(torch, e2e_step, e2e_steps)
    torch.cuda.synchronize()
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * ALG_BYTES / (e2e_ms * 1e-3) / 1e9
    del hw, hout

    extra = []
    if args.sections == "all":
        del w, out
        torch.cuda.empty_cache()
        try:
            extra = sections(torch, dev, peaks, world, rank, args.steps, args.warmup)
            add_live_peaks(peaks, live=not args.no_live_peaks)    # after the sections, so the probes' seconds-long loops do not pre-heat them
            fill_tensor_fractions(extra, peaks)
        except Exception as e:  # a failing section must not lose the headline
            extra = [{"name": "sections", "error": f"{type(e).__name__}: {e}"}]
    sampler.busy(False)
    clocks = sampler.stop()
    clocks.pop("power_w_max", None)
    code, detail = native.device_status()

    cpu_baseline = None
    if rank == 0 and world == 1:
        # the same leg the reference arm times: the PyTorch formula on CPU tensors, every host thread, all rows
        reps = 5
        gbs, dt, cores = time_cpu_reference(ROWS, 1, reps)
        cpu_baseline = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "ms_per_step": dt * 1e3,
                        "sample": f"all {ROWS} rows ({ALG_BYTES} algorithmic bytes) x {reps} passes, torch CPU reference formula, {cores} threads"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(world),
            "timed_region": launch_mode,
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / peaks["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "peak_source": f"of {peaks['source']}", "kernel": "tb200_k_dequant_int8_rowwise_bf16_wide",
                         "algorithmic_bytes_per_launch": ALG_BYTES},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": ROWS * COLS + ROWS * 4,
                    "d2h_bytes_per_step": ROWS * COLS * 2, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "device_status": {"code": code, "detail": detail},
            "cpu_baseline": cpu_baseline,
            "peaks": {"hbm_gbs": peaks["hbm_gbs"], "hbm_source": peaks["source"], "tflops": peaks["tflops"]},
            "multi_gpu": multi,
            "sections": extra,
        }
        print(json.dumps(line), file=args.out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _own_stdout():
    """Returns a file object on the real stdout and points fd 1 at stderr for the rest of the run, so
    that library banners (NCCL prints its version on stdout) cannot break the one-JSON-line contract."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sections", choices=["all", "multi", "none"], default="all",
                    help="all: every section; multi: headline + the multi_gpu section only (N > 1); none: headline only")
    ap.add_argument("--no-live-peaks", action="store_true",
                    help="skip the seconds-long library-GEMM probes (profiler runs); fractions then use the committed measure_peak block")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    args.out = _own_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    args.out.flush()


if __name__ == "__main__":
    main()
