"""Every operator through the benchmark engine on the GPU: seeded inputs -> PyTorch reference on the
device -> impl_cuda.run -> verify with the operator's tolerance -> timed only if verified.  These are the
BASELINE configurations themselves (all cases of configs 0-3, the single-GPU cases of config 4) plus a
sample of the reference operators' own grids."""
import math

import pytest

from tilebench_b200.core.engine import run_benchmark_suite

pytestmark = pytest.mark.gpu

FAST = {"warmup": 1, "repeat": 1}


def run_cases(op):
    import yaml
    from tilebench_b200.data.tensors import expand_cases
    from tilebench_b200.paths import operator_config
    with open(operator_config(op)) as f:
        return expand_cases(op, yaml.safe_load(f))


def check(rows, n, graph=True):
    """Verified, timed, and (where the operator's config asks for graph replay, as every single-GPU operator
    does) really timed as a captured CUDA graph: the timer falls back to eager calls when capture fails, and
    a backend whose run() cannot be captured would otherwise pass unnoticed."""
    assert len(rows) == n
    for r in rows:
        assert r["cuda_ok"], f"{r['params']}: {r['cuda_err']}"
        assert r["cuda_ms"] > 0 and not math.isnan(r["cuda_ms"]) and r["speedup_cuda"] > 0
        if graph:
            assert r["cuda_stats"]["mode"] == "graph", f"{r['params']}: timed in {r['cuda_stats']['mode']} mode"
            assert r["timing"]["timing_execution_mode"] == "graph"


def test_config0_int4_group_dequant(cuda_device):
    check(run_benchmark_suite("dequant_int4_group", FAST, ["cuda"]), 1)


def test_config1_int8_channel_dequant_all_sizes(cuda_device):
    check(run_benchmark_suite("dequant_int8_channel", FAST, ["cuda"]), 3)


def test_config2_w4a16_gemm_all_m(cuda_device):
    check(run_benchmark_suite("gemm_w4a16", FAST, ["cuda"]), 4)


def test_config3_fp8_blockscaled_gemm_all_sizes(cuda_device):
    check(run_benchmark_suite("gemm_fp8_blockscaled", FAST, ["cuda"]), 4)


def test_config4_npart_single_gpu_cases(cuda_device):
    # WORLD=1 with and without the (trivial) gather; the multi-rank cases run under torch.distributed
    check(run_benchmark_suite("gemm_w4a16_npart", {**FAST, "case_indices": [0, 1, 2, 3]}, ["cuda"]), 4, graph=False)


def test_config4_npart_single_gpu_under_graph_capture(cuda_device):
    check(run_benchmark_suite("gemm_w4a16_npart", {**FAST, "use_cuda_graph": True, "case_indices": [0, 1]}, ["cuda"]), 2)


def test_int4_group_quantiser(cuda_device):
    assert len(run_cases("quantize_int4_group")) == 6
    check(run_benchmark_suite("quantize_int4_group", {**FAST, "case_indices": [0, 3]}, ["cuda"]), 2)


def test_fp8_block_quantiser(cuda_device):
    check(run_benchmark_suite("quantize_fp8_block", {**FAST, "case_indices": [0, 1, 2, 3]}, ["cuda"]), 4)


def test_reference_operator_grids_sampled(cuda_device):
    check(run_benchmark_suite("dequantize_rowwise", {**FAST, "case_indices": [0, 9, 19]}, ["cuda"]), 3)
    # weight_dequant: M = 512 / 4096 / 10240 in fp16, bf16, fp32
    check(run_benchmark_suite("weight_dequant", {**FAST, "case_indices": [0, 22, 59]}, ["cuda"]), 3)
    # the reference's two GEMM operators: smallest and largest K of each grid
    check(run_benchmark_suite("matmul_int8", {**FAST, "case_indices": [0, 19]}, ["cuda"]), 2)
    check(run_benchmark_suite("matmul_fp32_fp16_fp8", {**FAST, "case_indices": [0, 29, 59]}, ["cuda"]), 3)


def test_cuda_graph_replay_protocol(cuda_device):
    """The reference protocol: 1 warm-up, 3 timed CUDA-graph replays with an L2 flush before each."""
    rows = run_benchmark_suite("dequant_int8_channel", {"case_indices": [1]}, ["cuda"])
    check(rows, 1)
    assert rows[0]["cuda_stats"]["mode"] == "graph" and len(rows[0]["cuda_stats"]["samples"]) == 3
    assert rows[0]["timing"]["timing_execution_mode"] == "graph"
