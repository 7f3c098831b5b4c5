"""Host logic of the harness on CPU: backend registry, case grid, verifier, metrics, and the engine's
verify-then-time control flow with injected fake operator modules (the reference tests its engine the
same way: tests/test_verify_tolerance.py:34-54, tests/test_engine_case_skip.py:17-48)."""
import math
import sys
import types

import pytest
import torch
import yaml

from tilebench_b200 import backends
from tilebench_b200.core import engine, metrics, verifier
from tilebench_b200.core.dtypes import dtype_size, resolve_dtype
from tilebench_b200.data import tensors
from tilebench_b200.paths import list_operators, operator_config


def test_backend_registry():
    assert backends.BACKEND_ORDER == ("cuda",)
    assert backends.parse_backends(None) == ["cuda"]
    assert backends.parse_backends("torch, CUDA") == ["cuda"]
    assert backends.parse_backends("all") == ["cuda"]
    assert backends.backend_tag([]) == "torch" and backends.backend_tag(["cuda"]) == "cuda"
    with pytest.raises(ValueError):
        backends.parse_backends("triton")


def test_case_counts_match_the_configs():
    want = {"dequant_int4_group": 1, "dequant_int8_channel": 3, "gemm_w4a16": 4, "gemm_fp8_blockscaled": 4,
            "gemm_w4a16_npart": 16, "dequantize_rowwise": 20, "weight_dequant": 60, "quantize_fp8_block": 6, "matmul_int8": 20,
            "matmul_fp32_fp16_fp8": 60, "quantize_int4_group": 6}
    assert sorted(list_operators()) == sorted(want)
    for op, n in want.items():
        cfg = yaml.safe_load(open(operator_config(op)))
        assert len(tensors.expand_cases(op, cfg)) == n, op
        bench = cfg["benchmark"]
        assert bench["warmup"] == 1 and bench["repeat"] == 3      # the reference's measurement protocol


def test_case_grid_expr_defaults_and_errors():
    cases = tensors._expand_case_grid({"M": {"expr": "[2 * i for i in range(1, 4)]"}, "dtype": ["fp16", "bf16"]}, {"T": 128})
    assert len(cases) == 6 and cases[0] == {"T": 128, "M": 2, "dtype": "fp16"}
    with pytest.raises(ValueError):
        tensors._expand_case_grid({}, {})
    with pytest.raises(ValueError):
        tensors._expand_case_grid({"M": []})
    assert tensors.expand_cases("x", {"test_cases": [{"a": 1}], "case_grid": {"a": [1, 2]}}) == [{"a": 1}]


def test_generators_are_seeded_and_shaped():
    a = tensors.generate_dequant_int4_group_inputs(64, 256, device="cpu", seed=1)
    b = tensors.generate_dequant_int4_group_inputs(64, 256, device="cpu", seed=1)
    c = tensors.generate_dequant_int4_group_inputs(64, 256, device="cpu", seed=2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and not torch.equal(a[0], c[0])
    assert a[0].shape == (64, 128) and a[0].dtype == torch.uint8 and a[1].shape == (64, 2) and a[1].dtype == torch.float16
    assert float(a[1].min()) >= 1e-3 - 1e-6
    w, s = tensors.generate_dequant_int8_channel_inputs(16, 64, device="cpu")
    assert int(w.min()) >= -127 and int(w.max()) <= 127 and s.dtype == torch.float32 and float(s.min()) >= 1e-4
    aq, sa, bq, sb = tensors.generate_gemm_fp8_blockscaled_inputs(S=256, device="cpu")
    assert aq.dtype == torch.float8_e4m3fn and sa.shape == (256, 2) and sb.shape == (2, 2)
    assert tensors.infer_problem_size("gemm_w4a16", {"M": 16, "N": 14336, "K": 4096}) == 16 * 14336
    a8, b8 = tensors.generate_matmul_int8_inputs(8, 16, 64, device="cpu")
    assert a8.dtype == torch.int8 and a8.shape == (8, 64) and int(a8.min()) >= -64 and int(a8.max()) <= 64
    assert b8.dtype == torch.uint8 and b8.shape == (16, 16)
    with pytest.raises(ValueError):
        tensors.generate_matmul_int8_inputs(8, 16, 66, device="cpu")


def test_dtypes():
    assert dtype_size("fp8_e4m3fn") == 1 and dtype_size("bf16") == 2 and dtype_size("mystery") == 4
    assert resolve_dtype("fp8_e4m3fn") is torch.float8_e4m3fn and resolve_dtype("bf16") is torch.bfloat16
    with pytest.raises(ValueError):
        resolve_dtype("fp3")


def test_verifier_tolerances_and_overrides():
    ref = torch.ones(4, dtype=torch.float16)
    assert verifier.verify(ref + 5e-4, ref)[0]
    assert not verifier.verify(ref + 1e-2, ref)[0]
    assert not verifier.verify(ref + 5e-4, ref, atol=0, rtol=0)[0]
    ok, err = verifier.verify((ref, ref + 1.0), (ref, ref))
    assert not ok and err.startswith("output[1]")
    f8 = torch.tensor([1.0, 2.0]).to(torch.float8_e4m3fn)
    assert verifier.verify(f8, f8)[0]
    assert verifier.config_tolerance({"atol": 1, "rtol": 2, "arch_overrides": {"blackwell": {"atol": 3}}}, "blackwell") == (3.0, 2.0)
    assert verifier.config_tolerance({}, None) == (None, None)
    # the reference's own tolerance table (tilebench/core/verifier.py:4-14)
    assert verifier.default_tolerance(torch.bfloat16) == (1e-2, 1.6e-2)
    assert verifier.default_tolerance(torch.float16) == (1e-3, 1e-3)
    assert verifier.default_tolerance(torch.int32) == (0, 0)


def test_metrics_formulas_for_the_configs():
    peak = metrics.load_peak_config("B200")
    cfg = yaml.safe_load(open(operator_config("dequant_int4_group")))["metrics"]
    row = {"params": {"N": 4096, "K": 4096, "GROUP": 128, "ZP": 8}, "dtype": "fp16", "torch_ms": 0.2, "cuda_ms": 0.01}
    d = metrics.compute_derived(row, cfg, peak)["cuda"]
    assert math.isclose(d["bandwidth_GBs"], 42_205_184 / 0.01e-3 / 1e9)
    assert math.isclose(d["pct_peak_bw"], d["bandwidth_GBs"] / 6539.4 * 100)
    assert math.isclose(d["pct_measured_bw"], d["bandwidth_GBs"] / peak["measured"]["hbm_GBs"] * 100)
    # every tensor-core input type of the path has a measured denominator (burst and sustained)
    for kind in ("fp16", "bf16", "tf32", "fp8_e4m3fn", "int8"):
        assert peak["measured"]["tflops"][kind] > peak["measured"]["tflops_sustained"][kind] > 0
    assert math.isclose(d["speedup"], 20.0)
    cfg = yaml.safe_load(open(operator_config("dequant_int8_channel")))["metrics"]
    for rows, nbytes in ((256, 3_146_752), (4096, 50_348_032), (65536, 805_568_512)):
        d = metrics.compute_derived({"params": {"rows": rows, "cols": 4096}, "dtype": "bf16", "cuda_ms": 1.0}, cfg, peak)
        assert math.isclose(d["cuda"]["bandwidth_GBs"], nbytes / 1e-3 / 1e9)
    cfg = yaml.safe_load(open(operator_config("gemm_fp8_blockscaled")))["metrics"]
    d = metrics.compute_derived({"params": {"S": 8192, "BLOCK": 128}, "dtype": "fp8_e4m3fn", "cuda_ms": 1.0}, cfg, peak)["cuda"]
    assert math.isclose(d["tflops"], 2 * 8192 ** 3 / 1e-3 / 1e12) and math.isclose(d["pct_peak_tflops"], d["tflops"] / 4500 * 100)
    cfg = yaml.safe_load(open(operator_config("gemm_w4a16")))["metrics"]
    d = metrics.compute_derived({"params": {"M": 4096, "K": 4096, "N": 14336, "GROUP": 128}, "dtype": "fp16", "cuda_ms": 1.0}, cfg, peak)["cuda"]
    assert math.isclose(d["tflops"], 2 * 4096 * 14336 * 4096 / 1e-3 / 1e12)
    # a backend that did not run on the GPU gets throughput but no % of GPU peak
    d = metrics.compute_derived({"params": {"S": 1024, "BLOCK": 128}, "dtype": "fp8_e4m3fn", "cpu_ms": 100.0}, cfg, peak)["cpu"]
    assert "pct_peak_tflops" not in d


# ---- engine control flow with fake operator modules -------------------------------------------

@pytest.fixture
def fake_op(monkeypatch, tmp_path):
    cfg = {"benchmark": {"warmup": 1, "repeat": 3}, "case_grid": {"n": [4, 8], "dtype": ["fp32"]},
           "verify": {"atol": 0, "rtol": 0}}
    path = tmp_path / "config.yaml"
    path.write_text(yaml.safe_dump(cfg))
    calls = {"cuda": 0, "bench": []}
    t = types.ModuleType("fake.impl_torch")
    t.run = lambda x: x * 2
    c = types.ModuleType("fake.impl_cuda")

    def cuda_run(x, block_size=0, autotune=False):
        calls["cuda"] += 1
        calls["kw"] = (block_size, autotune)
        if x.numel() == 8:
            return x * 2 + 1          # wrong on the second case
        return x * 2
    c.run = cuda_run
    monkeypatch.setitem(sys.modules, f"{engine.OPERATOR_PACKAGE}.fakeop.impl_torch", t)
    monkeypatch.setitem(sys.modules, f"{engine.OPERATOR_PACKAGE}.fakeop.impl_cuda", c)
    monkeypatch.setattr(engine, "operator_config", lambda name: path)
    monkeypatch.setattr(engine, "get_generator", lambda name: (lambda n, dtype, seed: (torch.arange(n, dtype=dtype),)))
    monkeypatch.setattr(engine, "HAS_CUDA", True)
    monkeypatch.setattr(engine, "_sync", lambda: None)
    monkeypatch.setattr(engine, "detect_arch", lambda: "blackwell")

    def fake_bench(fn, args, kwargs=None, **kw):
        calls["bench"].append((fn, kw["warmup"], kw["repeat"]))
        return {"mean": 2.0 if fn is t.run else 0.5}
    monkeypatch.setattr(engine, "report_benchmark", fake_bench)
    return calls, t, c


def test_engine_verifies_then_times_and_records_failures(fake_op):
    calls, t, c = fake_op
    rows = engine.run_benchmark_suite("fakeop", enabled_backends=["cuda"])
    assert len(rows) == 2
    good, bad = rows
    assert good["cuda_ok"] and good["cuda_ms"] == 0.5 and good["speedup_cuda"] == 4.0 and good["torch_ms"] == 2.0
    assert not bad["cuda_ok"] and math.isnan(bad["cuda_ms"]) and bad["cuda_err"] and bad["speedup_cuda"] == 0.0
    # the failing backend was never timed: torch twice, cuda once
    assert [fn for fn, _, _ in calls["bench"]].count(c.run) == 1
    assert all(w == 1 and r == 3 for _, w, r in calls["bench"])
    assert calls["kw"] == (1024, False)                 # block_size / autotune forwarded by signature
    assert good["seed"] != bad["seed"] and good["problem_size"] == 4


def test_engine_exception_becomes_error_row_and_case_indices(fake_op, monkeypatch):
    calls, t, c = fake_op

    def boom(x):
        raise RuntimeError("kernel said no")
    monkeypatch.setattr(c, "run", boom)
    rows = engine.run_benchmark_suite("fakeop", {"case_indices": [1]}, ["cuda"])
    assert len(rows) == 1 and rows[0]["params"] == {"n": 8}
    assert rows[0]["cuda_ok"] is False and rows[0]["cuda_err"] == "kernel said no" and math.isnan(rows[0]["cuda_ms"])
    with pytest.raises(ValueError):
        engine.run_benchmark_suite("fakeop", {"case_indices": [5]}, ["cuda"])


def test_engine_without_gpu_skips_cuda_and_can_time_cpu_reference(fake_op, monkeypatch):
    monkeypatch.setattr(engine, "HAS_CUDA", False)
    rows = engine.run_benchmark_suite("fakeop", {"cpu_baseline": True}, ["cuda"])
    assert all(not r["cuda_ok"] and "requires an NVIDIA GPU" in r["cuda_err"] for r in rows)
    assert all(r["cpu_ms"] >= 0 and r["cpu_stats"]["cores"] >= 1 for r in rows)
