"""The harness functions this package restates — case-grid expansion, verifier, tolerance lookup, derived
metrics — against the reference's OWN functions, on this package's operator configs.

Runs only where a TileBench checkout can be imported (TILEBENCH_REFERENCE=/path/to/checkout, or a `reference`
folder beside this repository); elsewhere — e.g. on a GPU box that only carries this repository — it is skipped,
and the committed fixtures under tests/golden/ are what ties the package to reference code."""
import importlib
import math
import os
import sys
from pathlib import Path

import pytest
import torch
import yaml

from tilebench_b200.core import metrics, verifier
from tilebench_b200.data import tensors
from tilebench_b200.paths import list_operators, operator_config

REF_ROOT = Path(os.environ.get("TILEBENCH_REFERENCE") or Path(__file__).resolve().parents[2] / "reference")


@pytest.fixture(scope="module")
def ref():
    if not (REF_ROOT / "tilebench" / "core" / "verifier.py").is_file():
        pytest.skip(f"no TileBench checkout at {REF_ROOT}")
    sys.path.insert(0, str(REF_ROOT))
    try:
        mods = {name: importlib.import_module(f"tilebench.{name}")
                for name in ("core.verifier", "core.metrics", "data.tensors", "core.dtypes", "paths", "backends")}
    except Exception as e:          # a checkout whose dependencies are missing here
        pytest.skip(f"reference not importable: {type(e).__name__}: {e}")
    finally:
        sys.path.remove(str(REF_ROOT))
    return mods


def configs():
    for op in list_operators():
        with open(operator_config(op)) as f:
            yield op, yaml.safe_load(f)


def test_expand_cases_equals_the_reference_on_every_config(ref):
    rt = ref["data.tensors"]
    for op, cfg in configs():
        assert tensors.expand_cases(op, cfg) == rt.expand_cases(op, cfg), op
    # explicit test_cases win over a grid, in both
    both = {"test_cases": [{"a": 1}, {"a": 2}], "case_grid": {"a": [3]}}
    assert tensors.expand_cases("x", both) == rt.expand_cases("x", both) == [{"a": 1}, {"a": 2}]
    # malformed grids are refused by both with a ValueError
    for bad in ({"case_grid": {}}, {"case_grid": {"a": []}}, {"case_grid": {"a": {"expr": "[]"}}}, {}):
        with pytest.raises(ValueError):
            tensors.expand_cases("x", bad)
        with pytest.raises(ValueError):
            rt.expand_cases("x", bad)


def test_config_tolerance_equals_the_reference(ref):
    rv = ref["core.verifier"]
    sections = [cfg.get("verify", {}) for _, cfg in configs()]
    sections += [{}, {"atol": 1}, {"rtol": "1e-2"}, {"atol": 0.5, "arch_overrides": {"blackwell": {"atol": 2.0}, "hopper": {"rtol": 3}}}]
    for sec in sections:
        for arch in (None, "blackwell", "hopper", "ampere"):
            assert verifier.config_tolerance(sec, arch) == rv.config_tolerance(sec, arch), (sec, arch)


def test_tolerance_table_and_verify_decisions_equal_the_reference(ref):
    rv = ref["core.verifier"]
    assert verifier._TOLERANCES == rv._TOLERANCES
    g = torch.Generator().manual_seed(0)
    pairs = []
    for dt in (torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.int32, torch.int8, torch.float64):
        base = (torch.randn(64, generator=g) * 4).to(dt)
        for bump in (0.0, 1e-6, 1e-3, 2e-2, 0.3, 2.0):
            other = (base.to(torch.float64) + bump).to(dt)
            pairs.append((other, base))
    pairs.append((torch.zeros(4), torch.zeros(5)))                                 # shape mismatch
    pairs.append((torch.zeros(4, dtype=torch.float16), torch.zeros(4)))           # dtype mismatch
    pairs.append(((torch.ones(3), torch.zeros(3)), (torch.ones(3), torch.ones(3))))   # tuple, second element differs
    for out, want in pairs:
        for tol in ({}, {"atol": 0, "rtol": 0}, {"atol": 0.5}, {"rtol": 0.5}):
            mine, theirs = verifier.verify(out, want, **tol), rv.verify(out, want, **tol)
            assert mine[0] == theirs[0], (out, tol)
            assert mine[1] == theirs[1]


def test_compute_derived_equals_the_reference(ref):
    rm = ref["core.metrics"]
    peak = metrics.load_peak_config("B200")
    assert peak["peak_bw_GBs"] == rm.load_peak_config("B200")["peak_bw_GBs"]
    assert peak["peak_tflops"]["fp16"] == rm.load_peak_config("B200")["peak_tflops"]["fp16"]
    for op, cfg in configs():
        for i, case in enumerate(tensors.expand_cases(op, cfg)[:6]):
            params = {k: v for k, v in case.items() if k not in ("dtype", "block_size")}
            row = {"params": params, "dtype": case.get("dtype", "fp32"), "torch_ms": 1.7 + i, "cuda_ms": 0.031 * (i + 1)}
            mine = metrics.compute_derived(row, cfg["metrics"], peak)
            # the reference has no `cuda` column: feed the same time through one of its GPU backends
            theirs = rm.compute_derived({**row, "triton_ms": row["cuda_ms"]}, cfg["metrics"], rm.load_peak_config("B200"))
            for backend_mine, backend_theirs in (("torch", "torch"), ("cuda", "triton")):
                for key, val in theirs[backend_theirs].items():
                    assert math.isclose(mine[backend_mine][key], val, rel_tol=1e-12), (op, case, key)
                extra = set(mine[backend_mine]) - set(theirs[backend_theirs])
                assert extra <= {"pct_measured_bw", "pct_measured_tflops"}, extra
    # dtype sizes used by bytes_expr
    from tilebench_b200.core.dtypes import dtype_size
    for name in ("fp32", "fp16", "bf16", "fp8_e4m3fn", "int8", "int32", "unknown"):
        assert dtype_size(name) == ref["core.dtypes"].dtype_size(name), name


def test_result_layout_is_where_the_reference_tools_look(ref, monkeypatch, tmp_path):
    """A run of this package's CLI writes its timing log under the name and folder the reference's path helpers give
    for a backend selection of ("cuda",) once `cuda` is a registered backend there, and the rows in it are read by the
    reference's compute_derived — i.e. the reference's plotting script finds and understands them."""
    import json
    import tilebench_b200.core.engine as engine
    from tilebench_b200 import run_bench
    rb, rp, rm = ref["backends"], ref["paths"], ref["core.metrics"]
    monkeypatch.setattr(rb, "BACKEND_ORDER", tuple(rb.BACKEND_ORDER) + ("cuda",))        # the one-line edit a checkout makes
    monkeypatch.setattr(rm, "BACKENDS", tuple(rm.BACKENDS) + ("cuda",))
    row = {"params": {"rows": 4096, "cols": 4096}, "problem_size": 4096 * 4096, "dtype": "bf16", "seed": 1, "torch_ms": 0.1,
           "torch_stats": {"mean": 0.1}, "cuda_ms": 0.01, "cuda_stats": {"mean": 0.01}, "cuda_ok": True, "cuda_err": "",
           "cuda_autotune_cfg": None, "speedup_cuda": 10.0, "timing": None}
    monkeypatch.setattr(engine, "run_benchmark_suite", lambda *a, **k: [dict(row)])
    assert run_bench.main(["--operator", "dequant_int8_channel", "--output-root", str(tmp_path)]) == 0
    theirs = rp.timing_log_path("B200", "dequant_int8_channel", "default", ["cuda"])
    mine = tmp_path / "B200" / "logs" / "time_measurement_logs" / "dequant_int8_channel_default_cuda.json"
    assert mine.is_file() and theirs.parts[-3:] == mine.parts[-3:]
    assert rp.provenance_log_path("B200", "dequant_int8_channel", "default", ["cuda"]).parts[-3:] == \
        (tmp_path / "B200" / "logs" / "provenance" / "dequant_int8_channel_default_cuda.json").parts[-3:]
    rows = json.loads(mine.read_text())
    cfg = yaml.safe_load(open(operator_config("dequant_int8_channel")))["metrics"]
    derived = rm.compute_derived(rows[0], cfg, rm.load_peak_config("B200"))
    assert derived["cuda"]["bandwidth_GBs"] == pytest.approx(rows[0]["derived"]["cuda"]["bandwidth_GBs"])
    assert derived["cuda"]["speedup"] == pytest.approx(10.0)
