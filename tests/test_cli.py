"""The command-line runner with a stubbed engine: result layout, CSV columns, derived metrics and the
empty-result guard (the reference tests its CLI the same way, tests/test_results_layout.py:150-187)."""
import csv
import json

import pytest

from tilebench_b200 import run_bench


def fake_results():
    return [{"params": {"N": 4096, "K": 4096, "GROUP": 128, "ZP": 8}, "problem_size": 4096 * 4096, "dtype": "fp16",
             "seed": 1, "torch_ms": 0.2, "torch_stats": {"mean": 0.2}, "cuda_ms": 0.01, "cuda_stats": {"mean": 0.01},
             "cuda_ok": True, "cuda_err": "", "cuda_autotune_cfg": None, "speedup_cuda": 20.0, "timing": None,
             "cpu_ms": 110.0}]


def test_cli_writes_timing_provenance_and_csv(monkeypatch, tmp_path, capsys):
    import tilebench_b200.core.engine as engine
    calls = {}

    def stub(op, overrides, backends, logs_dir=None):
        calls.update(op=op, overrides=overrides, backends=backends)
        return fake_results()
    monkeypatch.setattr(engine, "run_benchmark_suite", stub)
    rc = run_bench.main(["--gpu", "B200", "--operator", "dequant_int4_group", "--warmup", "2", "--repeat", "5",
                         "--case-indices", "0", "--cpu-baseline", "--output-root", str(tmp_path)])
    assert rc == 0
    assert calls["op"] == "dequant_int4_group" and calls["backends"] == ["cuda"]
    assert calls["overrides"] == {"warmup": 2, "repeat": 5, "cpu_baseline": True, "case_indices": [0]}
    timing = tmp_path / "B200" / "logs" / "time_measurement_logs" / "dequant_int4_group_default_cuda.json"
    prov = tmp_path / "B200" / "logs" / "provenance" / "dequant_int4_group_default_cuda.json"
    rows = json.loads(timing.read_text())
    assert rows[0]["derived"]["cuda"]["bandwidth_GBs"] == pytest.approx(42_205_184 / 0.01e-3 / 1e9)
    assert json.loads(prov.read_text())["device"]["requested_label"] == "B200"
    table = list(csv.reader(open(tmp_path / "B200" / "csv" / "dequant_int4_group_default.csv")))
    assert table[0][:5] == ["params", "dtype", "torch_ms", "cuda_ms", "speedup_cuda"]
    assert table[1][0] == "GROUP=128, K=4096, N=4096, ZP=8" and table[1][2:5] == ["0.2000", "0.0100", "20.00"]
    assert float(table[1][table[0].index("cuda_pct_measured_bw")]) == pytest.approx(4220.5184 / 6550.7 * 100, rel=1e-3)
    assert run_bench.timing_log_path("B200", "dequant_int4_group", "default", ["cuda"]).parts[-4:] == \
        ("B200", "logs", "time_measurement_logs", "dequant_int4_group_default_cuda.json")
    assert "Summary CSV" in capsys.readouterr().out


def test_cli_refuses_to_overwrite_with_an_empty_result(monkeypatch, tmp_path):
    import tilebench_b200.core.engine as engine
    monkeypatch.setattr(engine, "run_benchmark_suite", lambda *a, **k: [])
    assert run_bench.main(["--operator", "dequant_int8_channel", "--output-root", str(tmp_path)]) == 1
    assert not (tmp_path / "B200").exists()


def test_cli_rejects_unknown_backend():
    with pytest.raises(ValueError):
        run_bench.main(["--operator", "dequant_int8_channel", "--tile-language", "triton"])
