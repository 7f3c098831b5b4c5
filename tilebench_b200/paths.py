"""Package resource locations, resolved from this file (reference: tilebench/paths.py:22-60,192-206)."""
from __future__ import annotations

import os
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent
DATA_ROOT = PACKAGE_ROOT / "data"
OPERATOR_ROOT = PACKAGE_ROOT / "benchmarks" / "operators"
PEAK_PERFORMANCE_ROOT = DATA_ROOT / "peak_performance"
REPO_ROOT = Path(os.environ.get("TILEBENCH_REPO_ROOT") or PACKAGE_ROOT.parent).resolve()
RESULTS_ROOT = REPO_ROOT / "results"


def operator_dir(name: str) -> Path:
    return OPERATOR_ROOT / name


def operator_config(name: str) -> Path:
    return operator_dir(name) / "config.yaml"


def list_operators() -> list[str]:
    """Every operator directory that has a config.yaml, sorted."""
    if not OPERATOR_ROOT.is_dir():
        return []
    return sorted(p.name for p in OPERATOR_ROOT.iterdir() if (p / "config.yaml").is_file())


def results_csv_dir(gpu: str) -> Path:
    return RESULTS_ROOT / gpu / "csv"


def results_logs_dir(gpu: str) -> Path:
    return RESULTS_ROOT / gpu / "logs"
