"""Provenance sidecar of a benchmark run (reference: tilebench/provenance.py:100-136):
source revision, software versions, device and host, written next to the timing log."""
from __future__ import annotations

import socket
import subprocess
import sys
from datetime import datetime, timezone

from tilebench_b200 import hardware
from tilebench_b200.paths import REPO_ROOT

SCHEMA = "tilebench-b200-provenance/1"


def _git(*args: str) -> str | None:
    try:
        out = subprocess.run(["git", "-C", str(REPO_ROOT), *args], capture_output=True, text=True, timeout=10)
        return out.stdout.strip() if out.returncode == 0 else None
    except Exception:
        return None


def source_state() -> dict:
    dirty = _git("status", "--porcelain")
    return {"git_sha": _git("rev-parse", "HEAD"), "dirty": bool(dirty) if dirty is not None else None}


def software_state() -> dict:
    state = {"python": sys.version.split()[0], "torch": None, "torch_cuda": None, "tb200_abi": None}
    try:
        import torch
        state.update(torch=torch.__version__, torch_cuda=torch.version.cuda)
    except Exception:
        pass
    try:
        from tilebench_b200 import native
        state["tb200_abi"] = native.capi().tb200_abi_version()
    except Exception:
        pass
    return state


def device_state(requested_label: str) -> dict:
    dev = hardware.device_info()
    return {"requested_label": requested_label, "name": dev.name if dev else None,
            "vendor": dev.vendor if dev else None, "arch": hardware.detect_arch(),
            "compute_capability": list(dev.capability) if dev and dev.capability else None}


def collect(requested_label: str) -> dict:
    return {"schema": SCHEMA, "created_at_utc": datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ"),
            "source": source_state(), "software": software_state(), "device": device_state(requested_label),
            "host": {"hostname": socket.gethostname(), "argv": list(sys.argv)}}
