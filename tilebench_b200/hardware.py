"""Device probe: which architecture is present and how large its last-level cache is.

Mirrors the reference's tilebench/hardware.py:55-114 for the one architecture this backend
targets.  Holds no peak numbers (those live in data/peak_performance/).
"""
from __future__ import annotations

import functools
from dataclasses import dataclass

#: B200's L2 as the CUDA runtime reports it (bytes); used when no device is present.
B200_L2_BYTES = 132_644_864

_NVIDIA_ARCH = {(10, 0): "blackwell", (10, 3): "blackwell", (9, 0): "hopper"}


@dataclass(frozen=True)
class DeviceInfo:
    vendor: str
    name: str
    capability: tuple[int, int] | None


@functools.cache
def device_info() -> DeviceInfo | None:
    """The current CUDA device, or None when there is none."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        index = torch.cuda.current_device()
        props = torch.cuda.get_device_properties(index)
        return DeviceInfo("nvidia", props.name, tuple(torch.cuda.get_device_capability(index)))
    except Exception:
        return None


@functools.cache
def detect_arch() -> str | None:
    """"blackwell" (sm_100), "hopper" (sm_90) or None (no GPU / out of scope)."""
    dev = device_info()
    if dev is None:
        return None
    return _NVIDIA_ARCH.get(dev.capability)


def supports_tmem() -> bool:
    """Tensor memory / tcgen05: Blackwell only.  The cuda backend refuses to run without it."""
    return detect_arch() == "blackwell"


def supports_tma() -> bool:
    return detect_arch() in ("hopper", "blackwell")


def last_level_cache_bytes() -> int | None:
    """L2 size to evict for a cold-cache measurement, or None without a device."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).L2_cache_size)
    except Exception:
        return None
