"""dtype names used in operator configs (reference: tilebench/core/dtypes.py:6-47)."""
from __future__ import annotations

import torch

_SIZES = {
    "float32": 4, "fp32": 4, "float16": 2, "fp16": 2, "bfloat16": 2, "bf16": 2,
    "int8": 1, "uint8": 1, "int16": 2, "int32": 4, "int64": 8,
    "fp8": 1, "fp8_e5m2": 1, "fp8_e4m3fn": 1, "float8_e5m2": 1, "float8_e4m3fn": 1,
}
_ALIASES = {
    "fp32": "float32", "fp16": "float16", "bf16": "bfloat16",
    "fp8": "float8_e5m2", "fp8_e5m2": "float8_e5m2", "fp8_e4m3fn": "float8_e4m3fn",
}


def dtype_size(dtype_name: str) -> int:
    """Bytes per element; an unknown name counts as 4, as in the reference."""
    return _SIZES.get(dtype_name.lower(), 4)


def resolve_dtype(dtype_name: str) -> torch.dtype:
    key = dtype_name.lower()
    candidate = _ALIASES.get(key, key)
    dt = getattr(torch, candidate, None)
    if isinstance(dt, torch.dtype):
        return dt
    raise ValueError(f"Unsupported dtype '{dtype_name}' for this environment.")
