"""Backend selection for the engine and CLI.

Same surface as the reference's registry (tilebench/backends.py:13-47): a canonical order, the
default GPU selection, `--tile-language`-style parsing and an order-independent file tag.  The
only measured backend here is `cuda`; `torch` is the implicit baseline and never part of a
selection.
"""
from __future__ import annotations

#: Canonical order: drives result-key and CSV column order.
BACKEND_ORDER = ("cuda",)
#: What `all` (or no selection) means.
GPU_BACKENDS = ("cuda",)
#: Run modes as they appear in result file names.  The cuda backend has a static config table,
#: so `autotune` runs the same kernels; the name is kept for result-layout compatibility.
MODES = ("default", "autotune")


def canonical_backends(backends) -> list[str]:
    """Duplicate-free selection in canonical order; unknown names raise ValueError."""
    chosen = set(backends)
    unknown = sorted(chosen - set(BACKEND_ORDER))
    if unknown:
        raise ValueError(f"unknown backend(s) {unknown}; choose from {', '.join(BACKEND_ORDER)}")
    return [b for b in BACKEND_ORDER if b in chosen]


def parse_backends(text: str | None) -> list[str]:
    """Parse a comma-separated selection.  None / `all` -> every GPU backend; `torch` is ignored."""
    if text is None:
        return list(GPU_BACKENDS)
    tokens = [t.strip().lower() for t in text.split(",") if t.strip()]
    if "all" in tokens:
        return list(GPU_BACKENDS)
    return canonical_backends(t for t in tokens if t != "torch")


def backend_tag(backends) -> str:
    """File-name tag of a selection; a torch-only run is tagged `torch`."""
    return "-".join(canonical_backends(backends)) or "torch"
