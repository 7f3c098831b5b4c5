"""tilebench_b200 — a B200-native `cuda` backend for TileBench's quantized-inference path.

The package keeps TileBench's operator contract (per-operator `config.yaml`, a PyTorch reference
`impl_torch.run`, a backend entry point `impl_cuda.run`, dtype-aware verification, metric
formulas) and replaces the JIT DSL kernels with hand-written sm_100a CUDA behind a C ABI
(`include/tb200.h`, `tilebench_b200/csrc`).  There is no CPU fallback inside the backend:
`tilebench_b200.native.load()` raises when the compiled library is missing.
"""

__version__ = "0.1.0"
