import torch

from tilebench_b200.benchmarks.operators.gemm_w4a16.impl_torch import run as gemm_w4a16


def run(a, wp, scales, GROUP: int = 128, ZP: int = 8, WORLD: int = 1, GATHER: int = 1, **kwargs):
    """The full [M, N] product; what every rank must hold after the gather."""
    return gemm_w4a16(a, wp, scales, GROUP, ZP)
