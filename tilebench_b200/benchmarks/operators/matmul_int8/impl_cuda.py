"""cuda backend of the reference operator matmul_int8: tb200_matmul_int8_packed2 (tcgen05 kind::i8, the
2-bit fields unpacked in shared memory into MN-major operand planes).  Signature follows the reference's
Triton backend (tilebench/benchmarks/operators/matmul_int8/impl_triton.py:118-119)."""
import torch

from tilebench_b200 import native


def run(a: torch.Tensor, b: torch.Tensor, block_size=None, autotune: bool = False, **kwargs):
    ext = native.load()
    if a.dtype != torch.int8 or b.dtype != torch.uint8:
        raise ValueError(f"matmul_int8 expects int8 a and uint8 b, got {a.dtype} and {b.dtype}")
    if a.shape[1] != 4 * b.shape[0]:
        raise ValueError(f"a has K={a.shape[1]} but b has {b.shape[0]} packed rows; K must be 4 * K_b")
    out = torch.empty((a.shape[0], b.shape[1]), dtype=torch.int32, device=a.device)
    ext.matmul_int8_packed2(a.contiguous(), b.contiguous(), out)
    return out
