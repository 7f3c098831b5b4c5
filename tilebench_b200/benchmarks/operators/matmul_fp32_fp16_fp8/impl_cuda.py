"""cuda backend of the reference operator matmul_fp32_fp16_fp8: tb200_matmul_plain (tcgen05 kind::f16 /
kind::tf32 / kind::f8f6f4 with b read as an MN-major operand, so no transposed copy of b exists).
Signature follows the reference's Triton backend (block_size / autotune accepted and ignored)."""
import torch

from tilebench_b200 import native

_SUPPORTED = (torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn)


def run(a: torch.Tensor, b: torch.Tensor, block_size=None, autotune: bool = False, **kwargs):
    ext = native.load()
    if a.dtype != b.dtype or a.dtype not in _SUPPORTED:
        raise NotImplementedError(f"matmul_fp32_fp16_fp8 cuda backend supports float32, float16, bfloat16 and float8_e4m3fn, got {a.dtype} x {b.dtype}")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"shapes {tuple(a.shape)} x {tuple(b.shape)} do not form a GEMM")
    out = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=a.device)
    ext.matmul_plain(a.contiguous(), b.contiguous(), out)
    return out
