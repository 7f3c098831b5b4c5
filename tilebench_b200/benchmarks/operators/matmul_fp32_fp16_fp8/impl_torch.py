"""Torch reference of matmul_fp32_fp16_fp8, same arithmetic as the reference operator
(tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27): torch.matmul for fp32 (TF32 allowed
on the GPU) and fp16; for e4m3 a unit-scale torch._scaled_mm with bf16 output, cast back to e4m3.  On CPU,
where _scaled_mm with scale vectors is not available, the e4m3 path multiplies the decoded operands in fp32
and applies the same two roundings.  The column-major copy of b that _scaled_mm needs is rebuilt on every
call: nothing is cached across calls."""
import torch

torch.backends.cuda.matmul.allow_tf32 = True


def run(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.dtype == torch.float8_e4m3fn:
        if a.is_cuda:
            ones_a = torch.ones(a.shape[0], 1, device=a.device, dtype=torch.float32)
            ones_b = torch.ones(1, b.shape[1], device=b.device, dtype=torch.float32)
            out = torch._scaled_mm(a, b.t().contiguous().t(), scale_a=ones_a, scale_b=ones_b, out_dtype=torch.bfloat16)
        else:
            out = torch.matmul(a.float(), b.float()).bfloat16()
        return out.to(a.dtype)
    return torch.matmul(a, b)
