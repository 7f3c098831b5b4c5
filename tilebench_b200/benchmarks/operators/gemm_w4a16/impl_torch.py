import torch

from tilebench_b200.benchmarks.operators.dequant_int4_group.impl_torch import run as dequant_int4_group


def run(a: torch.Tensor, wp: torch.Tensor, scales: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    w = dequant_int4_group(wp, scales, GROUP, ZP)          # fp16 [N, K], as the kernel feeds the MMA
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.matmul(a.to(torch.float32), w.to(torch.float32).t()).to(torch.float16)
