"""cuda backend of gemm_fp8_blockscaled: tcgen05 kind::f8f6f4 with per-K-block scale application
while draining TMEM (tb200_gemm_fp8_blockscaled)."""
import torch

from tilebench_b200 import native


def run(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor, BLOCK: int = 128, **kwargs):
    if int(BLOCK) != 128:
        raise NotImplementedError("gemm_fp8_blockscaled: the kernel implements 1x128 / 128x128 scale blocks only")
    ext = native.load()
    out = torch.empty((aq.shape[0], bq.shape[0]), dtype=torch.bfloat16, device=aq.device)
    ext.gemm_fp8_blockscaled(aq, sa, bq, sb, out)
    return out
