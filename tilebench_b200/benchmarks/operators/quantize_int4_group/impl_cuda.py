"""cuda backend of quantize_int4_group: one streaming kernel, half a warp per group (tb200_quantize_int4_group)."""
import torch

from tilebench_b200 import native


def run(x: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    ext = native.load()
    n, k = x.shape
    wp = torch.empty((n, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((n, k // int(GROUP)), dtype=torch.float16, device=x.device)
    ext.quantize_int4_group(x.contiguous(), wp, scales, int(GROUP), int(ZP))
    return wp, scales
