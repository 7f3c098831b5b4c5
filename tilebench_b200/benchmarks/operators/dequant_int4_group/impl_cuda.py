"""cuda backend of dequant_int4_group: one streaming kernel (tb200_dequant_int4_group)."""
import torch

from tilebench_b200 import native


def run(wp: torch.Tensor, scales: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    ext = native.load()
    out = torch.empty((wp.shape[0], wp.shape[1] * 2), dtype=torch.float16, device=wp.device)
    ext.dequant_int4_group(wp, scales, out, int(GROUP), int(ZP))
    return out
