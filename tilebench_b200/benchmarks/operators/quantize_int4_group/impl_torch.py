import torch

from tilebench_b200.data.tensors import quantize_int4_groupwise


def run(x: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    """(wp uint8 [N, K/2], scales fp16 [N, K/GROUP]): s = fp16(amax / 7) per group, q = clamp(round(x / s) + ZP, 0, 15)."""
    return quantize_int4_groupwise(x, int(GROUP), int(ZP))
