"""cuda backend of the reference operator weight_dequant: one streaming kernel
(tb200_weight_dequant_block), same dtype in and out."""
import torch

from tilebench_b200 import native


def run(X: torch.Tensor, S: torch.Tensor, M: int, N: int, TILE_SIZE: int, block_size: int = 1024,
        autotune: bool = False, **kwargs):
    ext = native.load()
    Y = torch.empty_like(X)
    ext.weight_dequant_block(X, S, Y, int(M), int(N), int(TILE_SIZE))
    return Y
