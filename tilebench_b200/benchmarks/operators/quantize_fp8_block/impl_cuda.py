"""cuda backend of quantize_fp8_block: one streaming kernel per block shape (tb200_quantize_fp8_block)."""
import torch

from tilebench_b200 import native


def run(x: torch.Tensor, BLOCK_ROWS: int = 1, **kwargs):
    ext = native.load()
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty((rows // int(BLOCK_ROWS), cols // 128), dtype=torch.float32, device=x.device)
    ext.quantize_fp8_block(x, q, scales, int(BLOCK_ROWS))
    return q, scales
