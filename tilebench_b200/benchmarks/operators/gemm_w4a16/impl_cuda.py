"""cuda backend of gemm_w4a16: TMA-staged packed int4, in-warp dequant into TMEM, tcgen05 MMA
(tb200_gemm_w4a16); decode-sized M adds a deterministic split-K reduction kernel."""
import torch

from tilebench_b200 import native


def run(a: torch.Tensor, wp: torch.Tensor, scales: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    ext = native.load()
    m, k = a.shape
    n = wp.shape[0]
    out = torch.empty((m, n), dtype=torch.float16, device=a.device)
    ws_bytes = ext.gemm_w4a16_workspace_bytes(m, n, k)
    ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=a.device) if ws_bytes else None
    ext.gemm_w4a16(a, wp, scales, out, int(GROUP), int(ZP), 0, ws)
    return out
