import torch


def unpack_int4(wp: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/2] -> int16 [N, K]; low nibble = even k, high nibble = odd k."""
    lo = (wp & 0xF).to(torch.int16)
    hi = (wp >> 4).to(torch.int16)
    return torch.stack((lo, hi), dim=-1).reshape(wp.shape[0], wp.shape[1] * 2)


def run(wp: torch.Tensor, scales: torch.Tensor, GROUP: int = 128, ZP: int = 8, **kwargs):
    q = unpack_int4(wp)
    s = scales.to(torch.float32).repeat_interleave(GROUP, dim=1)
    return ((q - ZP).to(torch.float32) * s).to(torch.float16)
