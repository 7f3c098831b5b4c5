"""Threaded CPU baseline of the path — TEST / BASELINE INFRASTRUCTURE, not product code.

The reference's implementation of this path is its per-operator PyTorch `impl_torch.run`
(tilebench/benchmarks/operators/*/impl_torch.py), which runs on whatever device its inputs live
on.  These are the same formulas restated for CPU tensors so `bench.py --impl reference` and the
`cpu_baseline` leg can time them on every host core (torch's intra-op thread pool).  ref_ops.py
holds the numpy statements that the parity tests check against.
"""
from __future__ import annotations

import os

import torch


def use_all_cores() -> int:
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def dequant_int8_channel(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """bf16(float(w) * scale[r]) — form of dequantize_rowwise/impl_torch.py:4-7 without the 1/127."""
    return (w.to(torch.float32) * scale.unsqueeze(1)).to(torch.bfloat16)


def dequantize_rowwise(x: torch.Tensor, state_x: torch.Tensor) -> torch.Tensor:
    """dequantize_rowwise/impl_torch.py:4-7."""
    return (state_x.unsqueeze(1) * x * (1.0 / 127.0)).to(torch.float16)


def dequant_int4_group(wp: torch.Tensor, scales: torch.Tensor, group: int = 128, zp: int = 8) -> torch.Tensor:
    lo = (wp & 0xF).to(torch.int16)
    hi = (wp >> 4).to(torch.int16)
    q = torch.stack((lo, hi), dim=-1).reshape(wp.shape[0], wp.shape[1] * 2)
    return ((q - zp).to(torch.float32) * scales.to(torch.float32).repeat_interleave(group, dim=1)).to(torch.float16)


def gemm_w4a16(a, wp, scales, group: int = 128, zp: int = 8) -> torch.Tensor:
    """Unpack, then an fp32 matmul — the shape of matmul_int8/impl_torch.py:10-19."""
    w = dequant_int4_group(wp, scales, group, zp).to(torch.float32)
    return torch.matmul(a.to(torch.float32), w.t()).to(torch.float16)


def gemm_fp8_blockscaled(aq, sa, bq, sb, block: int = 128) -> torch.Tensor:
    a = aq.to(torch.float32) * sa.repeat_interleave(block, dim=1)
    b = bq.to(torch.float32) * sb.repeat_interleave(block, dim=0).repeat_interleave(block, dim=1)
    return torch.matmul(a, b.t()).to(torch.bfloat16)
