"""Torch reference of matmul_int8: A int8 [M, K] times the weights packed four 2-bit fields per byte in
b uint8 [K/4, N], int32 result.  Same semantics as the reference operator
(tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19): field i of byte b[kb, n] is the weight of
row i * K/4 + kb, stored with an offset of one.  The products are summed in fp32 like the reference does;
every partial sum is an integer below 2**24 for K <= 20480 (|a| <= 64, |w| <= 2), so the sum is exact."""
import torch


def run(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    M, K = a.shape
    K_b, N = b.shape
    if K != 4 * K_b:
        raise ValueError(f"a has K={K} but b has {K_b} packed rows; K must be 4 * K_b")
    fields = torch.stack([(b >> (2 * i)) & 3 for i in range(4)])           # [4, K_b, N]
    weights = (fields.to(torch.int8) - 1).reshape(K, N)
    return torch.matmul(a.to(torch.float32), weights.to(torch.float32)).to(torch.int32)
