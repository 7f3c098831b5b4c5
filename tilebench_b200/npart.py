"""N-partitioned execution over the GPUs of one node: one process per GPU, torch.distributed for
the plumbing, no data-path collective unless a replicated result is asked for.

  partition(n, world, rank)        rows [lo, hi) of the weight a rank owns (128-row tiles never straddle)
  gemm_w4a16_partitioned(...)      local GEMM on the rank's slice; gather=True all-gathers the column
                                   slices into [M, N] on every rank
The gather uses one NCCL all-gather of the contiguous per-rank slices [M, N/G] into a staging
buffer [G, M, N/G], followed by one interleave pass into row-major [M, N].
`partitioned_reference` runs the same partition -> local op -> gather path with any local function
and any backend (gloo on CPU), which is how the host logic is tested without GPUs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def world_and_rank() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def partition(n: int, world: int, rank: int, tile: int = 128) -> tuple[int, int]:
    """Even split of n rows in whole tiles; raises when n / world is not a multiple of `tile`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if n % (world * tile) != 0:
        raise ValueError(f"n={n} does not split into {world} slices of whole {tile}-row tiles")
    per = n // world
    return rank * per, (rank + 1) * per


def interleave_slices(staging: torch.Tensor) -> torch.Tensor:
    """[G, M, n] gathered slices -> [M, G*n] row-major (slice g holds columns [g*n, (g+1)*n))."""
    G, M, n = staging.shape
    return staging.permute(1, 0, 2).reshape(M, G * n)


def all_gather_columns(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of per-rank column slices [M, n] into [M, world*n] on every rank."""
    world, _ = world_and_rank()
    if world == 1:
        return local
    local = local.contiguous()
    staging = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(staging, local, group=group)     # one ncclAllGather, no extra copies
    else:
        dist.all_gather(list(staging.unbind(0)), local, group=group)  # gloo (CPU tests)
    return interleave_slices(staging)


def gemm_w4a16_partitioned(a, wp_local, scales_local, group_size: int = 128, zp: int = 8, gather: bool = True,
                           workspace=None):
    """This rank's slice of out = a @ dequant(wp)^T; the full [M, N] when gather=True."""
    from tilebench_b200 import native
    ext = native.load()
    m, k = a.shape
    n_local = wp_local.shape[0]
    out_local = torch.empty((m, n_local), dtype=torch.float16, device=a.device)
    ws_bytes = ext.gemm_w4a16_workspace_bytes(m, n_local, k)
    if ws_bytes and workspace is None:
        workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=a.device)
    ext.gemm_w4a16(a, wp_local.contiguous(), scales_local.contiguous(), out_local, int(group_size), int(zp), 0, workspace)
    return all_gather_columns(out_local) if gather else out_local


def partitioned_reference(local_fn, a, wp, scales, gather: bool = True):
    """Host-logic twin of gemm_w4a16_partitioned: `local_fn(a, wp_slice, scales_slice)` computes the
    rank's [M, n_local] slice with whatever implementation the caller passes (tests pass the oracle)."""
    world, rank = world_and_rank()
    lo, hi = partition(wp.shape[0], world, rank)
    local = local_fn(a, wp[lo:hi], scales[lo:hi])
    return all_gather_columns(local) if gather else local
