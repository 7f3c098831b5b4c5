"""N-partitioned execution over the GPUs of one node: one process per GPU, torch.distributed for
the plumbing, no data-path collective unless a replicated result is asked for.

  partition(n, world, rank)        rows [lo, hi) of the weight a rank owns (128-row tiles never straddle)
  gemm_w4a16_partitioned(...)      local GEMM on the rank's slice; gather=True all-gathers the column
                                   slices into [M, N] on every rank
Three gathers:
  "fused"  the GEMM epilogue stores every finished tile into the output buffer of EVERY rank
           (tb200_gemm_w4a16_gather: TMA store locally, 128-bit peer stores over NVLink), so the transfer
           overlaps the main loop.  The [M, N] output lives in a symmetric-memory buffer that is
           allocated once per shape and reused (peers must have it mapped before the call).
  "push"   the GEMM writes its slice in place into this rank's symmetric [M, N] buffer, then one streaming
           kernel (tb200_allgather_cols) pushes the slice into the same columns of every peer's buffer:
           slices land at their final strided place, no staging buffer and no interleave pass.  The
           unfused counterpart of "fused" (compute, then exchange).
  "nccl"   the library baseline: one NCCL all-gather of the contiguous per-rank slices [M, N/G] into a
           staging buffer [G, M, N/G], then one interleave pass into a row-major [M, N].  NCCL moves
           contiguous buffers only, so the strided landing costs that extra pass.
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


_symm_cache: dict = {}


def symmetric_output(m: int, n: int, device) -> tuple:
    """(tensor [m, n] fp16, handle) of a symmetric-memory buffer every rank has mapped; cached per shape."""
    import torch.distributed._symmetric_memory as symm_mem
    key = (m, n, str(device))
    if key not in _symm_cache:
        t = symm_mem.empty((m, n), dtype=torch.float16, device=device)
        hdl = symm_mem.rendezvous(t, dist.group.WORLD)
        _symm_cache[key] = (t, hdl)
    return _symm_cache[key]


def gemm_w4a16_push_gather(a, wp_local, scales_local, group_size: int = 128, zp: int = 8, workspace=None):
    """out = a @ dequant(wp)^T on every rank: local GEMM into this rank's columns of the symmetric buffer, then
    one push kernel to the peers.  Returns the shared buffer (overwritten by the next call)."""
    from tilebench_b200 import native
    ext = native.load()
    world, rank = world_and_rank()
    m, k = a.shape
    n_local = wp_local.shape[0]
    n = n_local * world
    out, hdl = symmetric_output(m, n, a.device)
    ws_bytes = ext.gemm_w4a16_workspace_bytes(m, n_local, k)
    if ws_bytes and workspace is None:
        workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=a.device)
    hdl.barrier()            # every rank is done reading the previous contents
    ext.gemm_w4a16(a, wp_local.contiguous(), scales_local.contiguous(), out, int(group_size), int(zp), rank * n_local, workspace)
    ext.allgather_cols(out[:, rank * n_local:(rank + 1) * n_local], [int(p) for p in hdl.buffer_ptrs], rank, n)
    hdl.barrier()            # every rank's stores have landed
    return out


def gemm_w4a16_fused_gather(a, wp_local, scales_local, group_size: int = 128, zp: int = 8):
    """out = a @ dequant(wp)^T on every rank, the all-gather done by the GEMM's epilogue (see module doc).
    Returns the shared symmetric buffer: its contents are overwritten by the next call."""
    from tilebench_b200 import native
    ext = native.load()
    world, rank = world_and_rank()
    m, k = a.shape
    n = wp_local.shape[0] * world
    out, hdl = symmetric_output(m, n, a.device)
    hdl.barrier()            # every rank is done reading the previous contents
    ext.gemm_w4a16_gather(a, wp_local.contiguous(), scales_local.contiguous(), [int(p) for p in hdl.buffer_ptrs], rank, n,
                          int(group_size), int(zp))
    hdl.barrier()            # every rank's stores have landed
    return out


def gemm_w4a16_partitioned(a, wp_local, scales_local, group_size: int = 128, zp: int = 8, gather=True,
                           workspace=None, out_local=None):
    """This rank's slice of out = a @ dequant(wp)^T, or the full [M, N]: gather=True / "nccl" gathers with
    NCCL into a fresh tensor, gather="fused" uses the epilogue peer stores (m > 64, world > 1), gather="push"
    the separate push kernel.  `out_local` ([M, n_local] fp16) and `workspace` may be passed in to keep
    allocation out of a timed loop."""
    from tilebench_b200 import native
    ext = native.load()
    m, k = a.shape
    n_local = wp_local.shape[0]
    if gather == "fused" and world_and_rank()[0] > 1 and m > 64:
        return gemm_w4a16_fused_gather(a, wp_local, scales_local, group_size, zp)
    if gather == "push" and world_and_rank()[0] > 1:
        return gemm_w4a16_push_gather(a, wp_local, scales_local, group_size, zp, workspace)
    if out_local is None:
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
