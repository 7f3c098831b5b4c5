"""cuda backend of gemm_w4a16_npart: each rank runs the W4A16 GEMM on its slice of the weight rows.
GATHER = 0 keeps the per-rank column slice, 1 all-gathers the slices with NCCL, 2 lets the GEMM epilogue
store every tile into all ranks' output buffers, 3 pushes the finished slice with a separate kernel
(tilebench_b200.npart)."""
import torch

from tilebench_b200 import npart


def run(a, wp, scales, GROUP: int = 128, ZP: int = 8, WORLD: int = 1, GATHER: int = 1, **kwargs):
    world, rank = npart.world_and_rank()
    if int(WORLD) != world:
        raise RuntimeError(f"gemm_w4a16_npart: case wants WORLD={WORLD} ranks, process group has {world}")
    lo, hi = npart.partition(wp.shape[0], world, rank)
    mode = {0: False, 1: "nccl", 2: "fused", 3: "push"}[int(GATHER)]
    out = npart.gemm_w4a16_partitioned(a, wp[lo:hi], scales[lo:hi], int(GROUP), int(ZP), gather=mode)
    if not GATHER and world > 1:
        # verification compares against the full product: place the local slice, leave the rest to the peers
        raise RuntimeError("gemm_w4a16_npart: GATHER=0 leaves a column slice per rank; verify it with npart tests")
    return out
