"""Two-GPU checks of the N-partitioned W4A16 GEMM (needs >= 2 GPUs; skipped on a single-GPU box):
the NCCL gather, the push kernel and the fused epilogue gather must all reproduce the single-GPU result on
every rank."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from tilebench_b200 import native, npart
        from tilebench_b200.data import tensors
        M, K, N = 300, 1024, 1024
        a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, device="cpu", seed=12)
        a, wp, sc = a.to(dev), wp.to(dev), sc.to(dev)
        lo, hi = npart.partition(N, world, rank)
        native.clear_device_status()
        via_nccl = npart.gemm_w4a16_partitioned(a, wp[lo:hi], sc[lo:hi], group, zp, gather="nccl")
        pushed = npart.gemm_w4a16_partitioned(a, wp[lo:hi], sc[lo:hi], group, zp, gather="push").clone()
        fused = npart.gemm_w4a16_partitioned(a, wp[lo:hi], sc[lo:hi], group, zp, gather="fused")
        torch.cuda.synchronize()
        fused_copy = fused.clone()
        again = npart.gemm_w4a16_partitioned(a, wp[lo:hi], sc[lo:hi], group, zp, gather="fused").clone()
        torch.cuda.synchronize()
        # the same fused gather with the tiles pushed by the epilogue threads' own stores instead of TMA stores
        os.environ["TB200_W4_GATHER"] = "stores"
        by_threads = npart.gemm_w4a16_partitioned(a, wp[lo:hi], sc[lo:hi], group, zp, gather="fused").clone()
        torch.cuda.synchronize()
        os.environ.pop("TB200_W4_GATHER")
        assert native.device_status()[0] == 0
        torch.save({"nccl": via_nccl.cpu(), "push": pushed.cpu(), "fused": fused_copy.cpu(), "again": again.cpu(),
                    "by_threads": by_threads.cpu()}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_gpu_partitioned_gemm_gathers_agree(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda
    from tilebench_b200.data import tensors
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(300, 1024, 1024, device="cuda", seed=12)
    single = impl_cuda.run(a, wp, sc, group, zp).cpu()
    for r in range(world):
        got = torch.load(tmp_path / f"r{r}.pt")
        assert torch.equal(got["nccl"], single), f"rank {r}: NCCL gather differs from the single-GPU result"
        assert torch.equal(got["push"], single), f"rank {r}: push gather differs from the single-GPU result"
        assert torch.equal(got["fused"], single), f"rank {r}: fused gather differs from the single-GPU result"
        assert torch.equal(got["again"], single)
        assert torch.equal(got["by_threads"], single), f"rank {r}: fused gather by thread stores differs"
