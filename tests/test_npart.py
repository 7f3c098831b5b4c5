"""N-partition host logic on CPU ranks: partition -> per-rank oracle -> all-gather over gloo must
reproduce the single-process result on every rank (world size 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tilebench_b200 import npart


def test_partition_rules():
    assert npart.partition(57344, 8, 3) == (3 * 7168, 4 * 7168)
    assert npart.partition(14336, 1, 0) == (0, 14336)
    for world in (1, 2, 4, 8):
        spans = [npart.partition(57344, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 57344
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((hi - lo) % 128 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        npart.partition(14336, 3, 0)
    with pytest.raises(ValueError):
        npart.partition(1024, 2, 2)


def test_interleave_slices_layout():
    staging = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = npart.interleave_slices(staging)
    assert full.shape == (3, 8)
    assert torch.equal(full[:, :4], staging[0]) and torch.equal(full[:, 4:], staging[1])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import ref_ops
        from tilebench_b200.data import tensors
        a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(8, 256, 512, device="cpu", seed=3)

        def local(a_, wp_, sc_):
            return torch.from_numpy(ref_ops.gemm_w4a16(a_.numpy(), wp_.numpy(), sc_.numpy(), group, zp))
        full = npart.partitioned_reference(local, a, wp, sc, gather=True)
        mine = npart.partitioned_reference(local, a, wp, sc, gather=False)
        np.save(os.path.join(out_dir, f"full_{rank}.npy"), full.numpy())
        np.save(os.path.join(out_dir, f"mine_{rank}.npy"), mine.numpy())
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reproduce_the_single_process_result(tmp_path):
    from oracle import ref_ops
    from tilebench_b200.data import tensors
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(8, 256, 512, device="cpu", seed=3)
    want = ref_ops.gemm_w4a16(a.numpy(), wp.numpy(), sc.numpy(), group, zp)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"full_{r}.npy"), want)
        lo, hi = npart.partition(512, world, r)
        assert np.array_equal(np.load(tmp_path / f"mine_{r}.npy"), want[:, lo:hi])
