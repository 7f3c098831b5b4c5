"""The bounded-wait expiry path, end to end, without faulting or hanging anything: a dedicated one-warp kernel
waits a few microseconds on a barrier nobody arrives on, gives up, records its status and returns; the host
reads the status, clears it, and the context keeps working.  Also the push kernel of the exchange step on one
GPU (two "ranks" are two buffers of the same device)."""
import ctypes

import pytest
import torch

from tilebench_b200 import native

pytestmark = pytest.mark.gpu

ST_WAIT_SELFTEST = 6


def test_bounded_wait_runs_out_and_the_context_stays_usable(cuda_device):
    ext = native.load()
    native.clear_device_status()
    assert native.device_status() == (0, 0)
    limit = 100_000                                   # ~50 us at 1.9 GHz
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ext.selftest_bounded_wait(limit)
    t1.record()
    torch.cuda.synchronize()                          # returns: the kernel ended by itself
    assert t0.elapsed_time(t1) < 50.0                 # ms; far below a hang, above zero
    code, detail = native.device_status()
    assert (code, detail) == (ST_WAIT_SELFTEST, limit)
    # a second expiry does not overwrite the first record; clearing resets it
    ext.selftest_bounded_wait(2 * limit)
    assert native.device_status() == (ST_WAIT_SELFTEST, limit)
    native.clear_device_status()
    assert native.device_status() == (0, 0)
    # the context is intact: a production kernel runs and verifies afterwards
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda, impl_torch
    w = torch.randint(-127, 128, (64, 256), dtype=torch.int8, device=cuda_device)
    s = torch.rand(64, device=cuda_device) + 0.1
    assert torch.equal(impl_cuda.run(w, s), impl_torch.run(w, s))
    assert native.device_status() == (0, 0)


def test_selftest_rejects_limits_outside_its_range(cuda_device):
    ext = native.load()
    with pytest.raises(Exception):
        ext.selftest_bounded_wait(0)
    with pytest.raises(Exception):
        ext.selftest_bounded_wait(1 << 30)
    assert native.device_status() == (0, 0)


@pytest.mark.parametrize("m,n_local,world", [(300, 256, 2), (64, 1792, 8), (5, 8, 3)])
def test_allgather_cols_push_lands_slices_in_place(cuda_device, m, n_local, world):
    """All `world` ranks emulated on one GPU: rank r's slice is pushed into columns [r*n_local, ...) of every
    rank's full buffer; afterwards every buffer equals the concatenation of the slices and guard columns stay."""
    ext = native.load()
    n = world * n_local
    ldo = n + 8
    g = torch.Generator(device=cuda_device).manual_seed(m + n)
    slices = [torch.randn(m, n_local, device=cuda_device, generator=g).half() for _ in range(world)]
    bufs = [torch.full((m, ldo), 9.0, dtype=torch.float16, device=cuda_device) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(world):
        if r % 2 == 0:                               # in place: the slice already sits in the rank's own buffer
            bufs[r][:, r * n_local:(r + 1) * n_local] = slices[r]
            ext.allgather_cols(bufs[r][:, r * n_local:(r + 1) * n_local], ptrs, r, ldo)
        else:                                        # from a separate contiguous slice
            ext.allgather_cols(slices[r], ptrs, r, ldo)
    torch.cuda.synchronize()
    want = torch.cat(slices, dim=1)
    for b in bufs:
        assert torch.equal(b[:, :n], want) and torch.all(b[:, n:] == 9.0)


def test_allgather_cols_rejects_misaligned_slices(cuda_device):
    lib = native.capi()
    buf = torch.zeros(4, 24, dtype=torch.float16, device=cuda_device)
    ptrs = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    rc = lib.tb200_allgather_cols(ctypes.c_void_p(buf.data_ptr()), 24, ptrs, 2, 0, 4, 3, 2, 24, None)   # 6-byte rows
    assert rc == 2 and "16 bytes" in native.last_error()
