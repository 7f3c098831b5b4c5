"""The allocation-free W4A16 entry point (tb200_gemm_w4a16_static) against the ordinary one.

Some users of the library cannot hand it a workspace: they run where device allocation is not
available to them (all memory already belongs to the host application's pool, or allocation calls
are forbidden at that point).  For them the split-K partial sums live in a fixed array inside the
library.  This test calls both entry points through the C ABI on the same inputs, twice in a row
with different data.  Both run the same kernels with the same split of K and add the partial sums
in the same order, so the fp16 results must be equal bit for bit (which is inside the GEMM
tolerance used elsewhere, atol 1e-3 / rtol 1e-3) — the second call proves that whatever the first
left in the shared array does not leak into later results.  The file sorts last so a `-x` run reaches it after everything else.
"""
import ctypes

import pytest
import torch

from tilebench_b200 import native
from tilebench_b200.data import tensors

pytestmark = pytest.mark.gpu


def vp(t):
    return ctypes.c_void_p(t.data_ptr())


def run_pair(lib, dev, m, n, k, seed):
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(m, k, n, device="cpu", seed=seed)
    a, wp, sc = a.to(dev), wp.to(dev), sc.to(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.tb200_gemm_w4a16_workspace_bytes(m, n, k)
    ws = torch.empty(max(need // 4, 1), dtype=torch.float32, device=dev)
    ref = torch.empty(m, n, dtype=torch.float16, device=dev)
    rc = lib.tb200_gemm_w4a16(vp(a), vp(wp), vp(sc), vp(ref), m, n, k, group, zp, n, 0, vp(ws), need, stream)
    assert rc == 0, native.last_error()
    got = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
    rc = lib.tb200_gemm_w4a16_static(vp(a), vp(wp), vp(sc), vp(got), m, n, k, group, zp, n, 0, stream)
    assert rc == 0, native.last_error()
    torch.cuda.synchronize()
    return need, got, ref


def test_static_scratch_matches_workspace_entry_point_twice(cuda_device):
    lib = native.capi()
    assert lib.tb200_gemm_w4a16_static_scratch_bytes() == 16 << 20
    native.clear_device_status()
    # small m above the streaming kernel's range on a narrow weight (32 tiles of 128 rows): the tensor-memory
    # GEMM splits K there, so the built-in array is really used
    for seed, m in ((101, 24), (202, 17)):
        need, got, ref = run_pair(lib, cuda_device, m, 4096, 4096, seed)
        assert 0 < need <= 16 << 20
        assert not torch.isnan(got).any()
        assert torch.equal(got, ref)
    assert native.device_status()[0] == 0


def test_static_entry_point_without_scratch_and_over_the_limit(cuda_device):
    lib = native.capi()
    need, got, ref = run_pair(lib, cuda_device, 256, 512, 1024, seed=303)      # large m: no scratch at all
    assert need == 0
    assert torch.equal(got, ref)
    # a shape whose partial sums do not fit is refused with a message, not run
    m, k = 64, 4096
    n = next((c for c in (9216, 8192, 7168, 6144) if lib.tb200_gemm_w4a16_workspace_bytes(m, c, k) > 16 << 20), None)
    if n is None:
        pytest.skip("no probe shape exceeds the built-in array on this device")
    t = torch.zeros(16, dtype=torch.uint8, device=cuda_device)
    rc = lib.tb200_gemm_w4a16_static(vp(t), vp(t), vp(t), vp(t), m, n, k, 128, 8, n, 0, None)
    assert rc == 5 and "built-in array" in native.last_error()
