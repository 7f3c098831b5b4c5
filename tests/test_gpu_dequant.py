"""GPU parity of the streaming dequant kernels against the CPU oracle: bit-exact, through the
operator entry point (impl_cuda.run -> PyTorch extension -> C ABI) and through ctypes on the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ref_ops
from tilebench_b200 import native
from tilebench_b200.data import tensors

pytestmark = pytest.mark.gpu


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("N,K,group", [(4096, 4096, 128), (256, 1024, 128), (64, 256, 32), (3, 128, 8), (17, 384, 64)])
def test_int4_group_bit_exact(cuda_device, N, K, group):
    from tilebench_b200.benchmarks.operators.dequant_int4_group import impl_cuda
    wp, sc = tensors.make_int4_group_weights(N, K, group, seed=11 + N)
    out = impl_cuda.run(wp.to(cuda_device), sc.to(cuda_device), group, 8)
    torch.cuda.synchronize()
    want = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), group, 8)
    assert np.array_equal(bits16(out), want.view(np.uint16))


def test_int4_all_nibbles_all_zero_points(cuda_device):
    ext = native.load()
    wp = torch.tensor([[(2 * i) | ((2 * i + 1) << 4) for i in range(8)]], dtype=torch.uint8)
    sc = torch.tensor([[0.3333]], dtype=torch.float16)
    for zp in range(16):
        out = torch.empty(1, 16, dtype=torch.float16, device=cuda_device)
        ext.dequant_int4_group(wp.to(cuda_device), sc.to(cuda_device), out, 16, zp)
        want = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 16, zp)
        assert np.array_equal(bits16(out), want.view(np.uint16)), zp


def test_int4_scalar_path_ragged_group(cuda_device):
    # group 4 is not a multiple of 8: the one-element-per-thread kernel runs
    ext = native.load()
    wp, _ = tensors.make_int4_group_weights(5, 24, 8, seed=3)
    sc = (torch.rand(5, 6) * 0.1 + 0.01).half()
    out = torch.empty(5, 24, dtype=torch.float16, device=cuda_device)
    ext.dequant_int4_group(wp.to(cuda_device), sc.to(cuda_device), out, 4, 8)
    assert np.array_equal(bits16(out), ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 4, 8).view(np.uint16))


def test_int4_subnormal_products_are_kept(cuda_device):
    ext = native.load()
    wp = torch.full((1, 64), 0x9F, dtype=torch.uint8)           # q = 15, 9 -> (q - 8) = 7, 1
    sc = torch.tensor([[6.0e-8]], dtype=torch.float16)          # fp16 subnormal scale
    out = torch.empty(1, 128, dtype=torch.float16, device=cuda_device)
    ext.dequant_int4_group(wp.to(cuda_device), sc.to(cuda_device), out, 128, 8)
    want = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 128, 8)
    assert want.astype(np.float32).max() > 0
    assert np.array_equal(bits16(out), want.view(np.uint16))


def test_int4_strided_output_and_guard_bands(cuda_device):
    # write a [n, k] result into the middle columns of a wider, sentinel-filled buffer via the C ABI
    lib = native.capi()
    n, k, ldo = 32, 256, 512
    wp, sc = tensors.make_int4_group_weights(n, k, 128, seed=5)
    wpd, scd = wp.to(cuda_device), sc.to(cuda_device)
    buf = torch.full((n + 2, ldo), 123.0, dtype=torch.float16, device=cuda_device)
    out_view = buf[1:n + 1, 128:128 + k]
    rc = lib.tb200_dequant_int4_group(ptr(wpd), ptr(scd), ctypes.c_void_p(out_view.data_ptr()), n, k, 128, 8, ldo, stream_ptr())
    assert rc == 0, native.last_error()
    torch.cuda.synchronize()
    want = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 128, 8)
    assert np.array_equal(bits16(out_view.contiguous()), want.view(np.uint16))
    untouched = buf.clone()
    untouched[1:n + 1, 128:128 + k] = 123.0
    assert torch.all(untouched == 123.0)


@pytest.mark.parametrize("rows,cols", [(256, 4096), (4096, 4096), (7, 4096), (33, 264), (5, 37)])
def test_int8_channel_bit_exact(cuda_device, rows, cols):
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    w, s = tensors.generate_dequant_int8_channel_inputs(rows, cols, device="cpu", seed=100 + rows)
    out = impl_cuda.run(w.to(cuda_device), s.to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(bits16(out), ref_ops.dequant_int8_channel(w.numpy(), s.numpy()))


def test_int8_channel_full_size_chunked_check(cuda_device):
    """65536 x 4096 (268M elements): compared with the oracle in row blocks, and by a checksum."""
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    rows, cols = 65536, 4096
    w, s = tensors.generate_dequant_int8_channel_inputs(rows, cols, device="cpu", seed=77)
    out = impl_cuda.run(w.to(cuda_device), s.to(cuda_device))
    torch.cuda.synchronize()
    for r0 in (0, 30000, rows - 2048):
        want = ref_ops.dequant_int8_channel(w[r0:r0 + 2048].numpy(), s[r0:r0 + 2048].numpy())
        assert np.array_equal(bits16(out[r0:r0 + 2048]), want)
    # linearity in the scale: doubling every scale doubles every output exactly (power of two)
    out2 = impl_cuda.run(w.to(cuda_device), (s * 2).to(cuda_device))
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_int4_group_matches_reference_fixture(cuda_device, golden_cfg, tag):
    # expected output computed by the reference's own multiply operator (tests/golden/make_golden.py)
    ext = native.load()
    group, zp = (int(v) for v in golden_cfg[f"i4_{tag}_gz"])
    wp = torch.from_numpy(golden_cfg[f"i4_{tag}_wp"]).to(cuda_device)
    sc = torch.from_numpy(golden_cfg[f"i4_{tag}_s"]).to(cuda_device)
    out = torch.empty(wp.shape[0], wp.shape[1] * 2, dtype=torch.float16, device=cuda_device)
    ext.dequant_int4_group(wp, sc, out, group, zp)
    assert np.array_equal(bits16(out), golden_cfg[f"i4_{tag}_out"].view(np.uint16))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_int8_channel_matches_reference_fixture(cuda_device, golden_cfg, tag):
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    out = impl_cuda.run(torch.from_numpy(golden_cfg[f"i8_{tag}_w"]).to(cuda_device),
                        torch.from_numpy(golden_cfg[f"i8_{tag}_scale"]).to(cuda_device))
    assert np.array_equal(bits16(out), golden_cfg[f"i8_{tag}_out"])


def test_int4_quantiser_matches_reference_fixture(cuda_device, golden_cfg):
    from tilebench_b200.benchmarks.operators.quantize_int4_group import impl_cuda
    wp, s = impl_cuda.run(torch.from_numpy(golden_cfg["q4_x"]).to(cuda_device), 128, 8)
    assert np.array_equal(wp.cpu().numpy(), golden_cfg["q4_wp"])
    assert np.array_equal(bits16(s), golden_cfg["q4_s"].view(np.uint16))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_dequantize_rowwise_matches_reference_fixture(cuda_device, golden, tag):
    from tilebench_b200.benchmarks.operators.dequantize_rowwise import impl_cuda
    x = torch.from_numpy(golden[f"dr_{tag}_x"]).to(cuda_device)
    st = torch.from_numpy(golden[f"dr_{tag}_state"]).to(cuda_device)
    out = impl_cuda.run(x, st)
    assert np.array_equal(bits16(out), golden[f"dr_{tag}_out"].view(np.uint16))


def test_dequantize_every_int8_value_keeps_its_sign(cuda_device):
    # the reference's own GPU test of this path: tests/test_arch_dispatch.py:159-170
    from tilebench_b200.benchmarks.operators.dequantize_rowwise import impl_cuda, impl_torch
    x = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8).reshape(1, 256).repeat(4, 1).to(cuda_device)
    st = torch.tensor([0.5, 1.0, 3.0, 10.0], device=cuda_device)
    out = impl_cuda.run(x, st)
    assert torch.equal(torch.sign(out.float()), torch.sign(x.float()))
    torch.testing.assert_close(out, impl_torch.run(x, st), atol=1e-3, rtol=1e-3)
    assert np.array_equal(bits16(out), ref_ops.dequantize_rowwise(x.cpu().numpy(), st.cpu().numpy()).view(np.uint16))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
@pytest.mark.parametrize("dname", ["f32", "f16", "bf16"])
def test_weight_dequant_matches_reference_fixture(cuda_device, golden, tag, dname):
    from tilebench_b200.benchmarks.operators.weight_dequant import impl_cuda
    m, n, t = (int(v) for v in golden[f"wd_{tag}_{dname}_mnt"])
    xs, ss, want = golden[f"wd_{tag}_{dname}_x"], golden[f"wd_{tag}_{dname}_s"], golden[f"wd_{tag}_{dname}_out"]
    if dname == "bf16":
        X = torch.from_numpy(xs.view(np.int16)).view(torch.bfloat16)
        S = torch.from_numpy(ss.view(np.int16)).view(torch.bfloat16)
    else:
        X, S = torch.from_numpy(xs), torch.from_numpy(ss)
    out = impl_cuda.run(X.to(cuda_device), S.to(cuda_device), m, n, t).cpu()
    got = out.view(torch.int16).numpy().view(np.uint16) if dname != "f32" else out.numpy()
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("M,dtype", [(4096, torch.float16), (1536, torch.bfloat16), (1000, torch.float32)])
def test_weight_dequant_reference_grid_sizes(cuda_device, M, dtype):
    from tilebench_b200.benchmarks.operators.weight_dequant import impl_cuda, impl_torch
    X, S, m, n, t = tensors.generate_weight_dequant_inputs(M, 128, dtype, device="cpu", seed=9)
    out = impl_cuda.run(X.to(cuda_device), S.to(cuda_device), m, n, t)
    assert torch.equal(out.cpu(), impl_torch.run(X, S, m, n, t))


def test_anti_cache_fresh_output_same_address_new_values_no_input_mutation(cuda_device):
    """The reference evaluator's anti-cache checks (tilebench/llm/v2/evaluation/anticache.py:93-134)."""
    from tilebench_b200.benchmarks.operators.dequant_int4_group import impl_cuda
    wp, sc = tensors.make_int4_group_weights(128, 512, 128, seed=1)
    wpd, scd = wp.to(cuda_device), sc.to(cuda_device)
    keep = wpd.clone()
    o1 = impl_cuda.run(wpd, scd, 128, 8)
    o2 = impl_cuda.run(wpd, scd, 128, 8)
    assert o1.data_ptr() != o2.data_ptr() and torch.equal(o1, o2)           # fresh storage, deterministic
    assert o1.data_ptr() not in (wpd.data_ptr(), scd.data_ptr())            # no aliasing
    wp2, _ = tensors.make_int4_group_weights(128, 512, 128, seed=2)
    wpd.copy_(wp2)                                                          # same address, new values
    o3 = impl_cuda.run(wpd, scd, 128, 8)
    assert np.array_equal(bits16(o3), ref_ops.dequant_int4_group(wp2.numpy(), sc.numpy(), 128, 8).view(np.uint16))
    assert torch.equal(wpd.cpu(), wp2) and not torch.equal(wpd, keep)       # input not mutated by run()


def test_capi_argument_errors_return_codes(cuda_device):
    lib = native.capi()
    t = torch.zeros(64, dtype=torch.uint8, device=cuda_device)
    assert lib.tb200_dequant_int4_group(None, ptr(t), ptr(t), 1, 8, 8, 8, 8, None) == 1          # null pointer
    assert "null" in native.last_error()
    assert lib.tb200_dequant_int4_group(ptr(t), ptr(t), ptr(t), 1, 7, 8, 8, 8, None) == 1        # odd k
    assert lib.tb200_dequant_int4_group(ptr(t), ptr(t), ptr(t), 1, 8, 8, 16, 8, None) == 1       # zero point
    assert lib.tb200_dequant_int8_rowwise(ptr(t), ptr(t), ptr(t), 1, 8, 0, 0, 1.0, None) == 3    # fp32 out unsupported
    assert lib.tb200_weight_dequant_block(ptr(t), ptr(t), ptr(t), 1, 8, 0, 1, None) == 1         # tile 0
    assert lib.tb200_dequant_int4_group(ptr(t), ptr(t), ptr(t), 0, 8, 8, 8, 8, None) == 0        # empty is fine


def test_runs_under_cuda_graph_capture(cuda_device):
    """The reference timer replays run() from a CUDA graph (tilebench/core/timer.py:120-143)."""
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    w, s = tensors.generate_dequant_int8_channel_inputs(512, 1024, device=cuda_device, seed=4)
    impl_cuda.run(w, s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = impl_cuda.run(w, s)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(bits16(out), ref_ops.dequant_int8_channel(w.cpu().numpy(), s.cpu().numpy()))


@pytest.mark.parametrize("rows,cols,block_rows", [(256, 512, 1), (3, 128, 1), (256, 384, 128), (1024, 1024, 128)])
def test_fp8_block_quantiser_bit_exact(cuda_device, rows, cols, block_rows):
    """q and scales must equal the PyTorch formula bit for bit, including an all-zero block and +-amax."""
    from tilebench_b200.benchmarks.operators.quantize_fp8_block import impl_cuda, impl_torch
    x = torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows + cols))
    x[0, :128] = 0.0
    if block_rows == 128:
        x[:128, :128] = 0.0
    q, s = impl_cuda.run(x.to(cuda_device), block_rows)
    q_ref, s_ref = impl_torch.run(x, block_rows)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert q.cpu().float().abs().max() == 448.0


# ---------------------------------------------------------------- int4 group quantiser

@pytest.mark.parametrize("N,K", [(1, 128), (3, 384), (64, 4096), (4096, 4096)])
def test_int4_group_quantiser_bit_exact_and_round_trip(cuda_device, N, K):
    from tilebench_b200.benchmarks.operators.quantize_int4_group import impl_cuda, impl_torch
    from tilebench_b200.benchmarks.operators.dequant_int4_group import impl_cuda as dequant
    x, group, zp = tensors.generate_quantize_int4_group_inputs(N, K, device="cpu", seed=N + K)
    x[0, :128] = 0.0                                        # an all-zero group: scale 1, codes = zero point
    if K > 128:
        x[0, 128] = 3.0                                     # one outlier sets its group's scale
    wp, sc = impl_cuda.run(x.to(cuda_device), group, zp)
    torch.cuda.synchronize()
    owp, osc = ref_ops.quantize_int4_group(x.numpy(), group, zp)
    assert np.array_equal(wp.cpu().numpy(), owp)
    assert np.array_equal(sc.cpu().numpy().view(np.uint16), osc.view(np.uint16))
    twp, tsc = impl_torch.run(x.to(cuda_device), group, zp)            # the same formula evaluated by PyTorch on the GPU
    assert torch.equal(wp, twp) and torch.equal(sc.view(torch.int16), tsc.view(torch.int16))
    back = dequant.run(wp, sc, group, zp).float().cpu()
    step = sc.float().cpu().repeat_interleave(group, dim=1)
    assert torch.all((x - back).abs() <= 0.51 * step)       # half a step + fp16 rounding of (q - zp) * s


def test_int4_group_quantiser_out_of_range_group(cuda_device):
    # amax / 7 beyond the fp16 range: infinite scale, every code of that group is the zero point (same as the formula)
    from tilebench_b200.benchmarks.operators.quantize_int4_group import impl_cuda
    x = torch.full((2, 256), 0.25)
    x[0, 3] = 1.0e6
    wp, s = impl_cuda.run(x.to(cuda_device), 128, 8)
    owp, osc = ref_ops.quantize_int4_group(x.numpy())
    assert np.array_equal(wp.cpu().numpy(), owp) and np.array_equal(bits16(s), osc.view(np.uint16))
    assert torch.isinf(s[0, 0]) and np.all(ref_ops.unpack_int4(owp)[0, :128] == 8)


def test_int4_group_quantiser_rejects_other_groups(cuda_device):
    ext = native.load()
    x = torch.zeros(4, 256, device=cuda_device)
    with pytest.raises(Exception):
        ext.quantize_int4_group(x, torch.empty(4, 128, dtype=torch.uint8, device=cuda_device),
                                torch.empty(4, 4, dtype=torch.float16, device=cuda_device), 64, 8)


def test_host_buffer_pipeline_matches_the_device_operator(cuda_device):
    # chunked upload / kernel / download over three streams must give the same bits as one device call,
    # for a row count that is not a multiple of the chunk and with the staging slots reused several times
    from tilebench_b200 import host_api
    from tilebench_b200.benchmarks.operators.dequant_int8_channel import impl_cuda
    rows, cols = 5000, 1024
    w, scale = tensors.generate_dequant_int8_channel_inputs(rows, cols, device="cpu", seed=11)
    hw, hs = w.pin_memory(), scale.pin_memory()
    hout = torch.empty((rows, cols), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):                                       # second call reuses the cached staging buffers
        host_api.dequant_int8_channel_host(hw, hs, hout, device=cuda_device, chunk_rows=384, depth=3)
        torch.cuda.synchronize()
        want = impl_cuda.run(w.to(cuda_device), scale.to(cuda_device)).cpu()
        assert torch.equal(hout.view(torch.int16), want.view(torch.int16))
    with pytest.raises(ValueError):
        host_api.dequant_int8_channel_host(w.to(cuda_device), hs, hout)


# ---------------------------------------------------------------- wide (256-bit) vs narrow kernel dispatch

def _offset_copy(t, byte_offset):
    """The same values in a fresh allocation whose data pointer is `byte_offset` bytes past a 256-byte boundary."""
    flat = torch.empty(t.numel() * t.element_size() + byte_offset, dtype=torch.uint8, device=t.device)
    view = flat[byte_offset:].view(t.dtype).view(t.shape)
    view.copy_(t)
    return view


@pytest.mark.parametrize("rows,cols", [(2048, 4096), (8192, 4096), (4096, 4104), (3000, 4128)])
def test_int8_wide_and_narrow_kernels_agree(cuda_device, rows, cols):
    # 32-byte aligned operands take the 256-bit kernels (deep or two-chunk variant by size), operands that are
    # only 16-byte aligned, or whose rows are not a multiple of 32, take the 128-bit kernel: same bits either way
    ext = native.load()
    w, scale = tensors.generate_dequant_int8_channel_inputs(rows, cols, device=cuda_device, seed=rows + cols)
    want = ref_ops.dequant_int8_channel(w.cpu().numpy(), scale.cpu().numpy())
    for w_off, o_off in ((0, 0), (16, 0), (0, 16), (8, 16)):
        wv = _offset_copy(w, w_off)
        out = _offset_copy(torch.zeros(rows, cols, dtype=torch.bfloat16, device=cuda_device), o_off)
        ext.dequant_int8_rowwise(wv, scale, out, False, 1.0)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().view(torch.int16).numpy().view(np.uint16), want), (w_off, o_off)


@pytest.mark.parametrize("N,K", [(4096, 4096), (512, 1024), (1024, 4224)])
def test_int4_wide_and_narrow_kernels_agree(cuda_device, N, K):
    ext = native.load()
    wp, sc, group, zp = tensors.generate_dequant_int4_group_inputs(N, K, device=cuda_device, seed=N + K)
    want = ref_ops.dequant_int4_group(wp.cpu().numpy(), sc.cpu().numpy(), group, zp)
    for w_off, o_off in ((0, 0), (4, 0), (0, 16)):
        wv = _offset_copy(wp, w_off)
        out = _offset_copy(torch.zeros(N, K, dtype=torch.float16, device=cuda_device), o_off)
        ext.dequant_int4_group(wv, sc, out, group, zp)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16)), (w_off, o_off)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_weight_dequant_wide_and_narrow_kernels_agree(cuda_device, dtype):
    from tilebench_b200.benchmarks.operators.weight_dequant import impl_torch
    ext = native.load()
    M = N = 2048
    X, S, _, _, T = tensors.generate_weight_dequant_inputs(M, 128, dtype, device=cuda_device, seed=77)
    want = impl_torch.run(X, S, M, N, T)
    for x_off, y_off in ((0, 0), (16, 0), (0, 16)):
        xv = _offset_copy(X, x_off)
        y = _offset_copy(torch.zeros(M, N, dtype=dtype, device=cuda_device), y_off)
        ext.weight_dequant_block(xv, S, y, M, N, T)
        torch.cuda.synchronize()
        assert torch.equal(y.view(torch.uint8), want.view(torch.uint8)), (x_off, y_off)
