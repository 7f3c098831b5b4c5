"""GPU parity of the tcgen05 GEMMs against the CPU oracle, within the operator's stated tolerance
(fp16: atol 1e-3 / rtol 1e-3; bf16: atol 1e-2 / rtol 1.6e-2), plus exact known-answer cases."""
import numpy as np
import pytest
import torch

from oracle import ref_ops
from tilebench_b200 import native
from tilebench_b200.data import tensors

pytestmark = pytest.mark.gpu

FP16_TOL = dict(atol=1e-3, rtol=1e-3)
BF16_TOL = dict(atol=1e-2, rtol=1.6e-2)


def status_clean():
    code, detail = native.device_status()
    assert code == 0, f"kernel wait timed out: code {code} detail {detail}"


def u8(t):
    return t.view(torch.uint8).cpu().numpy()


# ---------------------------------------------------------------- FP8 block-scaled

def fp8_case(M, N, K, seed, device):
    aq, sa, bq, sb = tensors.generate_gemm_fp8_blockscaled_inputs(M=M, N=N, K=K, device="cpu", seed=seed)
    from tilebench_b200.benchmarks.operators.gemm_fp8_blockscaled import impl_cuda
    native.clear_device_status()
    out = impl_cuda.run(aq.to(device), sa.to(device), bq.to(device), sb.to(device))
    torch.cuda.synchronize()
    status_clean()
    want = ref_ops.bf16_bits_to_f32(ref_ops.gemm_fp8_blockscaled(u8(aq), sa.numpy(), u8(bq), sb.numpy()))
    return out.float().cpu().numpy(), want


def test_fp8_small_integers_exact(cuda_device):
    """Small integer operands and power-of-two scales: every partial sum is exact, so the result
    must equal the oracle bit for bit — this pins the operand layout (swizzle, descriptors, K order)."""
    from tilebench_b200.benchmarks.operators.gemm_fp8_blockscaled import impl_cuda
    g = torch.Generator().manual_seed(0)
    M, N, K = 128, 128, 256
    a = torch.randint(-3, 4, (M, K), generator=g).float()
    b = torch.randint(-3, 4, (N, K), generator=g).float()
    aq, bq = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
    sa = torch.tensor([0.5, 2.0]).repeat(M, 1)
    sb = torch.tensor([[4.0, 0.25]])
    native.clear_device_status()
    out = impl_cuda.run(aq.to(cuda_device), sa.to(cuda_device), bq.to(cuda_device), sb.to(cuda_device))
    torch.cuda.synchronize()
    status_clean()
    want = ref_ops.gemm_fp8_blockscaled(u8(aq), sa.numpy(), u8(bq), sb.numpy())
    got = out.cpu().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)


def test_fp8_matches_reference_fixture(cuda_device, golden_cfg):
    """Expected output = the reference's fp32 matmul operator on operands dequantised by the reference's
    block-scale multiply (tests/golden/make_golden.py); ragged m, an all-zero block in each operand,
    +-448 codes and a subnormal fp32 scale."""
    from tilebench_b200.benchmarks.operators.gemm_fp8_blockscaled import impl_cuda
    aq = torch.from_numpy(golden_cfg["f8_aq"]).view(torch.float8_e4m3fn).to(cuda_device)
    bq = torch.from_numpy(golden_cfg["f8_bq"]).view(torch.float8_e4m3fn).to(cuda_device)
    native.clear_device_status()
    out = impl_cuda.run(aq, torch.from_numpy(golden_cfg["f8_sa"]).to(cuda_device), bq, torch.from_numpy(golden_cfg["f8_sb"]).to(cuda_device))
    torch.cuda.synchronize()
    status_clean()
    np.testing.assert_allclose(out.float().cpu().numpy(), ref_ops.bf16_bits_to_f32(golden_cfg["f8_out"]), **BF16_TOL)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1024, 1024, 1024), (200, 256, 384), (1, 128, 128)])
def test_fp8_matches_oracle_n128_tiles(cuda_device, M, N, K):
    got, want = fp8_case(M, N, K, seed=M + N + K, device=cuda_device)
    np.testing.assert_allclose(got, want, **BF16_TOL)


def test_fp8_matches_oracle_n256_tiles(cuda_device):
    # 32 x 20 = 640 tiles of 128 x 256 >= 148: takes the wide-tile kernel, several tiles per CTA
    got, want = fp8_case(4096, 5120, 512, seed=21, device=cuda_device)
    np.testing.assert_allclose(got, want, **BF16_TOL)


def test_fp8_4096_cube_vs_torch_reference(cuda_device):
    from tilebench_b200.benchmarks.operators.gemm_fp8_blockscaled import impl_cuda, impl_torch
    inputs = tensors.generate_gemm_fp8_blockscaled_inputs(S=4096, device=cuda_device, seed=5)
    native.clear_device_status()
    out = impl_cuda.run(*inputs)
    torch.cuda.synchronize()
    status_clean()
    torch.testing.assert_close(out, impl_torch.run(*inputs), **BF16_TOL)
    again = impl_cuda.run(*inputs)
    assert torch.equal(out, again)                      # run-to-run deterministic


@pytest.mark.parametrize("variant", ["pair", "n256", "n128"])
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (300, 512, 1024), (1000, 1792, 512), (2048, 2048, 2048),
                                   (4096, 4096, 256), (2432, 4096, 256)])      # the last two: split last wave (68 / 8 tiles)
def test_fp8_kernel_variants_agree_bit_for_bit(cuda_device, monkeypatch, variant, M, N, K):
    # The CTA-pair kernel (one MMA across two SMs), the 128 x 256 and the 128 x 128 kernel add the same
    # scaled K-block products in the same order: their results must be identical, ragged M included.
    from tilebench_b200.benchmarks.operators.gemm_fp8_blockscaled import impl_cuda
    inputs = [t.to(cuda_device) for t in tensors.generate_gemm_fp8_blockscaled_inputs(M=M, N=N, K=K, device="cpu", seed=M + K)]
    native.clear_device_status()
    monkeypatch.delenv("TB200_FP8_VARIANT", raising=False)
    base = impl_cuda.run(*inputs)
    monkeypatch.setenv("TB200_FP8_VARIANT", variant)
    other = impl_cuda.run(*inputs)
    torch.cuda.synchronize()
    status_clean()
    assert torch.equal(base, other)


def test_fp8_rejects_bad_shapes(cuda_device):
    ext = native.load()
    a = torch.zeros(128, 192, device=cuda_device).to(torch.float8_e4m3fn)
    with pytest.raises(Exception):
        ext.gemm_fp8_blockscaled(a, torch.ones(128, 1, device=cuda_device), a, torch.ones(1, 1, device=cuda_device),
                                 torch.empty(128, 128, dtype=torch.bfloat16, device=cuda_device))


# ---------------------------------------------------------------- W4A16

@pytest.mark.parametrize("m", [1, 16, 33, 130])
def test_w4a16_matches_reference_fixture(cuda_device, golden_cfg, m):
    """Expected output = the reference's fp32 matmul operator on the activations and the weights dequantised
    by the reference's multiply (tests/golden/make_golden.py); one height per kernel family."""
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda
    group, zp = (int(v) for v in golden_cfg["w4_gz"])
    native.clear_device_status()
    out = impl_cuda.run(torch.from_numpy(golden_cfg[f"w4_m{m}_a"]).to(cuda_device), torch.from_numpy(golden_cfg["w4_wp"]).to(cuda_device),
                        torch.from_numpy(golden_cfg["w4_s"]).to(cuda_device), group, zp)
    torch.cuda.synchronize()
    status_clean()
    np.testing.assert_allclose(out.float().cpu().numpy(), golden_cfg[f"w4_m{m}_out"].astype(np.float32), **FP16_TOL)


def w4_case(M, N, K, seed, device, group=128):
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, GROUP=group, device="cpu", seed=seed)
    native.clear_device_status()
    out = impl_cuda.run(a.to(device), wp.to(device), sc.to(device), group, zp)
    torch.cuda.synchronize()
    status_clean()
    want = ref_ops.gemm_w4a16(a.numpy(), wp.numpy(), sc.numpy(), group, zp)
    return out.float().cpu().numpy(), want.astype(np.float32)


@pytest.mark.parametrize("M", [128, 16])
def test_w4a16_one_hot_rows_read_out_weight_columns_exactly(cuda_device, M):
    """Activation row i is one-hot at column k_i: the output row must be the dequantised weight
    column k_i, bit for bit — pins nibble order, group scales, operand layout and K order
    (M = 128: tensor-memory GEMM; M = 16: the streaming mma.sync kernel and its permuted K order)."""
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda
    N, K = 256, 512
    wp, sc = tensors.make_int4_group_weights(N, K, 128, seed=3)
    ks = torch.randperm(K, generator=torch.Generator().manual_seed(1))[:M]
    a = torch.zeros(M, K, dtype=torch.float16)
    a[torch.arange(M), ks] = 1.0
    native.clear_device_status()
    out = impl_cuda.run(a.to(cuda_device), wp.to(cuda_device), sc.to(cuda_device), 128, 8)
    torch.cuda.synchronize()
    status_clean()
    w = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 128, 8)          # [N, K] fp16
    want = w[:, ks.numpy()].T
    assert np.array_equal(out.cpu().numpy().view(np.uint16), np.ascontiguousarray(want).view(np.uint16))


@pytest.mark.parametrize("variant", ["ring", "stream"])
@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (2, 256, 384), (8, 1024, 4096), (9, 384, 640), (16, 1792, 4096), (5, 128, 8192),
                                   (16, 128, 4608), (12, 256, 8192)])
def test_w4a16_decode_kernels_match_oracle(cuda_device, monkeypatch, variant, M, N, K):
    """Both decode-sized kernels (TMA ring per warp; register-staged stream) against the oracle: K that is and is
    not a multiple of the ring's 256-wide box, K beyond what fits in shared memory (falls back to the stream
    kernel by itself), several units per warp (N = 1792 x 8 rows over 148 CTAs needs 13 warps)."""
    monkeypatch.setenv("TB200_GEMV_VARIANT", variant)
    got, want = w4_case(M, N, K, seed=300 + M + K, device=cuda_device)
    np.testing.assert_allclose(got, want, **FP16_TOL)


def test_w4a16_decode_ring_is_deterministic_and_exact_on_one_hot_rows(cuda_device, monkeypatch):
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda
    monkeypatch.setenv("TB200_GEMV_VARIANT", "ring")
    N, K, M = 14336, 4096, 16
    wp, sc = tensors.make_int4_group_weights(N, K, 128, seed=31)
    ks = torch.randperm(K, generator=torch.Generator().manual_seed(2))[:M]
    a = torch.zeros(M, K, dtype=torch.float16)
    a[torch.arange(M), ks] = 1.0
    native.clear_device_status()
    ad, wpd, scd = a.to(cuda_device), wp.to(cuda_device), sc.to(cuda_device)
    out = impl_cuda.run(ad, wpd, scd, 128, 8)
    again = impl_cuda.run(ad, wpd, scd, 128, 8)
    torch.cuda.synchronize()
    status_clean()
    w = ref_ops.dequant_int4_group(wp.numpy(), sc.numpy(), 128, 8)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), np.ascontiguousarray(w[:, ks.numpy()].T).view(np.uint16))
    assert torch.equal(out, again)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 24, 64, 127, 128, 129, 300])
def test_w4a16_matches_oracle_across_m(cuda_device, M):
    got, want = w4_case(M, 512, 1024, seed=40 + M, device=cuda_device)
    np.testing.assert_allclose(got, want, **FP16_TOL)


@pytest.mark.parametrize("M", [8, 24, 300])
@pytest.mark.parametrize("group", [64, 192, 256])
def test_w4a16_other_group_sizes_follow_the_workspace_query(cuda_device, M, group):
    """Groups of 64 and 192 (not multiples of 128: decode-sized m takes the tensor-memory kernel instead of the
    streaming one; 192 = three K blocks per group, the one size whose scale index needs a division) and 256, through
    impl_cuda.run, i.e. with exactly the workspace the query reports."""
    K = 1536 if group == 192 else 1024
    got, want = w4_case(M, 1024, K, seed=90 + M + group, device=cuda_device, group=group)
    np.testing.assert_allclose(got, want, **FP16_TOL)
    # the benchmark's weight shape, where the split-K choice is the interesting one
    got, want = w4_case(M, 14336, K, seed=91 + M + group, device=cuda_device, group=group)
    np.testing.assert_allclose(got, want, **FP16_TOL)


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 256, 384), (100, 128, 128), (128, 384, 256), (9, 256, 128)])
def test_w4a16_short_k_fewer_blocks_than_issuers(cuda_device, M, N, K):
    """K of only 2-6 blocks of 64: some of the MMA issuer threads get no block and must contribute zero."""
    got, want = w4_case(M, N, K, seed=70 + M + K, device=cuda_device)
    np.testing.assert_allclose(got, want, **FP16_TOL)


@pytest.mark.parametrize("M", [1, 16, 17, 40, 64, 128])
def test_w4a16_config_shapes_small_m(cuda_device, M):
    got, want = w4_case(M, 14336, 4096, seed=50 + M, device=cuda_device)
    np.testing.assert_allclose(got, want, **FP16_TOL)


def test_w4a16_config_shape_m4096_vs_torch_reference(cuda_device):
    from tilebench_b200.benchmarks.operators.gemm_w4a16 import impl_cuda, impl_torch
    inputs = tensors.generate_gemm_w4a16_inputs(4096, 4096, 14336, device=cuda_device, seed=6)
    native.clear_device_status()
    out = impl_cuda.run(*inputs)
    torch.cuda.synchronize()
    status_clean()
    torch.testing.assert_close(out, impl_torch.run(*inputs), **FP16_TOL)
    assert torch.equal(out, impl_cuda.run(*inputs))     # deterministic, split-K or not


@pytest.mark.parametrize("M,N", [(512, 10240), (300, 10240), (256, 1792), (200, 1792), (4096, 1280), (300, 640)])
def test_w4a16_tail_units_are_bit_identical(cuda_device, monkeypatch, M, N):
    """When the last wave of the persistent grid of 256-row tiles is at most half full, its tiles are cut into
    two 128-row units.  A unit adds the same K blocks in the same order, so the result must equal the uncut
    schedule bit for bit (TB200_W4_TAIL=0), ragged M and the non-TMA-store epilogue (odd column offset) included."""
    ext = native.load()
    K = 512
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, device="cpu", seed=M + N)
    ad, wpd, scd = a.to(cuda_device), wp.to(cuda_device), sc.to(cuda_device)
    native.clear_device_status()
    res = {}
    for knob in ("1", "0"):
        monkeypatch.setenv("TB200_W4_TAIL", knob)
        out = torch.full((M, N + 8), 3.0, dtype=torch.float16, device=cuda_device)
        ext.gemm_w4a16(ad, wpd, scd, out, group, zp, 0, None)
        odd = torch.full((M, N + 8), 3.0, dtype=torch.float16, device=cuda_device)
        ext.gemm_w4a16(ad, wpd, scd, odd, group, zp, 3, None)        # 6-byte column offset: stores from registers
        torch.cuda.synchronize()
        res[knob] = (out, odd)
    status_clean()
    assert torch.equal(res["1"][0], res["0"][0]) and torch.equal(res["1"][1], res["0"][1])
    assert torch.equal(res["1"][0][:, :N], res["1"][1][:, 3:N + 3])
    assert torch.all(res["1"][0][:, N:] == 3.0) and torch.all(res["1"][1][:, :3] == 3.0)
    if N <= 1792:
        want = ref_ops.gemm_w4a16(a.numpy(), wp.numpy(), sc.numpy(), group, zp).astype(np.float32)
        np.testing.assert_allclose(res["1"][0][:, :N].float().cpu().numpy(), want, **FP16_TOL)


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (300, 1024, 2560), (1000, 512, 10240), (4096, 4096, 14336),
                                   (700, 512, 19200)])
def test_w4a16_cta_pair_kernel_is_bit_identical(cuda_device, monkeypatch, M, K, N):
    """The opt-in CTA-pair form of the 256-row tile (TB200_W4_VARIANT=pair: cta_group::2 MMAs over two SMs, each CTA
    converting its own 128 weight rows) adds the same K blocks in the same order as the single-CTA kernel, so the
    results must be equal bit for bit — ragged M, half-height tail units (10240 / 256 = 40 and 19200 / 256 = 75 tiles
    against 74 pairs) and repeated calls included."""
    ext = native.load()
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, device=cuda_device, seed=M + K + N)
    native.clear_device_status()
    res = {}
    for variant in ("single", "pair"):
        monkeypatch.setenv("TB200_W4_VARIANT", variant)
        out = torch.full((M, N + 8), 3.0, dtype=torch.float16, device=cuda_device)
        ext.gemm_w4a16(a, wp, sc, out, group, zp, 0, None)
        torch.cuda.synchronize()
        res[variant] = out
    for _ in range(5):                                     # still "pair"
        again = torch.full((M, N + 8), 3.0, dtype=torch.float16, device=cuda_device)
        ext.gemm_w4a16(a, wp, sc, again, group, zp, 0, None)
        assert torch.equal(again, res["pair"])
    status_clean()
    assert torch.equal(res["single"], res["pair"])
    assert torch.all(res["pair"][:, N:] == 3.0)


@pytest.mark.parametrize("M,K,N,reps", [(4096, 8192, 57344, 60), (128, 4096, 14336, 300), (40, 4096, 14336, 300), (300, 4096, 14336, 200)])
def test_w4a16_repeated_calls_are_bit_identical(cuda_device, M, K, N, reps):
    """The kernels are deterministic by construction (fixed summation order), so any run-to-run difference is a
    race.  Repeats the largest benchmark shapes many times: a packed-weight stage released to the TMA refill
    before the loads from it had completed once showed up exactly like this — single output columns differing in
    about one call of twenty — and in nothing else."""
    ext = native.load()
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, device=cuda_device, seed=77)
    out = torch.empty(M, N, dtype=torch.float16, device=cuda_device)
    native.clear_device_status()
    ext.gemm_w4a16(a, wp, sc, out, group, zp, 0, None)
    first = out.clone()
    scratch = torch.empty(32 << 20, dtype=torch.float32, device=cuda_device)
    for r in range(reps):
        if r % 3 == 0:
            scratch.fill_(float(r))                      # vary what the caches hold, to shake the timing
        out.fill_(float("nan"))
        ext.gemm_w4a16(a, wp, sc, out, group, zp, 0, None)
        assert torch.equal(out, first), f"call {r} differs from the first in {int((out != first).sum())} elements"
    status_clean()


@pytest.mark.parametrize("M", [64, 300])
def test_w4a16_column_offset_writes_only_its_slice(cuda_device, M):
    """N-partition building block: two calls with col_offset fill one [M, N] buffer; guard columns stay.
    M = 300 takes the 256-row tiles whose epilogue goes through shared memory and TMA stores (clipped at M)."""
    ext = native.load()
    N, K = 512, 512
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(M, K, N, device="cpu", seed=8)
    ad, wpd, scd = a.to(cuda_device), wp.to(cuda_device), sc.to(cuda_device)
    out = torch.full((M, N + 64), 7.0, dtype=torch.float16, device=cuda_device)
    half = N // 2
    for r in range(2):
        n_local = half
        wsb = ext.gemm_w4a16_workspace_bytes(M, n_local, K)
        ws = torch.empty(max(wsb // 4, 1), dtype=torch.float32, device=cuda_device)
        ext.gemm_w4a16(ad, wpd[r * half:(r + 1) * half].contiguous(), scd[r * half:(r + 1) * half].contiguous(),
                       out, group, zp, r * half, ws)
    torch.cuda.synchronize()
    want = ref_ops.gemm_w4a16(a.numpy(), wp.numpy(), sc.numpy(), group, zp).astype(np.float32)
    np.testing.assert_allclose(out[:, :N].float().cpu().numpy(), want, **FP16_TOL)
    assert torch.all(out[:, N:] == 7.0)


def test_w4a16_workspace_too_small_is_an_error(cuda_device):
    ext = native.load()
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(24, 4096, 4096, device=cuda_device, seed=9)
    assert ext.gemm_w4a16_workspace_bytes(24, 4096, 4096) > 0        # narrow weight: the split-K path
    assert ext.gemm_w4a16_workspace_bytes(24, 14336, 4096) == 0      # wide weight: one wave of 128-row tiles, no scratch
    out = torch.empty(24, 4096, dtype=torch.float16, device=cuda_device)
    with pytest.raises(ValueError):
        ext.gemm_w4a16(a, wp, sc, out, group, zp, 0, None)


# ---------------------------------------------------------------- int8 x packed 2-bit (reference operator matmul_int8)

def i8_run(a, b, device):
    from tilebench_b200.benchmarks.operators.matmul_int8 import impl_cuda
    native.clear_device_status()
    out = impl_cuda.run(a.to(device), b.to(device))
    torch.cuda.synchronize()
    status_clean()
    return out.cpu().numpy()


@pytest.mark.parametrize("N", [128, 256, 512, 4864])      # 4864: enough 256-wide tiles for the wide kernel
def test_int8_one_hot_rows_read_out_every_unpacked_weight(cuda_device, N):
    # a = one-hot rows: out[r, :] is row k_r of the unpacked weight matrix, so every (k, n) position of the
    # operand layout (field plane, swizzle, 128-column block, sub-step) is pinned individually.
    K = 512
    g = torch.Generator().manual_seed(N)
    b = torch.randint(0, 256, (K // 4, N), dtype=torch.uint8, generator=g)
    a = torch.zeros(K, K, dtype=torch.int8)
    a[torch.arange(K), torch.arange(K)] = 1
    got = i8_run(a, b, cuda_device)
    want = ref_ops.matmul_int8_packed2bit(a.numpy(), b.numpy())
    assert np.array_equal(got, want)


@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (100, 256, 512), (128, 384, 1024), (300, 2048, 2048), (2048, 2048, 1024)])
def test_int8_matches_oracle_exactly(cuda_device, M, N, K):
    a, b = tensors.generate_matmul_int8_inputs(M, N, K, device="cpu", seed=M + N + K)
    got = i8_run(a, b, cuda_device)
    assert np.array_equal(got, ref_ops.matmul_int8_packed2bit(a.numpy(), b.numpy()))


def test_int8_extreme_values_and_longest_k(cuda_device):
    # a = -128 / 127 everywhere with weights 2 / -1: the largest magnitudes the format allows, K = 20480
    from tilebench_b200.benchmarks.operators.matmul_int8 import impl_torch
    M, N, K = 256, 256, 20480
    a = torch.full((M, K), 127, dtype=torch.int8)
    a[::2] = -128
    b = torch.full((K // 4, N), 0xFF, dtype=torch.uint8)      # every field 3 -> weight 2
    b[:, ::2] = 0x00                                          # every field 0 -> weight -1
    got = i8_run(a, b, cuda_device)
    want = np.empty((M, N), dtype=np.int64)
    want[0::2, 0::2] = -128 * -1 * K
    want[0::2, 1::2] = -128 * 2 * K
    want[1::2, 0::2] = 127 * -1 * K
    want[1::2, 1::2] = 127 * 2 * K
    assert np.array_equal(got.astype(np.int64), want)
    a2, b2 = tensors.generate_matmul_int8_inputs(2048, 2048, K, device=cuda_device, seed=3)
    out = impl_cuda_i8(a2, b2)
    assert torch.equal(out, impl_torch.run(a2, b2))


def impl_cuda_i8(a, b):
    from tilebench_b200.benchmarks.operators.matmul_int8 import impl_cuda
    native.clear_device_status()
    out = impl_cuda.run(a, b)
    torch.cuda.synchronize()
    status_clean()
    return out


def test_int8_rejects_unsupported_shapes(cuda_device):
    ext = native.load()
    a = torch.zeros(16, 200, dtype=torch.int8, device=cuda_device)
    b = torch.zeros(50, 128, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(Exception):
        ext.matmul_int8_packed2(a, b, torch.empty(16, 128, dtype=torch.int32, device=cuda_device))


# ---------------------------------------------------------------- plain GEMM (reference operator matmul_fp32_fp16_fp8)

def plain_run(a, b):
    from tilebench_b200.benchmarks.operators.matmul_fp32_fp16_fp8 import impl_cuda
    native.clear_device_status()
    out = impl_cuda.run(a, b)
    torch.cuda.synchronize()
    status_clean()
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float8_e4m3fn])
@pytest.mark.parametrize("N", [128, 256, 4864])          # 4864: enough 256-wide tiles for the wide kernel
def test_plain_one_hot_rows_read_out_b_exactly(cuda_device, dtype, N):
    # a = identity: out must equal b bit for bit (every value of b is exact in tf32 / fp16 / e4m3), which pins
    # the MN-major operand layout of b — column block, swizzle, K step — element by element.
    K = 512
    g = torch.Generator().manual_seed(N)
    b = torch.randint(-8, 9, (K, N), generator=g).to(torch.float32).to(dtype).to(cuda_device)
    a = torch.eye(K, dtype=torch.float32).to(dtype).to(cuda_device)
    out = plain_run(a, b)
    assert torch.equal(out.view(torch.uint8), b.view(torch.uint8))


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (100, 256, 512), (300, 384, 1024), (2048, 2048, 1024)])
def test_plain_fp16_matches_oracle(cuda_device, M, N, K):
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=torch.float16, device="cpu", seed=M + N + K)
    got = plain_run(a.to(cuda_device), b.to(cuda_device)).cpu().numpy().astype(np.float32)
    want = ref_ops.matmul_plain(a.numpy(), b.numpy(), "fp16").astype(np.float32)
    np.testing.assert_allclose(got, want, atol=1e-3, rtol=1e-3)       # fp16 tolerance of the reference's verifier


@pytest.mark.parametrize("M,N,K", [(1, 128, 32), (100, 256, 512), (300, 384, 1024), (2048, 2048, 1024)])
def test_plain_fp32_is_a_tf32_gemm(cuda_device, M, N, K):
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=torch.float32, device="cpu", seed=M + N + K)
    got = plain_run(a.to(cuda_device), b.to(cuda_device)).cpu().numpy()
    want = ref_ops.matmul_plain(a.numpy(), b.numpy(), "tf32")         # operands with the low 13 mantissa bits dropped
    np.testing.assert_allclose(got, want, atol=1e-4, rtol=1e-4)
    # and within TF32's input precision (2**-10 relative per operand) of the true fp32 product
    np.testing.assert_allclose(got, ref_ops.matmul_plain(a.numpy(), b.numpy(), "fp32"), atol=5e-3, rtol=5e-3)


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (100, 256, 512), (300, 384, 1024), (2048, 2048, 2048)])
def test_plain_fp8_matches_oracle_up_to_rounding_ties(cuda_device, M, N, K):
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=torch.float8_e4m3fn, device="cpu", seed=M + N + K)
    got = plain_run(a.to(cuda_device), b.to(cuda_device)).cpu().view(torch.uint8).numpy()
    want = ref_ops.matmul_plain(a.view(torch.uint8).numpy(), b.view(torch.uint8).numpy(), "fp8")
    # Products of e4m3 values are exact in fp32; only the order of the fp32 additions differs, which can move
    # a sum across a bf16 / e4m3 rounding boundary: such elements differ by one e4m3 step and are rare.
    diff = got != want
    assert diff.mean() < 2e-3
    step = np.abs(got[diff].astype(np.int16) - want[diff].astype(np.int16))
    assert step.size == 0 or step.max() == 1


def test_plain_fp8_overflow_becomes_nan_like_torch(cuda_device):
    # 28 * 16 = 448 (largest finite), 30 * 16 = 480 and -30 * 16 overflow: PyTorch's cast gives NaN, not 448
    K, N = 128, 128
    a = torch.zeros(4, K)
    a[0, 0], a[1, 0], a[2, 0], a[3, 0] = 28.0, 30.0, -30.0, 1.0
    b = torch.zeros(K, N)
    b[0, :] = 16.0
    out = plain_run(a.to(torch.float8_e4m3fn).to(cuda_device), b.to(torch.float8_e4m3fn).to(cuda_device)).float().cpu()
    assert torch.all(out[0] == 448.0) and torch.all(out[3] == 16.0)
    assert torch.isnan(out[1]).all() and torch.isnan(out[2]).all()


@pytest.mark.parametrize("dtype,K", [(torch.float16, 4096), (torch.float32, 2048), (torch.float8_e4m3fn, 8192)])
def test_plain_reference_shape_vs_torch_reference(cuda_device, dtype, K):
    from tilebench_b200.benchmarks.operators.matmul_fp32_fp16_fp8 import impl_torch
    from tilebench_b200.core import verifier
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(4096, 4096, K, dtype=dtype, device=cuda_device, seed=K)
    out = plain_run(a, b)
    ok, err = verifier.verify(out, impl_torch.run(a, b), atol=5.0, rtol=0.1)     # the reference's own tolerance
    assert ok, err
    tight = {torch.float16: 2e-3, torch.float32: 5e-3, torch.float8_e4m3fn: 0.13}[dtype]
    torch.testing.assert_close(out.float(), impl_torch.run(a, b).float(), atol=tight, rtol=tight)
    assert torch.equal(out.view(torch.uint8), plain_run(a, b).view(torch.uint8))    # deterministic


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float8_e4m3fn])
@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (300, 512, 1024), (1000, 1792, 512), (2048, 2048, 2048)])
def test_plain_pair_and_single_cta_kernels_agree_bit_for_bit(cuda_device, monkeypatch, dtype, M, N, K):
    # the CTA-pair kernel (one MMA across two SMs) adds the same products in the same order as the single-CTA one
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=dtype, device=cuda_device, seed=M + K)
    monkeypatch.setenv("TB200_PLAIN_VARIANT", "single")
    single = plain_run(a, b)
    monkeypatch.setenv("TB200_PLAIN_VARIANT", "pair")
    pair = plain_run(a, b)
    assert torch.equal(single.view(torch.uint8), pair.view(torch.uint8))


def test_plain_rejects_unsupported(cuda_device):
    from tilebench_b200.benchmarks.operators.matmul_fp32_fp16_fp8 import impl_cuda
    a = torch.zeros(16, 100, dtype=torch.float16, device=cuda_device)
    with pytest.raises(Exception):
        impl_cuda.run(a, torch.zeros(100, 128, dtype=torch.float16, device=cuda_device))
    with pytest.raises(NotImplementedError):
        impl_cuda.run(a.to(torch.float64), torch.zeros(100, 128, dtype=torch.float64, device=cuda_device))


@pytest.mark.parametrize("M,N,K", [(100, 256, 512), (2048, 2048, 1024)])
def test_plain_bf16_matches_fp32_reference(cuda_device, M, N, K):
    a, b = tensors.generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=torch.bfloat16, device="cpu", seed=M + K)
    got = plain_run(a.to(cuda_device), b.to(cuda_device)).float().cpu().numpy()
    want = ref_ops.bf16_bits_to_f32(ref_ops.f32_to_bf16_bits(ref_ops.matmul_f32(a.float().numpy(), b.float().numpy())))
    np.testing.assert_allclose(got, want, atol=1e-2, rtol=1.6e-2)          # bf16 tolerance of the reference's verifier
    eye = torch.eye(512, dtype=torch.bfloat16, device=cuda_device)
    bb = torch.randint(-8, 9, (512, 256), dtype=torch.int32).to(torch.bfloat16).to(cuda_device)
    assert torch.equal(plain_run(eye, bb), bb)


# ---------------------------------------------------------------- run-to-run identity of every tensor-core kernel

@pytest.mark.parametrize("which", ["fp8_4096", "fp8_ragged_pair", "int8_k20480", "plain_f16", "plain_tf32", "plain_e4m3"])
def test_gemm_kernels_repeated_calls_are_bit_identical(cuda_device, monkeypatch, which):
    """Every GEMM here sums in a fixed order, so identical calls must give identical bits; a difference is a race
    (a stage or accumulator handed over too early).  Many repeats with the caches disturbed in between."""
    ext = native.load()
    g = torch.Generator(device=cuda_device).manual_seed(5)
    if which.startswith("fp8"):
        if which == "fp8_ragged_pair":
            monkeypatch.setenv("TB200_FP8_VARIANT", "pair")
            M, N, K, reps = 3000, 4096, 2048, 100
        else:
            M, N, K, reps = 4096, 4096, 4096, 100
        aq, sa = tensors.quantize_fp8_blockwise(torch.randn(M, K, device=cuda_device, generator=g), 1, 128)
        bq, sb = tensors.quantize_fp8_blockwise(torch.randn(N, K, device=cuda_device, generator=g), 128, 128)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=cuda_device)
        call = lambda: ext.gemm_fp8_blockscaled(aq, sa, bq, sb, out)
    elif which == "int8_k20480":
        M, N, K, reps = 2048, 2048, 20480, 100
        a = torch.randint(-64, 65, (M, K), dtype=torch.int8, device=cuda_device, generator=g)
        b = torch.randint(0, 256, (K // 4, N), dtype=torch.uint8, device=cuda_device, generator=g)
        out = torch.empty(M, N, dtype=torch.int32, device=cuda_device)
        call = lambda: ext.matmul_int8_packed2(a, b, out)
    else:
        dt = {"plain_f16": torch.float16, "plain_tf32": torch.float32, "plain_e4m3": torch.float8_e4m3fn}[which]
        M, N, K, reps = 4096, 4096, 4096, 60
        a = (torch.randn(M, K, device=cuda_device, generator=g) * K ** -0.5).to(dt)
        b = (torch.randn(K, N, device=cuda_device, generator=g) * K ** -0.5).to(dt)
        out = torch.empty(M, N, dtype=dt, device=cuda_device)
        call = lambda: ext.matmul_plain(a, b, out)
    native.clear_device_status()
    call()
    first = out.clone().view(torch.uint8)
    scratch = torch.empty(32 << 20, dtype=torch.float32, device=cuda_device)
    for r in range(reps):
        if r % 3 == 0:
            scratch.fill_(float(r))
        out.view(torch.uint8).fill_(0xAA)
        call()
        assert torch.equal(out.view(torch.uint8), first), f"{which}: call {r} differs from the first"
    status_clean()
