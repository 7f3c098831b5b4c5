"""CPU oracle for the quantized-inference path — TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module, and
only as the checker or the timed CPU baseline.  Nothing under tilebench_b200/ imports it.

Plain numpy restatements, one function per operator, each citing the reference file it follows
(paths inside the TileBench project).  16-bit float results are produced by an explicit
round-to-nearest-even from fp32, so the integer -> float paths are bit-exact statements:
  * fp16  via numpy's float32 -> float16 cast (IEEE RN-even, subnormals kept)
  * bf16  as uint16 bit patterns via `f32_to_bf16_bits`
  * e4m3  decoded from the format definition by `e4m3_table`

Pinning — every function is checked against outputs of REFERENCE code, generated from a reference
checkout by tests/golden/make_golden.py and committed as fixtures:
  * dequantize_rowwise, weight_dequant, the 2-bit matmul_int8 and the fp16/fp32 matmul: outputs of the
    reference's own impl_torch.run (tests/golden/reference_ops.npz), plus the worked examples in
    tilebench/problems/*_current.md.
  * dequant_int4_group, dequant_int8_channel, gemm_w4a16, gemm_fp8_blockscaled, quantize_int4_group have
    no operator of their own in the reference (it has no int4, W4A16 or block-scaled FP8 operator), so
    their fixtures (tests/golden/baseline_configs.npz) are computed THROUGH the reference operators that
    carry their arithmetic: weight_dequant.impl_torch.run with TILE_SIZE = 1 is the elementwise fp32
    multiply of both dequant formulas (and, with TILE_SIZE = 128, the block scaling of the FP8 weights),
    matmul_fp32_fp16_fp8.impl_torch.run on fp32 tensors is the "fp32 matmul of the dequantised operands"
    the GEMM configurations name, quantize_global.impl_torch.run is the fp16 cast of the quantiser's
    scale.  Around them only nibble extraction, broadcasting and the final cast to the output type are
    added.  The dequant fixtures are matched bit for bit; the GEMM fixtures within the operator's
    tolerance (two fp32 GEMMs with different summation orders) with over 98 % of the outputs identical.
  * Beside the fixtures: hand-computable known answers (all 16 nibbles, all 256 int8 / e4m3 codes,
    identity scales, one-hot activations).
  * The e4m3 row of matmul_plain follows torch._scaled_mm, which does not run on CPU: no reference
    fixture; its pieces (decode table, encoder) are checked against PyTorch's casts on dense sweeps.
"""
from __future__ import annotations

import numpy as np


# ---- number formats ---------------------------------------------------------------------------

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + bias) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def e4m3_table() -> np.ndarray:
    """All 256 float8_e4m3fn codes as float32: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no
    infinities; S.1111.111 is NaN; exponent 0 is subnormal (mantissa / 8 * 2^-6)."""
    t = np.empty(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = sign * (m / 8.0) * 2.0 ** -6
        else:
            v = sign * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[code] = v
    return t


_E4M3 = e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return _E4M3[np.ascontiguousarray(codes, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> float8_e4m3fn codes (uint8), round to nearest, ties to the even mantissa; magnitudes
    that round past 448 (above 464, or exactly 464 rounding to the odd neighbour) and NaN become NaN
    (S.1111.111) — the behaviour of PyTorch's cast, which the reference's fp8 path ends in
    (tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:26)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    pos = _E4M3[:127].astype(np.float64)                          # codes 0..126: 0 .. 448, increasing
    hi = np.clip(np.searchsorted(pos, mag, side="left"), 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    d_lo, d_hi = mag - pos[lo], pos[hi] - mag
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    # beyond the last finite value: the next step of the grid would be 480; the tie at 464 goes to 448 (even)
    code = np.where(mag > 464.0, np.uint8(0x7F), code)
    code = np.where(np.isnan(x), np.uint8(0x7F), code)
    sign = (x.view(np.uint32) >> np.uint32(24)).astype(np.uint8) & np.uint8(0x80)
    return (code | sign).astype(np.uint8)


# ---- dequantisation ---------------------------------------------------------------------------

def unpack_int4(wp: np.ndarray) -> np.ndarray:
    """uint8 [N, K/2] -> int32 [N, K]: low nibble = even k, high nibble = odd k."""
    wp = np.ascontiguousarray(wp, dtype=np.uint8)
    q = np.empty((wp.shape[0], wp.shape[1] * 2), dtype=np.int32)
    q[:, 0::2] = wp & 0xF
    q[:, 1::2] = wp >> 4
    return q


def dequant_int4_group(wp, scales_f16, group: int = 128, zp: int = 8) -> np.ndarray:
    """fp16((q - zp) * float(scale[r, c // group])).  New operator; written in the form of the
    reference's block-scale multiply (tilebench/benchmarks/operators/weight_dequant/impl_torch.py:4-8)
    with the fp32-then-cast precision rule of its contract
    (tilebench/llm/v2/contracts/data/weight_dequant/contract.md:60-67)."""
    q = unpack_int4(wp)
    s = np.repeat(np.asarray(scales_f16, dtype=np.float16).astype(np.float32), group, axis=1)
    with np.errstate(over="ignore"):                   # products beyond 65504 round to +-inf, as IEEE says
        return ((q - zp).astype(np.float32) * s).astype(np.float16)


def quantize_int4_group(x_f32, group: int = 128, zp: int = 8):
    """fp32 [N, K] -> (packed uint8 [N, K/2], fp16 scales [N, K/group]): s = fp16(amax / 7) per group (1 where
    that rounds to zero), q = clamp(rint(x / s) + zp, 0, 15), low nibble = even k.  New operator (the
    reference's quantiser is a cast, tilebench/benchmarks/operators/quantize_global/impl_torch.py:4-5);
    the inverse of dequant_int4_group up to rounding."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    n, k = x.shape
    xg = x.reshape(n, k // group, group)
    amax = np.abs(xg).max(axis=2)
    s16 = (amax / np.float32(7.0)).astype(np.float16)
    s16 = np.where(s16.astype(np.float32) == 0.0, np.float16(1.0), s16)
    q = np.clip(np.rint(xg / s16.astype(np.float32)[:, :, None]) + np.float32(zp), 0, 15).astype(np.uint8).reshape(n, k)
    return (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8), s16


def dequant_int8_channel(w_i8, scale_f32) -> np.ndarray:
    """bf16 bits of float(w) * scale[r] (one fp32 rounding, then RN-even to bf16).  New operator in the
    form of tilebench/benchmarks/operators/dequantize_rowwise/impl_torch.py:4-7 without the 1/127."""
    prod = np.asarray(w_i8, dtype=np.int8).astype(np.float32) * np.asarray(scale_f32, dtype=np.float32)[:, None]
    return f32_to_bf16_bits(prod)


def dequantize_rowwise(x_i8, state_x_f32) -> np.ndarray:
    """fp16((state_x[r] * float(x)) * float32(1/127)) — the reference operator
    tilebench/benchmarks/operators/dequantize_rowwise/impl_torch.py:4-7: the Python scalar 1/127
    enters the fp32 tensor arithmetic as a float32, after the state*x product was rounded."""
    prod = np.asarray(state_x_f32, dtype=np.float32)[:, None] * np.asarray(x_i8, dtype=np.int8).astype(np.float32)
    return (prod * np.float32(1.0 / 127.0)).astype(np.float16)


def weight_dequant(x, s, m: int, n: int, tile: int) -> np.ndarray:
    """Y = X * S[i // T, j // T] — tilebench/benchmarks/operators/weight_dequant/impl_torch.py:4-8.
    x, s: float32 or float16 arrays, or uint16 bf16 bit patterns; the result has the same
    representation.  16-bit products are exact in fp32 and rounded once."""
    rows = np.arange(m) // tile
    cols = np.arange(n) // tile
    if x.dtype == np.uint16:  # bf16 bits
        scale = bf16_bits_to_f32(s)[rows[:, None], cols[None, :]]
        return f32_to_bf16_bits(bf16_bits_to_f32(x).reshape(m, n) * scale)
    scale = np.asarray(s)[rows[:, None], cols[None, :]].astype(np.float32)
    return (np.asarray(x).reshape(m, n).astype(np.float32) * scale).astype(x.dtype)


# ---- GEMMs ------------------------------------------------------------------------------------

def matmul_f32(a, b) -> np.ndarray:
    """fp32 GEMM (tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:27 for fp32)."""
    return np.matmul(np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32))


def tf32_truncate(x: np.ndarray) -> np.ndarray:
    """fp32 with the low 13 mantissa bits cleared: the part of an fp32 operand a TF32 tensor-core MMA reads."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


def matmul_plain(a, b, kind: str) -> np.ndarray:
    """out = a[M, K] @ b[K, N] as tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27
    computes it, per input type:
      "fp16": fp16 operands, fp32 accumulation, one rounding to fp16 (torch.matmul of halves)
      "fp32": plain fp32 GEMM (what the reference gives on CPU)
      "tf32": fp32 operands read as TF32 (allow_tf32 is set by the reference module; its GPU result)
      "fp8" : e4m3 codes in, unit scales, fp32 accumulation, rounded to bf16 and then to e4m3 codes
              (torch._scaled_mm(..., out_dtype=bfloat16).to(float8_e4m3fn); does not run on CPU)"""
    if kind == "fp16":
        return matmul_f32(np.asarray(a, dtype=np.float16), np.asarray(b, dtype=np.float16)).astype(np.float16)
    if kind == "fp32":
        return matmul_f32(a, b)
    if kind == "tf32":
        return matmul_f32(tf32_truncate(a), tf32_truncate(b))
    if kind == "fp8":
        acc = matmul_f32(e4m3_decode(a), e4m3_decode(b))
        return e4m3_encode(bf16_bits_to_f32(f32_to_bf16_bits(acc)))
    raise ValueError(f"unknown kind {kind!r}")


def gemm_w4a16(a_f16, wp, scales_f16, group: int = 128, zp: int = 8) -> np.ndarray:
    """fp16(A_f32 @ float(W_f16)^T) with W_f16 = dequant_int4_group(...): weights are rounded to fp16
    before the product (that is what the kernel feeds the tensor core), accumulation in fp32.
    New operator; packed-weight GEMM in the form of
    tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19 (unpack, then an fp32 matmul)."""
    w = dequant_int4_group(wp, scales_f16, group, zp).astype(np.float32)
    return matmul_f32(np.asarray(a_f16, dtype=np.float16).astype(np.float32), w.T).astype(np.float16)


def gemm_fp8_blockscaled(aq_codes, sa, bq_codes, sb, block: int = 128) -> np.ndarray:
    """bf16 bits of (Aq * sa_block) @ (Bq * sb_block)^T, operands dequantised to fp32 first.
    New operator; the reference's fp8 GEMM (unit scales through torch._scaled_mm,
    tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-26) does not run on CPU."""
    a = e4m3_decode(aq_codes) * np.repeat(np.asarray(sa, dtype=np.float32), block, axis=1)
    b = e4m3_decode(bq_codes) * np.repeat(np.repeat(np.asarray(sb, dtype=np.float32), block, axis=0), block, axis=1)
    return f32_to_bf16_bits(matmul_f32(a, b.T))


def matmul_int8_packed2bit(a_i8, b_u8) -> np.ndarray:
    """int32 GEMM with 2-bit packed B — tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19:
    field i of byte b[kb, n] decodes to ((b >> 2i) & 3) - 1 and lands at row i*K_b + kb."""
    a = np.asarray(a_i8, dtype=np.int8).astype(np.int64)
    b = np.asarray(b_u8, dtype=np.uint8).astype(np.int64)
    kb = b.shape[0]
    unpacked = np.empty((4 * kb, b.shape[1]), dtype=np.int64)
    for i in range(4):
        unpacked[i * kb:(i + 1) * kb] = ((b >> (2 * i)) & 3) - 1
    return (a @ unpacked).astype(np.int32)
