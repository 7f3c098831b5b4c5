"""Seeded input generators and the case grid.

The reference generates unseeded tensors on the device (tilebench/data/tensors.py:11, :179-184,
:416-448, :492-499).  Parity on identical inputs needs a seed, so every generator here draws on
the CPU from an explicit torch.Generator and then moves the tensors to `device`; the same CPU
tensors feed the oracle.  `expand_cases` / `infer_problem_size` / `GENERATORS` keep the
reference's surface (tensors.py:26-39, :560-627, :630-785).
"""
from __future__ import annotations

import math
from itertools import product

import torch

DEFAULT_DEVICE = "cuda" if torch.cuda.is_available() else "cpu"
#: Base seed; a case's seed is SEED0 + 1000 * operator index + case index unless given.
SEED0 = 20261125

FP8_MAX = 448.0


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


class CaseGridError(ValueError):
    """A case_grid / test_cases block that cannot be expanded."""


def _axis_values(spec, axis: str) -> list:
    """Candidate values of one grid axis.  An axis is written either as a plain list or as
    `{expr: "<python>"}`, a Python expression yielding the list (the configs shipped with the package use it for
    arithmetic progressions such as `[1024 * i for i in range(1, 21)]`)."""
    if isinstance(spec, dict) and "expr" in spec:
        spec = eval(spec["expr"], {"__builtins__": __builtins__}, {})  # noqa: S307 - configs are package files, not user input
        origin = "expr of axis"
    else:
        origin = "axis"
    if isinstance(spec, (list, tuple)) and len(spec) > 0:
        return list(spec)
    raise CaseGridError(f"case_grid: {origin} '{axis}' needs a non-empty list of candidates, got {spec!r}")


def _expand_case_grid(case_grid, case_defaults=None):
    """Cartesian product of the grid axes, in the order the config lists them (last axis fastest), each case
    laid over a copy of `case_defaults`."""
    if not isinstance(case_grid, dict) or not case_grid:
        raise CaseGridError("case_grid has to map at least one parameter name to its candidates")
    axes = [(axis, _axis_values(spec, axis)) for axis, spec in case_grid.items()]
    names = [axis for axis, _ in axes]
    base = dict(case_defaults or {})
    return [{**base, **dict(zip(names, point))} for point in product(*(vals for _, vals in axes))]


# kept under the reference's name for callers that expand a single axis
_normalize_sequence = _axis_values


def expand_cases(operator_name, config):
    """The operator's case list: `test_cases` verbatim when given, else `case_grid` expanded over `case_defaults`."""
    explicit = config.get("test_cases")
    if explicit:
        return list(explicit)
    grid = config.get("case_grid")
    if grid is not None:
        return _expand_case_grid(grid, config.get("case_defaults"))
    raise CaseGridError(f"operator '{operator_name}': the config defines neither test_cases nor case_grid")


# ---- quantised-weight inputs ------------------------------------------------------------------

def make_int4_group_weights(N, K, GROUP=128, seed=SEED0):
    """Packed uint8 [N, K/2] (each nibble uniform 0..15, low nibble = even k) and fp16 scales
    [N, K/GROUP] drawn as |N(0,1)| * 0.01 + 1e-3."""
    g = _gen(seed)
    wp = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    scales = (torch.randn(N, K // GROUP, generator=g).abs() * 0.01 + 1e-3).to(torch.float16)
    return wp, scales


def generate_dequant_int4_group_inputs(N, K, GROUP=128, ZP=8, dtype=torch.float16, device=DEFAULT_DEVICE,
                                       seed=SEED0, **kwargs):
    wp, scales = make_int4_group_weights(N, K, GROUP, seed)
    return (wp.to(device), scales.to(device), GROUP, ZP)


def generate_dequant_int8_channel_inputs(rows, cols, dtype=torch.bfloat16, device=DEFAULT_DEVICE,
                                         seed=SEED0 + 1000, **kwargs):
    g = _gen(seed)
    w = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, generator=g)
    scale = torch.randn(rows, generator=g).abs() * 0.02 + 1e-4
    return (w.to(device), scale.to(device))


def generate_gemm_w4a16_inputs(M, K, N, GROUP=128, ZP=8, dtype=torch.float16, device=DEFAULT_DEVICE,
                               seed=SEED0 + 2000, **kwargs):
    g = _gen(seed)
    a = torch.randn(M, K, generator=g).to(torch.float16)
    wp, scales = make_int4_group_weights(N, K, GROUP, seed + 1)
    return (a.to(device), wp.to(device), scales.to(device), GROUP, ZP)


def quantize_fp8_blockwise(x: torch.Tensor, block_rows: int, block_cols: int = 128):
    """e4m3 quantisation with one fp32 scale = amax/448 per [block_rows x block_cols] block
    (scale 1 for an all-zero block).  Returns (q, scales[rows/block_rows, cols/block_cols])."""
    R, C = x.shape
    xb = x.reshape(R // block_rows, block_rows, C // block_cols, block_cols)
    amax = xb.abs().amax(dim=(1, 3))
    # tensor / tensor: a true IEEE division on every device (tensor / python-scalar becomes a multiplication
    # by the rounded reciprocal on CUDA, which differs from amax / 448 in the last bit for most blocks)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, FP8_MAX), torch.ones_like(amax)).to(torch.float32)
    q = (xb / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(R, C).to(torch.float8_e4m3fn)
    return q, scale


def generate_gemm_fp8_blockscaled_inputs(S=None, BLOCK=128, M=None, N=None, K=None, dtype=torch.float8_e4m3fn,
                                         device=DEFAULT_DEVICE, seed=SEED0 + 3000, **kwargs):
    M = M or S
    N = N or S
    K = K or S
    g = _gen(seed)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(N, K, generator=g)
    aq, sa = quantize_fp8_blockwise(a, 1, BLOCK)
    bq, sb = quantize_fp8_blockwise(b, BLOCK, BLOCK)
    return (aq.to(device), sa.to(device), bq.to(device), sb.to(device))


def generate_gemm_w4a16_npart_inputs(M, K, N, WORLD=1, GATHER=1, GROUP=128, ZP=8, dtype=torch.float16,
                                     device=DEFAULT_DEVICE, seed=SEED0 + 4000, **kwargs):
    a, wp, scales, group, zp = generate_gemm_w4a16_inputs(M, K, N, GROUP, ZP, device=device, seed=seed)
    return (a, wp, scales, group, zp, WORLD, GATHER)


def quantize_int4_groupwise(x: torch.Tensor, group: int = 128, zp: int = 8):
    """int4 group quantisation: s = fp16(amax / 7) per group (1 where that rounds to zero),
    q = clamp(round(x / s) + zp, 0, 15), two values per byte with the even k in the low nibble.
    Returns (wp uint8 [N, K/2], scales fp16 [N, K/group])."""
    n, k = x.shape
    xg = x.reshape(n, k // group, group).to(torch.float32)
    amax = xg.abs().amax(dim=2)
    s16 = (amax / torch.full_like(amax, 7.0)).to(torch.float16)          # tensor / tensor: a true IEEE division
    s16 = torch.where(s16.float() == 0, torch.ones_like(s16), s16)
    q = (torch.round(xg / s16.float()[:, :, None]) + float(zp)).clamp(0, 15).to(torch.uint8).reshape(n, k)
    return q[:, 0::2] | (q[:, 1::2] << 4), s16


def generate_quantize_int4_group_inputs(N, K, GROUP=128, ZP=8, dtype=torch.float32, device=DEFAULT_DEVICE,
                                        seed=SEED0 + 9000, **kwargs):
    x = torch.randn(N, K, generator=_gen(seed)) * 0.05
    return (x.to(device), int(GROUP), int(ZP))


def generate_quantize_fp8_block_inputs(S, BLOCK_ROWS=1, dtype=torch.float32, device=DEFAULT_DEVICE,
                                       seed=SEED0 + 7000, **kwargs):
    x = torch.randn(S, S, generator=_gen(seed))
    return (x.to(device), int(BLOCK_ROWS))


# ---- the reference's own operators (seeded versions of tensors.py:179-184 and :492-499) -------

def generate_dequantize_rowwise_inputs(rows, cols, device=DEFAULT_DEVICE, seed=SEED0 + 5000, **kwargs):
    g = _gen(seed)
    x = torch.randint(-128, 127, (rows, cols), dtype=torch.int8, generator=g)
    state_x = torch.rand(rows, dtype=torch.float32, generator=g) * 10.0
    return (x.to(device), state_x.to(device))


def generate_weight_dequant_inputs(M, TILE_SIZE, dtype, N=None, device=DEFAULT_DEVICE, seed=SEED0 + 6000, **kwargs):
    if N is None:
        N = M
    g = _gen(seed)
    X = torch.randn(M, N, generator=g).to(dtype)
    S = torch.randn(math.ceil(M / TILE_SIZE), math.ceil(N / TILE_SIZE), generator=g).to(dtype)
    return (X.to(device), S.to(device), M, N, TILE_SIZE)


def generate_matmul_int8_inputs(M, N, K, device=DEFAULT_DEVICE, seed=SEED0 + 7000, **kwargs):
    """Seeded version of tilebench/data/tensors.py:439-448: a int8 in [-64, 64], b uint8 [K/4, N] with four
    2-bit fields per byte (all 256 byte values, so every field takes every value 0..3)."""
    if K % 4:
        raise ValueError("K must be divisible by 4 (b holds four fields per byte)")
    g = _gen(seed)
    a = torch.randint(-64, 65, (M, K), dtype=torch.int8, generator=g)
    b = torch.randint(0, 256, (K // 4, N), dtype=torch.uint8, generator=g)
    return (a.to(device), b.to(device))


def generate_matmul_fp32_fp16_fp8_inputs(M, N, K, dtype=torch.float32, device=DEFAULT_DEVICE, seed=SEED0 + 8000, **kwargs):
    """Seeded version of tilebench/data/tensors.py:416-436: standard normal operands scaled by K**-0.5 so
    the output stays O(1) whatever K is; fp8 operands are made in fp32 and cast."""
    g = _gen(seed)
    scale = K ** -0.5
    a = (torch.randn(M, K, dtype=torch.float32, generator=g) * scale).to(dtype)
    b = (torch.randn(K, N, dtype=torch.float32, generator=g) * scale).to(dtype)
    return (a.to(device), b.to(device))


GENERATORS = {
    "dequant_int4_group": generate_dequant_int4_group_inputs,
    "dequant_int8_channel": generate_dequant_int8_channel_inputs,
    "gemm_w4a16": generate_gemm_w4a16_inputs,
    "gemm_fp8_blockscaled": generate_gemm_fp8_blockscaled_inputs,
    "gemm_w4a16_npart": generate_gemm_w4a16_npart_inputs,
    "quantize_fp8_block": generate_quantize_fp8_block_inputs,
    "quantize_int4_group": generate_quantize_int4_group_inputs,
    "dequantize_rowwise": generate_dequantize_rowwise_inputs,
    "weight_dequant": generate_weight_dequant_inputs,
    "matmul_int8": generate_matmul_int8_inputs,
    "matmul_fp32_fp16_fp8": generate_matmul_fp32_fp16_fp8_inputs,
}


def get_generator(operator_name):
    if operator_name not in GENERATORS:
        raise ValueError(f"Unsupported operator '{operator_name}'. Available operators: {list(GENERATORS)}")
    return GENERATORS[operator_name]


def infer_problem_size(operator_name, params):
    """Element count of the case's main output; the x axis of size plots."""
    if "n" in params:
        return int(params["n"])
    p = params
    if operator_name == "dequant_int4_group":
        return int(p["N"]) * int(p["K"])
    if operator_name in ("dequant_int8_channel", "dequantize_rowwise"):
        return int(p["rows"]) * int(p["cols"])
    if operator_name in ("gemm_w4a16", "gemm_w4a16_npart"):
        return int(p["M"]) * int(p["N"])
    if operator_name == "gemm_fp8_blockscaled":
        s = int(p.get("S") or 0)
        return int(p.get("M") or s) * int(p.get("N") or s)
    if operator_name == "quantize_fp8_block":
        return int(p["S"]) ** 2
    if operator_name == "quantize_int4_group":
        return int(p["N"]) * int(p["K"])
    if operator_name == "weight_dequant":
        return int(p["M"]) * int(p.get("N") or p["M"])
    if operator_name in ("matmul_int8", "matmul_fp32_fp16_fp8"):
        return 2 * int(p["M"]) * int(p["N"]) * int(p["K"])       # the reference sizes GEMMs by FLOPs (tensors.py:703-704)
    return 1
