"""Generates tests/golden/reference_ops.npz and tests/golden/baseline_configs.npz by running the
REFERENCE's own PyTorch operators (impl_torch.run of a TileBench checkout) on seeded CPU inputs.

    python tests/golden/make_golden.py /path/to/TileBench-checkout

The checkout is only needed to regenerate; the tests read the committed .npz.  bf16 tensors are
stored as uint16 bit patterns, everything else in its own dtype.  Shapes are small and include
ragged ones (rows / cols that are not multiples of the vector width or the tile).

reference_ops.npz holds the four operators the reference has.  baseline_configs.npz holds the
operators it lacks (int4 group dequant, int8 per-channel dequant, W4A16 GEMM, block-scaled FP8
GEMM, int4 group quantiser), each computed THROUGH reference code:
  * the dequant arithmetic is weight_dequant.impl_torch.run with TILE_SIZE = 1, i.e. the
    reference's elementwise X * S in fp32, followed by the cast to the operator's output type;
    what is added around it (nibble extraction, broadcasting the scales to [M, N]) is exact
    integer / copy work;
  * the GEMMs are matmul_fp32_fp16_fp8.impl_torch.run on fp32 CPU tensors of the dequantised
    operands (the "fp32 matmul of the dequantised weights" the configurations name), cast to the
    output type;
  * the int4 quantiser's scale cast is quantize_global.impl_torch.run (the reference's fp16 cast).
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "reference_ops.npz"
OUT_CONFIGS = Path(__file__).resolve().parent / "baseline_configs.npz"


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    ops = "tilebench.benchmarks.operators"
    wd = importlib.import_module(f"{ops}.weight_dequant.impl_torch")
    dr = importlib.import_module(f"{ops}.dequantize_rowwise.impl_torch")
    mi = importlib.import_module(f"{ops}.matmul_int8.impl_torch")
    mm = importlib.import_module(f"{ops}.matmul_fp32_fp16_fp8.impl_torch")
    g = torch.Generator().manual_seed(1234)
    out: dict[str, np.ndarray] = {}

    # dequantize_rowwise: every int8 value appears (row 0 = -128..127), plus ragged shapes
    for tag, (rows, cols) in {"a": (8, 256), "b": (5, 37), "c": (16, 1024)}.items():
        x = torch.randint(-128, 128, (rows, cols), dtype=torch.int8, generator=g)
        if tag == "a":
            x[0] = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
        state = torch.rand(rows, generator=g) * 10.0
        out[f"dr_{tag}_x"], out[f"dr_{tag}_state"] = x.numpy(), state.numpy()
        out[f"dr_{tag}_out"] = dr.run(x, state).numpy()

    # weight_dequant in the three dtypes, aligned and ragged
    for tag, (m, n, t) in {"a": (128, 128, 64), "b": (130, 70, 32), "c": (64, 256, 128)}.items():
        for dname, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
            X = torch.randn(m, n, generator=g).to(dt)
            S = torch.randn(-(-m // t), -(-n // t), generator=g).to(dt)
            out[f"wd_{tag}_{dname}_x"], out[f"wd_{tag}_{dname}_s"] = bits(X), bits(S)
            out[f"wd_{tag}_{dname}_out"] = bits(wd.run(X, S, m, n, t))
            out[f"wd_{tag}_{dname}_mnt"] = np.array([m, n, t])

    # matmul_int8 with 2-bit packed B
    a = torch.randint(-64, 65, (16, 64), dtype=torch.int8, generator=g)
    b = torch.randint(0, 256, (16, 24), dtype=torch.uint8, generator=g)
    out["mi_a"], out["mi_b"], out["mi_out"] = a.numpy(), b.numpy(), mi.run(a, b).numpy()

    # plain fp32 / fp16 matmul (the GEMM the W4A16 and FP8 oracles end in)
    a32 = torch.randn(32, 96, generator=g) * 96 ** -0.5
    b32 = torch.randn(96, 48, generator=g) * 96 ** -0.5
    out["mm_f32_a"], out["mm_f32_b"], out["mm_f32_out"] = a32.numpy(), b32.numpy(), mm.run(a32, b32).numpy()
    a16, b16 = a32.half(), b32.half()
    out["mm_f16_a"], out["mm_f16_b"], out["mm_f16_out"] = a16.numpy(), b16.numpy(), mm.run(a16, b16).numpy()

    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(out)} arrays)")
    baseline_configs(wd, mm, importlib.import_module(f"{ops}.quantize_global.impl_torch"))


def nibbles(wp: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/2] -> int16 [N, K]; low nibble = even k (exact integer work, no arithmetic to pin)."""
    return torch.stack(((wp & 0xF).to(torch.int16), (wp >> 4).to(torch.int16)), dim=-1).reshape(wp.shape[0], -1)


def baseline_configs(wd, mm, qg) -> None:
    g = torch.Generator().manual_seed(4321)
    out: dict[str, np.ndarray] = {}

    def int4_dequant(wp, sc, group, zp):
        n, k = wp.shape[0], wp.shape[1] * 2
        x = (nibbles(wp) - zp).to(torch.float32)
        s = sc.to(torch.float32).repeat_interleave(group, dim=1)
        return wd.run(x, s, n, k, 1).to(torch.float16)

    # ---- config 0: int4 group dequant.  Row 0 walks every nibble pair; one fp16-subnormal scale,
    # one scale at the top of the fp16 range; a second case with group 32 and zero point 3.
    for tag, (n, k, group, zp) in {"a": (32, 512, 128, 8), "b": (5, 96, 32, 3)}.items():
        wp = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
        wp[0, :min(256, k // 2)] = torch.arange(min(256, k // 2), dtype=torch.int16).to(torch.uint8)
        sc = (torch.randn(n, k // group, generator=g).abs() * 0.01 + 1e-3).to(torch.float16)
        sc[1, 0] = 6.0e-8
        sc[2, 0] = 8000.0
        out[f"i4_{tag}_wp"], out[f"i4_{tag}_s"] = wp.numpy(), sc.numpy()
        out[f"i4_{tag}_gz"] = np.array([group, zp])
        out[f"i4_{tag}_out"] = int4_dequant(wp, sc, group, zp).numpy()

    # ---- config 1: int8 per-channel dequant to bf16.  Row 0 = every int8 value; ragged shape too.
    for tag, (rows, cols) in {"a": (9, 256), "b": (5, 37), "c": (16, 4096)}.items():
        w = torch.randint(-127, 128, (rows, cols), dtype=torch.int8, generator=g)
        if cols >= 256:
            w[0, :256] = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
        w[1, 0], w[1, 1] = 127, -127
        scale = torch.randn(rows, generator=g).abs() * 0.02 + 1e-4
        y = wd.run(w.to(torch.float32), scale[:, None].expand(rows, cols), rows, cols, 1)
        out[f"i8_{tag}_w"], out[f"i8_{tag}_scale"] = w.numpy(), scale.numpy()
        out[f"i8_{tag}_out"] = bits(y.to(torch.bfloat16))

    # ---- config 2: W4A16 GEMM = reference fp32 matmul of the activations and the fp16-rounded
    # dequantised weights, cast to fp16.  One weight set, activation heights on both sides of every
    # kernel boundary (streaming <= 16, split-K <= 64, tiled above).
    n, k, group, zp = 128, 256, 128, 8
    wp = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
    sc = (torch.randn(n, k // group, generator=g).abs() * 0.01 + 1e-3).to(torch.float16)
    wdq = int4_dequant(wp, sc, group, zp)
    out["w4_wp"], out["w4_s"], out["w4_gz"] = wp.numpy(), sc.numpy(), np.array([group, zp])
    for m in (1, 16, 33, 130):
        a = torch.randn(m, k, generator=g).to(torch.float16)
        out[f"w4_m{m}_a"] = a.numpy()
        out[f"w4_m{m}_out"] = mm.run(a.to(torch.float32), wdq.to(torch.float32).t()).to(torch.float16).numpy()

    # ---- config 3: block-scaled FP8 GEMM = reference fp32 matmul of the dequantised operands, cast
    # to bf16.  Quantised as the configuration says (scale = amax / 448, so every non-zero block
    # holds a +-448 code); one all-zero block in each operand, one subnormal fp32 scale.
    m, n, k = 130, 128, 384
    a = torch.randn(m, k, generator=g)
    b = torch.randn(n, k, generator=g)
    a[3, 128:256] = 0.0
    b[:, 256:384] = 0.0
    a[5, 0:128] *= 1e-37
    sa = a.reshape(m, k // 128, 128).abs().amax(dim=2) / 448.0
    sa = torch.where(sa == 0, torch.ones_like(sa), sa)
    aq = (a / sa.repeat_interleave(128, dim=1)).to(torch.float8_e4m3fn)
    sb = b.reshape(n // 128, 128, k // 128, 128).abs().amax(dim=(1, 3)) / 448.0
    sb = torch.where(sb == 0, torch.ones_like(sb), sb)
    bq = (b / sb.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)).to(torch.float8_e4m3fn)
    adq = wd.run(aq.to(torch.float32), sa.repeat_interleave(128, dim=1), m, k, 1)
    bdq = wd.run(bq.to(torch.float32), sb, n, k, 128)          # the reference's own 128 x 128 block scaling
    out["f8_aq"], out["f8_sa"] = aq.view(torch.uint8).numpy(), sa.numpy()
    out["f8_bq"], out["f8_sb"] = bq.view(torch.uint8).numpy(), sb.numpy()
    out["f8_out"] = bits(mm.run(adq, bdq.t()).to(torch.bfloat16))

    # ---- int4 group quantiser: scale cast by the reference's quantiser operator, codes checked by
    # dequantising them through the reference multiply above.
    x = torch.randn(8, 256, generator=g) * 0.05
    x[1] = 0.0
    amax = x.reshape(8, 2, 128).abs().amax(dim=2)
    s16 = qg.run(amax / 7.0)
    s16 = torch.where(s16.to(torch.float32) == 0, torch.ones_like(s16), s16)
    q = torch.clamp(torch.round(x / s16.to(torch.float32).repeat_interleave(128, dim=1)) + 8.0, 0, 15).to(torch.uint8)
    qwp = q[:, 0::2] | (q[:, 1::2] << 4)
    out["q4_x"], out["q4_s"], out["q4_wp"] = x.numpy(), s16.numpy(), qwp.numpy()
    out["q4_back"] = int4_dequant(qwp, s16, 128, 8).numpy()

    np.savez_compressed(OUT_CONFIGS, **out)
    print(f"wrote {OUT_CONFIGS} ({OUT_CONFIGS.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/TileBench-checkout")
    main(sys.argv[1])
