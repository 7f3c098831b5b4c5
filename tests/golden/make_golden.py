"""Generates tests/golden/reference_ops.npz by running the REFERENCE's own PyTorch operators
(impl_torch.run of a TileBench checkout) on seeded CPU inputs.

    python tests/golden/make_golden.py /path/to/TileBench-checkout

The checkout is only needed to regenerate; the tests read the committed .npz.  bf16 tensors are
stored as uint16 bit patterns, everything else in its own dtype.  Shapes are small and include
ragged ones (rows / cols that are not multiples of the vector width or the tile).
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "reference_ops.npz"


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


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/TileBench-checkout")
    main(sys.argv[1])
