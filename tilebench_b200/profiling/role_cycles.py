"""Cycle accounting of the roles of the W4A16 and the block-scaled FP8 GEMM kernels, measured inside the kernels.

Builds a diagnostic variant of the library (`-DTB200_ROLE_CYCLES`: the statements wrapped in TB200_RC(...) in
csrc/gemm_w4a16.cu and csrc/gemm_fp8.cu read the SM cycle counter around the phases of the issuing threads', the convert
warps' and the drain warps' loops and add the intervals up for CTA 0), runs one case and prints cycles per K block.
The product library is not touched and contains none of these statements.

    python -m tilebench_b200.profiling.role_cycles --m 4096 [--k 4096 --n 14336 --repeats 5]      # W4A16
    python -m tilebench_b200.profiling.role_cycles --fp8 4096                                     # FP8, S x S x S
"""
from __future__ import annotations

import argparse
import ctypes

ISSUER = ["loop back edge", "blocking wait", "fence", "first MMA", "probes + slot arithmetic", "other MMAs + commit"]
CONVERT = ["wait: packed stage", "loads + unpack + release", "wait: operand slot", "tcgen05.st + arrive", "between visits"]
FP8_DRAIN = ["wait: MMAs complete", "TMEM loads, batch 1", "FMAs, batch 1", "TMEM loads, batch 2", "release", "FMAs, batch 2", "loop top"]
FP8_ISSUER = ["waits: operands, buffer", "fence + 4 MMAs + commit", "loop overhead"]
VARIANT_SOURCES = ["gemm_w4a16.cu", "gemm_fp8.cu"]


def run_fp8(lib, size: int, repeats: int) -> None:
    import torch
    from tilebench_b200.data import tensors
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.tb200_gemm_fp8_blockscaled.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
    lib.tb200_fp8_role_cycles.argtypes = [vp, ci]
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(1)
    aq, sa = tensors.quantize_fp8_blockwise(torch.randn(size, size, device=dev, generator=gen), 1, 128)
    bq, sb = tensors.quantize_fp8_blockwise(torch.randn(size, size, device=dev, generator=gen), 128, 128)
    out = torch.empty(size, size, dtype=torch.bfloat16, device=dev)

    def call():
        rc = lib.tb200_gemm_fp8_blockscaled(vp(aq.data_ptr()), vp(sa.data_ptr()), vp(bq.data_ptr()), vp(sb.data_ptr()), vp(out.data_ptr()),
                                            size, size, size, size, vp(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"tb200_gemm_fp8_blockscaled returned {rc}")

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * 32)()
    lib.tb200_fp8_role_cycles(buf, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(repeats):
        call()
    e1.record()
    torch.cuda.synchronize()
    lib.tb200_fp8_role_cycles(buf, 0)
    v = list(buf)
    ms = e0.elapsed_time(e1) / repeats
    blocks, own = max(v[7], 1), max(v[11], 1)
    print(f"gemm_fp8_blockscaled S={size}: {ms * 1e3:.1f} us per call, {2 * size ** 3 / ms / 1e9:.0f} TFLOPS (instrumented build)")
    print(f"first drain warp, cycles per K block ({blocks} blocks of CTA 0):")
    for i, name in enumerate(FP8_DRAIN):
        print(f"  {name:28s} {v[i] / blocks:7.0f}")
    print(f"  {'total':28s} {sum(v[:7]) / blocks:7.0f}")
    print(f"issuing threads, cycles per own K block ({own} blocks, two threads taking turns):")
    for i, name in enumerate(FP8_ISSUER):
        print(f"  {name:28s} {v[8 + i] / own:7.0f}")
    print(f"  {'total':28s} {sum(v[8:11]) / own:7.0f}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--fp8", type=int, default=0, metavar="S", help="account the block-scaled FP8 GEMM at S x S x S instead")
    args = ap.parse_args(argv)

    import torch
    from tilebench_b200 import native
    from tilebench_b200.csrc import build
    from tilebench_b200.data import tensors

    native.load()                                        # fails loudly without the CUDA extension or a B200
    lib = ctypes.CDLL(str(build.build_variant("role_cycles", ["TB200_ROLE_CYCLES=1"], VARIANT_SOURCES)))
    if args.fp8:
        torch.cuda.set_device(0)
        run_fp8(lib, args.fp8, args.repeats)
        print("device status", native.device_status())
        return 0
    vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.tb200_gemm_w4a16.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ci, i64, i64, vp, sz, vp]
    lib.tb200_gemm_w4a16_workspace_bytes.argtypes = [i64, i64, i64]
    lib.tb200_gemm_w4a16_workspace_bytes.restype = sz
    lib.tb200_w4a16_role_cycles.argtypes = [vp, ci]

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    a, wp, sc, group, zp = tensors.generate_gemm_w4a16_inputs(args.m, args.k, args.n, device=dev, seed=1)
    out = torch.empty(args.m, args.n, dtype=torch.float16, device=dev)
    ws_bytes = lib.tb200_gemm_w4a16_workspace_bytes(args.m, args.n, args.k)
    ws = torch.empty(max(ws_bytes // 4, 1), dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def call():
        rc = lib.tb200_gemm_w4a16(vp(a.data_ptr()), vp(wp.data_ptr()), vp(sc.data_ptr()), vp(out.data_ptr()), args.m, args.n,
                                  args.k, group, zp, args.n, 0, vp(ws.data_ptr()), ws_bytes, vp(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"tb200_gemm_w4a16 returned {rc}")

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * 32)()
    lib.tb200_w4a16_role_cycles(buf, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms = 0.0
    for _ in range(args.repeats):
        flush.zero_()
        e0.record(); call(); e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1)
    lib.tb200_w4a16_role_cycles(buf, 0)
    v = list(buf)
    blocks, visits = max(v[6], 1), max(v[13], 1)
    print(f"gemm_w4a16 M={args.m} K={args.k} N={args.n}: {total_ms / args.repeats * 1e3:.1f} us per call (cold L2, instrumented build)")
    print(f"issuing thread(s), cycles per own K block ({blocks} blocks of CTA 0):")
    for i, name in enumerate(ISSUER):
        print(f"  {name:28s} {v[i] / blocks:7.0f}")
    print(f"  {'total':28s} {sum(v[:6]) / blocks:7.0f}")
    print(f"convert warps, cycles per visit ({visits} visits, one warp per group):")
    for i, name in enumerate(CONVERT):
        print(f"  {name:28s} {v[8 + i] / visits:7.0f}")
    print(f"  {'total':28s} {sum(v[8:13]) / visits:7.0f}")
    items = max(v[17], 1)
    print(f"CTA 0: {v[16] / args.repeats:.0f} cycles from start to the end of its epilogue per call, {items // args.repeats} work items, "
          f"{v[18] / items:.0f} cycles between items (accumulator drained before the next item's first MMA)")
    print("device status", native.device_status())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
