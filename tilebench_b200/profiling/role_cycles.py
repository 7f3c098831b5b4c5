"""Cycle accounting of the W4A16 tensor-memory kernel's roles, measured inside the kernel.

Builds a diagnostic variant of the library (`-DTB200_ROLE_CYCLES`: the statements wrapped in TB200_RC(...) in
csrc/gemm_w4a16.cu read the SM cycle counter around the phases of the issuing thread's and the convert warps' loops and
add the intervals up for CTA 0), runs one case and prints cycles per K block.  The product library is not touched and
contains none of these statements.

    python -m tilebench_b200.profiling.role_cycles --m 4096 [--k 4096 --n 14336 --repeats 5]
"""
from __future__ import annotations

import argparse
import ctypes

ISSUER = ["loop back edge", "blocking wait", "fence", "first MMA", "probes + slot arithmetic", "other MMAs + commit"]
CONVERT = ["wait: packed stage", "loads + unpack + release", "wait: operand slot", "tcgen05.st + arrive", "between visits"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--repeats", type=int, default=5)
    args = ap.parse_args(argv)

    import torch
    from tilebench_b200 import native
    from tilebench_b200.csrc import build
    from tilebench_b200.data import tensors

    native.load()                                        # fails loudly without the CUDA extension or a B200
    lib = ctypes.CDLL(str(build.build_variant("role_cycles", ["TB200_ROLE_CYCLES=1"], ["gemm_w4a16.cu"])))
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
