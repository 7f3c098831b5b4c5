// Plain GEMM out[M, N] = a[M, K] . b[K, N] for the reference operator matmul_fp32_fp16_fp8
// (tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27), both operands row-major as
// the reference's generator makes them (tilebench/data/tensors.py:416-436):
//   fp16  x fp16  -> fp16   tcgen05 kind::f16,    fp32 accumulation   (bf16 x bf16 -> bf16 likewise)
//   fp32  x fp32  -> fp32   tcgen05 kind::tf32 (the reference sets allow_tf32), fp32 accumulation
//   e4m3  x e4m3  -> e4m3   tcgen05 kind::f8f6f4, fp32 accumulation, rounded to bf16 and then to e4m3 as the
//                           reference does (_scaled_mm with unit scales and out_dtype bf16, then a cast)
// b is [K, N] with N contiguous.  The tensor core reads such a tile as an MN-major operand, so b goes
// from global memory to the MMA untouched: no transposed copy is made or cached (the reference's fp8
// path keeps a column-major copy of b across calls).
//
// One persistent CTA per SM, 128 x BN output tiles, stages of 128 bytes of K per row of a:
//   warp 0      TMA producer: one [128 x 128 B] box of a (K-major, 128-byte swizzle) and one
//               [BK x 128 B] box of b per 128-byte column block (MN-major, 128-byte swizzle)
//   warp 1      MMA issuer: four MMAs per stage (32 bytes of K each) into one of two TMEM accumulators
//   warps 4..7  epilogue: tcgen05.ld, convert, 16-byte stores; overlaps the next tile's main loop
// Every mbarrier wait is bounded and reports through g_status.
#include "common.cuh"
#include <cuda_fp8.h>
#include <cstdlib>
#include <cstring>

namespace tb200 {
namespace {

constexpr int kPlBM = 128;
constexpr int kPlStages = 4;
constexpr int kPlGroupM = 16;

enum PlainKind : int { PK_F16 = 0, PK_TF32 = 1, PK_F8 = 2, PK_BF16 = 3 };

template <int KIND> struct PlainTraits;
template <> struct PlainTraits<PK_F16> {
    using In = __half;
    using Out = __half;
    static constexpr int kFmt = 0;          // f16
};
template <> struct PlainTraits<PK_BF16> {
    using In = __nv_bfloat16;
    using Out = __nv_bfloat16;
    static constexpr int kFmt = 1;          // bf16
};
template <> struct PlainTraits<PK_TF32> {
    using In = float;
    using Out = float;
    static constexpr int kFmt = 2;          // tf32
};
template <> struct PlainTraits<PK_F8> {
    using In = uint8_t;
    using Out = uint8_t;
    static constexpr int kFmt = 0;          // e4m3
};

template <int KIND, int BN> struct PlainCfg {
    using T = PlainTraits<KIND>;
    static constexpr int kElem = sizeof(typename T::In);
    static constexpr int kBK = 128 / kElem;                     // elements of K per stage
    static constexpr int kKInst = 32 / kElem;                   // elements of K per MMA
    static constexpr int kAtomCols = 128 / kElem;               // columns of b per 128-byte block
    static constexpr int kAtoms = BN / kAtomCols;
    static constexpr int kABytes = kPlBM * 128;
    static constexpr int kAtomBytes = kBK * 128;                // one [BK x 128 B] box of b
    static constexpr int kBBytes = kAtoms * kAtomBytes;         // == BK * BN * elem
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kThreads = 256;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kPlStages * kStageBytes + kBarBytes + 1024;
};

// MN-major operand, 128-byte swizzle: rows of k 128 bytes apart, 8-row groups 1024 bytes apart
// (stride offset), 128-byte column blocks `atom_pitch` bytes apart (leading offset).
// 32-bit elements are transposed by the tensor core in 32-byte units and need the variant of the swizzle
// whose unit is 32 bytes (layout code 1): it repeats every 4 rows, so the row groups are 512 bytes apart.
template <bool k32BitElems>
__device__ __forceinline__ uint64_t pl_desc_mn_sw128(uint32_t smem_addr, uint32_t atom_pitch) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(atom_pitch >> 4) << 16;
    d |= static_cast<uint64_t>((k32BitElems ? 512 : 1024) >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(k32BitElems ? 1 : 2) << 61;
    return d;
}
// D = f32, A K-major, B MN-major (bit 16)
__host__ __device__ constexpr uint32_t pl_idesc(uint32_t fmt, uint32_t m, uint32_t n) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
template <int KIND>
__device__ __forceinline__ void pl_mma(uint32_t issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == PK_F16 || KIND == PK_BF16) {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    } else if constexpr (KIND == PK_TF32) {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    }
}

template <int KIND>
__device__ __forceinline__ void pl_mma_pair(uint32_t issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == PK_F16 || KIND == PK_BF16) {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    } else if constexpr (KIND == PK_TF32) {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                     "@q tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate), "r"(issue) : "memory");
    }
}

struct PlTile { int m_blk, n_blk; };
__device__ __forceinline__ PlTile pl_tile(int t, int tiles_m, int tiles_n) {
    const int per_group = kPlGroupM * tiles_n;
    const int g = t / per_group;
    const int first_m = g * kPlGroupM;
    const int gsz = min(kPlGroupM, tiles_m - first_m);
    const int r = t - g * per_group;
    return {first_m + r % gsz, r / gsz};
}

// 32 fp32 accumulator values of one row -> output elements, 16-byte stores
__device__ __forceinline__ void pl_store32(__half* dst, const uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __half2 h = __floats2half2_rn(__uint_as_float(v[8 * q + 2 * e]), __uint_as_float(v[8 * q + 2 * e + 1]));
            w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + 8 * q) = o;
    }
}
__device__ __forceinline__ void pl_store32(__nv_bfloat16* dst, const uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]), __uint_as_float(v[8 * q + 2 * e + 1]));
            w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + 8 * q) = o;
    }
}
__device__ __forceinline__ void pl_store32(float* dst, const uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(dst + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
}
// fp32 -> bf16 -> e4m3, both round-to-nearest-even.  The hardware conversion saturates; PyTorch's cast does
// not: a bf16 value above 464 (the last one that rounds down to 448) becomes NaN there, so it does here.
__device__ __forceinline__ uint32_t pl_e4m3x2(float x, float y) {
    const float rx = __bfloat162float(__float2bfloat16_rn(x));
    const float ry = __bfloat162float(__float2bfloat16_rn(y));
    uint32_t q = __nv_cvt_float2_to_fp8x2(make_float2(rx, ry), __NV_SATFINITE, __NV_E4M3);
    if (fabsf(rx) > 464.0f) q |= 0x007Fu;
    if (fabsf(ry) > 464.0f) q |= 0x7F00u;
    return q;
}
__device__ __forceinline__ void pl_store32(uint8_t* dst, const uint32_t (&v)[32]) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 16 * q + 4 * e;
            w[e] = pl_e4m3x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])) |
                   (pl_e4m3x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])) << 16);
        }
        *reinterpret_cast<uint4*>(dst + 16 * q) = o;
    }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

template <int KIND, int BN>
__device__ __forceinline__ void gemm_plain_body(const CUtensorMap* __restrict__ tmap_a, const CUtensorMap* __restrict__ tmap_b,
                                                typename PlainTraits<KIND>::Out* __restrict__ out, int M, int N, int K,
                                                int64_t ldo) {
    using Cfg = PlainCfg<KIND, BN>;
    constexpr int S = kPlStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
    uint64_t* bar_empty = bar_full + S;
    uint64_t* bar_afull = bar_empty + S;      // [2] accumulator complete
    uint64_t* bar_aempty = bar_afull + 2;     // [2] accumulator drained (4 epilogue warps)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_aempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int KB = K / Cfg::kBK;
    const int tiles_m = (M + kPlBM - 1) / kPlBM;
    const int tiles_n = N / BN;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_afull[b], 1);
            mbar_init(&bar_aempty[b], 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(tmap_a);
        tma_prefetch_desc(tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const PlTile tc = pl_tile(t, tiles_m, tiles_n);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    if (!mbar_wait(&bar_empty[s], ((it / S) & 1) ^ 1, ST_WAIT_SMEM_EMPTY, kb)) { ok = false; break; }
                    uint8_t* stage = smem + s * Cfg::kStageBytes;
                    mbar_expect_tx(&bar_full[s], Cfg::kStageBytes);
                    tma_load_2d(stage, tmap_a, &bar_full[s], kb * Cfg::kBK, tc.m_blk * kPlBM);
#pragma unroll
                    for (int at = 0; at < Cfg::kAtoms; ++at)
                        tma_load_2d(stage + Cfg::kABytes + at * Cfg::kAtomBytes, tmap_b, &bar_full[s],
                                    tc.n_blk * BN + at * Cfg::kAtomCols, kb * Cfg::kBK);
                }
            }
            if (!ok) {
                for (int s = 0; s < S; ++s) {
                    if (it > static_cast<uint32_t>(s)) {
                        const uint32_t last = it - 1 - ((it - 1 - s) % S);
                        (void)mbar_wait(&bar_full[s], (last / S) & 1, ST_WAIT_SMEM_FULL, -1);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp walks the loop (waits and slot arithmetic are warp-uniform) and lane 0 issues: a lone
        // thread inside an `if (lane == 0)` region pays 100-250 cycles per branch.  The stage's descriptors are a
        // base plus a slot offset, the slot and its phase advance by addition, and the next slot's barrier is probed
        // (non-blocking) between the first and second MMA, so the blocking wait is skipped when the copies are ahead.
        {
            constexpr uint32_t idesc = pl_idesc(PlainTraits<KIND>::kFmt, kPlBM, BN);
            constexpr uint32_t kStageDesc = Cfg::kStageBytes >> 4;
            const bool leader = lane == 0;
            const uint64_t a_desc0 = umma_desc_sw128(smem_u32(smem));
            const uint64_t b_desc0 = pl_desc_mn_sw128<KIND == PK_TF32>(smem_u32(smem) + Cfg::kABytes, Cfg::kAtomBytes);
            uint32_t s = 0, ph = 0, tile_cnt = 0;
            bool ready = false;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_cnt) {
                const uint32_t acc = tile_cnt & 1;
                if (!mbar_wait(&bar_aempty[acc], ((tile_cnt >> 1) & 1) ^ 1, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < KB; ++kb) {
                    if (!ready && !mbar_wait(&bar_full[s], ph, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + s * kStageDesc;
                    const uint64_t b_desc = b_desc0 + s * kStageDesc;
                    uint64_t* const freed = &bar_empty[s];
                    if (++s == static_cast<uint32_t>(S)) { s = 0; ph ^= 1; }
                    // predicated, not branched: every lane runs the statements, lane 0's instructions take effect
                    pl_mma<KIND>(leader, d_tmem, a_desc, b_desc, idesc, kb > 0 ? 1u : 0u);
                    ready = mbar_test_wait(&bar_full[s], ph);
#pragma unroll
                    for (int k = 1; k < 4; ++k) {
                        // a: +32 bytes along K inside the swizzle atom; b: the next kKInst rows of k (16-byte units)
                        pl_mma<KIND>(leader, d_tmem, a_desc + 2 * k, b_desc + static_cast<uint64_t>(k * Cfg::kKInst * 128 / 16), idesc, 1u);
                    }
                    tc_commit_if(leader, freed);
                }
                if (ok && leader) tc_commit(&bar_afull[acc]);
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue ----------------
        using Out = typename PlainTraits<KIND>::Out;
        const int ew = warp - 4;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
        uint32_t tile_cnt = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_cnt) {
            const PlTile tc = pl_tile(t, tiles_m, tiles_n);
            const uint32_t acc = tile_cnt & 1;
            const int m = tc.m_blk * kPlBM + ew * 32 + lane;
            if (!mbar_wait(&bar_afull[acc], (tile_cnt >> 1) & 1, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
            tc_fence_after();
            Out* dst = out + static_cast<int64_t>(m < M ? m : 0) * ldo + tc.n_blk * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
                uint32_t v0[32], v1[32];
                tmem_ld32(t_lane + acc * BN + c * 64, v0);
                tmem_ld32(t_lane + acc * BN + c * 64 + 32, v1);
                tmem_wait_ld();
                if (c == BN / 64 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_aempty[acc]);
                }
                if (m < M) {
                    pl_store32(dst + c * 64, v0);
                    pl_store32(dst + c * 64 + 32, v1);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs on neighbouring SMs share one 256 x 256 output tile.  Each
// CTA loads its 128 rows of a and its 128-column half of b; the leader's MMA thread issues M = 256 MMAs
// that read both CTAs' shared memory, so every SM fetches and re-reads only half of the b tile.
// "Stage full" lives in the leader (both CTAs' TMA bytes are counted there), the commits arrive on
// "stage free" and "accumulator complete" in both CTAs, "accumulator drained" lives in the leader.
template <int KIND> struct PlainPairCfg {
    using Base = PlainCfg<KIND, 256>;
    static constexpr int kStages = 6;
    static constexpr int kAtoms = Base::kAtoms / 2;             // this CTA's column blocks of b
    static constexpr int kBBytes = kAtoms * Base::kAtomBytes;
    static constexpr int kStageBytes = Base::kABytes + kBBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + Base::kBarBytes + 1024;
};

template <int KIND>
__device__ __forceinline__ void gemm_plain_pair_body(const CUtensorMap* __restrict__ tmap_a, const CUtensorMap* __restrict__ tmap_b,
                                                     typename PlainTraits<KIND>::Out* __restrict__ out, int M, int N, int K,
                                                     int64_t ldo) {
    using Cfg = PlainCfg<KIND, 256>;
    using PCfg = PlainPairCfg<KIND>;
    constexpr int S = PCfg::kStages;
    constexpr int BN = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + S * PCfg::kStageBytes);
    uint64_t* bar_empty = bar_full + S;
    uint64_t* bar_afull = bar_empty + S;
    uint64_t* bar_aempty = bar_afull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_aempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = static_cast<int>(cluster_ctarank());       // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int npairs = gridDim.x >> 1;
    const int KB = K / Cfg::kBK;
    const int tiles_m = (M + 2 * kPlBM - 1) / (2 * kPlBM);
    const int tiles_n = N / BN;
    const int tiles = tiles_m * tiles_n;
    auto coord = [&](int t) {
        constexpr int kGroup = kPlGroupM / 2;
        const int per_group = kGroup * tiles_n;
        const int g = t / per_group;
        const int first_m = g * kGroup;
        const int gsz = min(kGroup, tiles_m - first_m);
        const int r = t - g * per_group;
        return PlTile{first_m + r % gsz, r / gsz};
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_afull[b], 1);
            mbar_init(&bar_aempty[b], 8);                        // 4 epilogue warps in each CTA
        }
        mbar_fence_init();
        tma_prefetch_desc(tmap_a);
        tma_prefetch_desc(tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                          // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += npairs) {
                const PlTile tc = coord(t);
                const int a_row = tc.m_blk * 2 * kPlBM + rank * kPlBM;
                const int b_col = tc.n_blk * BN + rank * (BN / 2);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    if (!mbar_wait(&bar_empty[s], ((it / S) & 1) ^ 1, ST_WAIT_SMEM_EMPTY, kb)) { ok = false; break; }
                    uint8_t* stage = smem + s * PCfg::kStageBytes;
                    if (rank == 0) mbar_expect_tx(&bar_full[s], 2 * PCfg::kStageBytes);     // both CTAs' bytes
                    tma_load_2d_pair(stage, tmap_a, &bar_full[s], kb * Cfg::kBK, a_row);
#pragma unroll
                    for (int at = 0; at < PCfg::kAtoms; ++at)
                        tma_load_2d_pair(stage + Cfg::kABytes + at * Cfg::kAtomBytes, tmap_b, &bar_full[s],
                                         b_col + at * Cfg::kAtomCols, kb * Cfg::kBK);
                }
            }
            if (!ok) {
                // copies in flight land within microseconds; a bounded pause before the CTA may exit
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 21)) {}
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ---------------- MMA issuer (leader only; whole warp in the loop, lane 0 issues — see the single-CTA kernel) ----------------
        {
            constexpr uint32_t idesc = pl_idesc(PlainTraits<KIND>::kFmt, 2 * kPlBM, BN);
            constexpr uint32_t kStageDesc = PCfg::kStageBytes >> 4;
            const bool leader = lane == 0;
            const uint64_t a_desc0 = umma_desc_sw128(smem_u32(smem));
            const uint64_t b_desc0 = pl_desc_mn_sw128<KIND == PK_TF32>(smem_u32(smem) + Cfg::kABytes, Cfg::kAtomBytes);
            uint32_t s = 0, ph = 0, tile_cnt = 0;
            bool ready = false;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += npairs, ++tile_cnt) {
                const uint32_t acc = tile_cnt & 1;
                if (!mbar_wait(&bar_aempty[acc], ((tile_cnt >> 1) & 1) ^ 1, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < KB; ++kb) {
                    if (!ready && !mbar_wait(&bar_full[s], ph, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t a_desc = a_desc0 + s * kStageDesc;
                    const uint64_t b_desc = b_desc0 + s * kStageDesc;
                    uint64_t* const freed = &bar_empty[s];
                    if (++s == static_cast<uint32_t>(S)) { s = 0; ph ^= 1; }
                    pl_mma_pair<KIND>(leader, d_tmem, a_desc, b_desc, idesc, kb > 0 ? 1u : 0u);
                    ready = mbar_test_wait(&bar_full[s], ph);
#pragma unroll
                    for (int k = 1; k < 4; ++k)
                        pl_mma_pair<KIND>(leader, d_tmem, a_desc + 2 * k, b_desc + static_cast<uint64_t>(k * Cfg::kKInst * 128 / 16), idesc, 1u);
                    if (leader) tc_commit_pair(freed, 0x3);
                }
                if (ok && leader) tc_commit_pair(&bar_afull[acc], 0x3);
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue (both CTAs; each owns 128 rows of the tile) ----------------
        using Out = typename PlainTraits<KIND>::Out;
        const int ew = warp - 4;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
        uint32_t tile_cnt = 0;
        bool ok = true;
        for (int t = pair; t < tiles && ok; t += npairs, ++tile_cnt) {
            const PlTile tc = coord(t);
            const uint32_t acc = tile_cnt & 1;
            const int m = tc.m_blk * 2 * kPlBM + rank * kPlBM + ew * 32 + lane;
            if (!mbar_wait(&bar_afull[acc], (tile_cnt >> 1) & 1, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
            tc_fence_after();
            Out* dst = out + static_cast<int64_t>(m < M ? m : 0) * ldo + tc.n_blk * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
                uint32_t v0[32], v1[32];
                tmem_ld32(t_lane + acc * BN + c * 64, v0);
                tmem_ld32(t_lane + acc * BN + c * 64 + 32, v1);
                tmem_wait_ld();
                if (c == BN / 64 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_leader(&bar_aempty[acc]);
                }
                if (m < M) {
                    pl_store32(dst + c * 64, v0);
                    pl_store32(dst + c * 64 + 32, v1);
                }
            }
        }
    }

    // neither CTA may leave while the other can still read its shared memory or signal its barriers
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

#define TB200_PLAIN_PAIR_KERNEL(name, KIND)                                                                             \
    extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)                                      \
    name(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,                        \
         typename PlainTraits<KIND>::Out* out, int M, int N, int K, int64_t ldo) {                                      \
        gemm_plain_pair_body<KIND>(&tmap_a, &tmap_b, out, M, N, K, ldo);                                                \
    }
TB200_PLAIN_PAIR_KERNEL(tb200_k_gemm_f16_pair, PK_F16)
TB200_PLAIN_PAIR_KERNEL(tb200_k_gemm_tf32_pair, PK_TF32)
TB200_PLAIN_PAIR_KERNEL(tb200_k_gemm_f8_pair, PK_F8)
TB200_PLAIN_PAIR_KERNEL(tb200_k_gemm_bf16_pair, PK_BF16)

#define TB200_PLAIN_KERNEL(name, KIND, BN)                                                                              \
    extern "C" __global__ void __launch_bounds__(256, 1)                                                                \
    name(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,                        \
         typename PlainTraits<KIND>::Out* out, int M, int N, int K, int64_t ldo) {                                      \
        gemm_plain_body<KIND, BN>(&tmap_a, &tmap_b, out, M, N, K, ldo);                                                 \
    }
TB200_PLAIN_KERNEL(tb200_k_gemm_f16_n256, PK_F16, 256)
TB200_PLAIN_KERNEL(tb200_k_gemm_f16_n128, PK_F16, 128)
TB200_PLAIN_KERNEL(tb200_k_gemm_tf32_n256, PK_TF32, 256)
TB200_PLAIN_KERNEL(tb200_k_gemm_tf32_n128, PK_TF32, 128)
TB200_PLAIN_KERNEL(tb200_k_gemm_f8_n256, PK_F8, 256)
TB200_PLAIN_KERNEL(tb200_k_gemm_f8_n128, PK_F8, 128)
TB200_PLAIN_KERNEL(tb200_k_gemm_bf16_n256, PK_BF16, 256)
TB200_PLAIN_KERNEL(tb200_k_gemm_bf16_n128, PK_BF16, 128)

TB200_DEFINE_STATUS_HOOKS(gemm_plain)

template <int KIND, int BN, typename Kern>
static int launch_plain(Kern kern, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int64_t ldo,
                        cudaStream_t st) {
    using Cfg = PlainCfg<KIND, BN>;
    static PerDeviceInt attr_set;
    {
        const int rc_attr = ensure_max_smem(attr_set, reinterpret_cast<const void*>(kern), Cfg::kSmemBytes);
        if (rc_attr != TB200_OK) return rc_attr;
    }
    const CUtensorMapDataType dt = KIND == PK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : KIND == PK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : KIND == PK_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMap ta, tb;
    int rc = encode_tmap_2d(&ta, a, dt, Cfg::kElem, m, k, k * Cfg::kElem, kPlBM, Cfg::kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tb, b, dt, Cfg::kElem, k, n, n * Cfg::kElem, Cfg::kBK, Cfg::kAtomCols,
                        KIND == PK_TF32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    const int64_t tiles = ((m + kPlBM - 1) / kPlBM) * (n / BN);
    const int grid = static_cast<int>(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(ta, tb, static_cast<typename PlainTraits<KIND>::Out*>(out),
                                                        static_cast<int>(m), static_cast<int>(n), static_cast<int>(k), ldo);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

template <int KIND, typename Kern>
static int launch_plain_pair(Kern kern, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int64_t ldo,
                             cudaStream_t st) {
    using Cfg = PlainCfg<KIND, 256>;
    using PCfg = PlainPairCfg<KIND>;
    static PerDeviceInt max_pairs_tab;
    int dev = 0;
    {
        const int rc_dev = current_device(&dev);
        if (rc_dev != TB200_OK) return rc_dev;
    }
    int max_pairs = max_pairs_tab.v[dev].load(std::memory_order_acquire);
    if (max_pairs == 0) {
        TB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PCfg::kSmemBytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(num_sms() & ~1), 1, 1);
        cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
        cfg.dynamicSmemBytes = PCfg::kSmemBytes;
        int clusters = 0;
        TB200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg));
        if (clusters < 1) return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: no CTA pair fits on this device");
        max_pairs = clusters;
        max_pairs_tab.v[dev].store(clusters, std::memory_order_release);
    }
    const CUtensorMapDataType dt = KIND == PK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : KIND == PK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : KIND == PK_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMap ta, tb;
    int rc = encode_tmap_2d(&ta, a, dt, Cfg::kElem, m, k, k * Cfg::kElem, kPlBM, Cfg::kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tb, b, dt, Cfg::kElem, k, n, n * Cfg::kElem, Cfg::kBK, Cfg::kAtomCols,
                        KIND == PK_TF32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    const int64_t tiles = ((m + 2 * kPlBM - 1) / (2 * kPlBM)) * (n / 256);
    const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    kern<<<2 * pairs, Cfg::kThreads, PCfg::kSmemBytes, st>>>(ta, tb, static_cast<typename PlainTraits<KIND>::Out*>(out),
                                                              static_cast<int>(m), static_cast<int>(n), static_cast<int>(k), ldo);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_matmul_plain(const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int dtype,
                                  int64_t ldo, void* stream) {
    clear_error();
    if (!a || !b || !out) return fail(TB200_ERR_ARG, "matmul_plain: null pointer");
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(TB200_ERR_ARG, "matmul_plain: non-positive size m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    if (dtype != TB200_DT_F32 && dtype != TB200_DT_F16 && dtype != TB200_DT_BF16 && dtype != TB200_DT_F8E4M3)
        return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: dtype %d is not one of F32 (tf32 math), F16, BF16, F8E4M3", dtype);
    const int elem = dtype == TB200_DT_F32 ? 4 : (dtype == TB200_DT_F8E4M3 ? 1 : 2);
    const int64_t bk = 128 / elem;
    if (k % bk != 0 || n % 128 != 0)
        return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: k=%lld must be a multiple of %lld and n=%lld of 128", (long long)k, (long long)bk, (long long)n);
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: dimension too large");
    if (ldo < n || (ldo * elem) % 16 != 0) return fail(TB200_ERR_ALIGN, "matmul_plain: ldo=%lld must be >= n with 16-byte aligned rows", (long long)ldo);
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return fail(TB200_ERR_ALIGN, "matmul_plain: a, b, out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t tiles256 = ((m + kPlBM - 1) / kPlBM) * (n / 256);
    const bool wide = n % 256 == 0 && 2 * tiles256 > num_sms();
    // CTA pairs on 256 x 256 tiles once there are enough tiles to occupy most pairs of SMs: measured 1.1x
    // (fp16), 1.25x (fp32) and up to 1.15x (e4m3) over the single-CTA kernel at 4096 x 4096 outputs, with
    // bit-identical results.  TB200_PLAIN_VARIANT = "pair" | "single" overrides the choice (tuning and tests).
    const char* force = getenv("TB200_PLAIN_VARIANT");
    const int64_t tiles_pair = ((m + 2 * kPlBM - 1) / (2 * kPlBM)) * (n / 256);
    const bool pair = force ? !strcmp(force, "pair") : 4 * tiles_pair >= num_sms();
    if (pair && n % 256 == 0 && tiles_pair >= 1) {
        if (dtype == TB200_DT_F16) return launch_plain_pair<PK_F16>(tb200_k_gemm_f16_pair, a, b, out, m, n, k, ldo, st);
        if (dtype == TB200_DT_BF16) return launch_plain_pair<PK_BF16>(tb200_k_gemm_bf16_pair, a, b, out, m, n, k, ldo, st);
        if (dtype == TB200_DT_F32) return launch_plain_pair<PK_TF32>(tb200_k_gemm_tf32_pair, a, b, out, m, n, k, ldo, st);
        return launch_plain_pair<PK_F8>(tb200_k_gemm_f8_pair, a, b, out, m, n, k, ldo, st);
    }
    if (dtype == TB200_DT_BF16)
        return wide ? launch_plain<PK_BF16, 256>(tb200_k_gemm_bf16_n256, a, b, out, m, n, k, ldo, st)
                    : launch_plain<PK_BF16, 128>(tb200_k_gemm_bf16_n128, a, b, out, m, n, k, ldo, st);
    if (dtype == TB200_DT_F16)
        return wide ? launch_plain<PK_F16, 256>(tb200_k_gemm_f16_n256, a, b, out, m, n, k, ldo, st)
                    : launch_plain<PK_F16, 128>(tb200_k_gemm_f16_n128, a, b, out, m, n, k, ldo, st);
    if (dtype == TB200_DT_F32)
        return wide ? launch_plain<PK_TF32, 256>(tb200_k_gemm_tf32_n256, a, b, out, m, n, k, ldo, st)
                    : launch_plain<PK_TF32, 128>(tb200_k_gemm_tf32_n128, a, b, out, m, n, k, ldo, st);
    return wide ? launch_plain<PK_F8, 256>(tb200_k_gemm_f8_n256, a, b, out, m, n, k, ldo, st)
                : launch_plain<PK_F8, 128>(tb200_k_gemm_f8_n128, a, b, out, m, n, k, ldo, st);
}
