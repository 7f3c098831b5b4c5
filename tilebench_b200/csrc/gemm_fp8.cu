// FP8 e4m3 block-scaled GEMM for sm_100a:  out[m,n] = bf16( sum_kb sa[m,kb] * sb[n/128,kb] * (A_kb . B_kb^T) ).
//
// One persistent CTA per SM walks a grouped tile order.  Warp roles:
//   warp 0        TMA producer: per 128-wide K block, one [128 x 128 B] box of A and one
//                 [BN x 128 B] box of B into a 128-byte-swizzled shared-memory stage
//   warp 1        MMA issuer: four tcgen05.mma kind::f8f6f4 (K = 32 each) per K block into a fresh
//                 TMEM accumulator (two buffers of BN fp32 columns, alternating per K block)
//   warps 2..     drain: tcgen05.ld the finished K block's accumulator, multiply by the block's
//                 two scales and add into fp32 registers (the per-K-block scales cannot be applied
//                 after the full sum), then release the buffer; after the last K block convert to
//                 bf16 and store the thread's output row segment
// The running sum lives in registers, so the MMA warp starts the next tile while the drain warps
// still store the previous one.  Every mbarrier wait is bounded and reports through g_status.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 128;           // bytes == elements (fp8); one scale block, one swizzle atom
constexpr int kGroupM = 16;        // tile-order grouping for L2 reuse

template <int BN> struct Fp8Cfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kDrainWarps = 4 * (BN / 128);
    static constexpr int kCtrlWarps = 4;                        // warp 0 TMA, warp 1 MMA, 2 idle: one warpgroup
    static constexpr int kThreads = 32 * (kCtrlWarps + kDrainWarps);
    // 384-thread CTAs start at 168 registers per thread; the control warpgroup gives most of its
    // share back and the drain warpgroups take it (setmaxnreg), so 128 running sums plus 64
    // in-flight TMEM values fit without spilling.  The 256-thread variant has room as launched.
    static constexpr bool kReallocRegs = BN == 256;
    static constexpr int kTmemCols = 2 * BN;                    // two accumulator buffers
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

struct TileCoord { int m_blk, n_blk; };
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
    const int per_group = kGroupM * tiles_n;
    const int g = t / per_group;
    const int first_m = g * kGroupM;
    const int gsz = min(kGroupM, tiles_m - first_m);
    const int r = t - g * per_group;
    return {first_m + r % gsz, r / gsz};
}

}  // namespace
}  // namespace tb200

using namespace tb200;

template <int BN>
__device__ __forceinline__ void gemm_fp8_body(const CUtensorMap* __restrict__ tmap_a, const CUtensorMap* __restrict__ tmap_b,
                                              const float* __restrict__ sa, const float* __restrict__ sb,
                                              __nv_bfloat16* __restrict__ out, int M, int N, int K, int64_t ldo) {
    using Cfg = Fp8Cfg<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
    uint64_t* bar_empty = bar_full + S;
    uint64_t* bar_tempty = bar_empty + S;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int KB = K / kBK;
    const int tiles_m = (M + kBM - 1) / kBM;
    const int tiles_n = N / BN;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tempty[b], Cfg::kDrainWarps);   // one arrival per drain warp
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

    if (warp < Cfg::kCtrlWarps) {
      if constexpr (Cfg::kReallocRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
      if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (!mbar_wait(&bar_empty[s], ph ^ 1, ST_WAIT_SMEM_EMPTY, kb)) { ok = false; break; }
                    uint8_t* stage = smem + s * Cfg::kStageBytes;
                    mbar_expect_tx(&bar_full[s], Cfg::kStageBytes);
                    tma_load_2d(stage, tmap_a, &bar_full[s], kb * kBK, tc.m_blk * kBM);
                    tma_load_2d(stage + Cfg::kABytes, tmap_b, &bar_full[s], kb * kBK, tc.n_blk * BN);
                }
            }
            if (!ok) {
                // give copies already in flight a bounded chance to land before the CTA exits
                for (int s = 0; s < S; ++s) {
                    if (it > static_cast<uint32_t>(s)) {
                        uint32_t last = it - 1 - ((it - 1 - s) % S);   // last iteration issued on stage s
                        (void)mbar_wait(&bar_full[s], (last / S) & 1, ST_WAIT_SMEM_FULL, -1);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(0, 0, kBM, BN);  // e4m3 x e4m3 -> f32
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    const int buf = it & 1;
                    if (!mbar_wait(&bar_tempty[buf], ((it >> 1) & 1) ^ 1, ST_WAIT_TMEM_EMPTY, kb)) { ok = false; break; }
                    if (!mbar_wait(&bar_full[s], (it / S) & 1, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + Cfg::kABytes);
                    const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        // +32 bytes along K inside the swizzle atom = +2 in the descriptor's 16-byte units
                        umma_f8_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    }
                    // one commit per K block: "MMAs of this block are complete" both frees the smem
                    // stage for the producer and tells the drain warps the accumulator is ready
                    tc_commit(&bar_empty[s]);
                }
            }
        }
      }
    } else {
        if constexpr (Cfg::kReallocRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ---------------- drain warps ----------------
        const int dw = warp - Cfg::kCtrlWarps;
        const int lane_grp = warp & 3;             // TMEM lanes this warp may read: 32*(warp%4)..+31
        const int half = dw >> 2;                  // which 128-column half of the tile
        const int row_in_tile = lane_grp * 32 + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + half * 128;
        const int KBs = KB;
        uint32_t it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
            const int m = tc.m_blk * kBM + row_in_tile;
            const bool row_ok = m < M;
            const float* sa_row = sa + static_cast<int64_t>(row_ok ? m : 0) * KBs;
            const float* sb_row = sb + static_cast<int64_t>(tc.n_blk * (BN / 128) + half) * KBs;
            uint64_t acc2[64];                               // 128 running sums as packed f32 pairs
#pragma unroll
            for (int j = 0; j < 64; ++j) acc2[j] = 0ull;
            // scales are prefetched two K blocks ahead of their use
            float sc0 = __ldg(sa_row) * __ldg(sb_row);
            float sc1 = KB > 1 ? __ldg(sa_row + 1) * __ldg(sb_row + 1) : 0.f;
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const int buf = it & 1;
                float sc2 = 0.f;
                if (kb + 2 < KB) sc2 = __ldg(sa_row + kb + 2) * __ldg(sb_row + kb + 2);
                if (!mbar_wait(&bar_empty[it % S], (it / S) & 1, ST_WAIT_TMEM_FULL, kb)) { ok = false; break; }
                tc_fence_after();
                uint64_t scale2;
                asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "f"(sc0));
#pragma unroll
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t v0[32], v1[32];
                    tmem_ld32(t_lane + buf * BN + c * 64, v0);
                    tmem_ld32(t_lane + buf * BN + c * 64 + 32, v1);
                    tmem_wait_ld();
                    if (c == 1) {                            // everything is in registers: free the buffer now
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_tempty[buf]);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        uint64_t p;
                        asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(v0[2 * j]), "r"(v0[2 * j + 1]));
                        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[c * 32 + j]) : "l"(p), "l"(scale2));
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        uint64_t p;
                        asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(v1[2 * j]), "r"(v1[2 * j + 1]));
                        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[c * 32 + 16 + j]) : "l"(p), "l"(scale2));
                    }
                }
                sc0 = sc1;
                sc1 = sc2;
            }
            float acc[128];
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                uint32_t lo, hi;
                asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(acc2[j]));
                acc[2 * j] = __uint_as_float(lo);
                acc[2 * j + 1] = __uint_as_float(hi);
            }
            if (ok && row_ok) {
                __nv_bfloat16* dst = out + static_cast<int64_t>(m) * ldo + tc.n_blk * BN + half * 128;
#pragma unroll
                for (int j = 0; j < 128; j += 8) {
                    uint4 o;
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[j + 0], acc[j + 1]);
                    __nv_bfloat162 p1 = __floats2bfloat162_rn(acc[j + 2], acc[j + 3]);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[j + 4], acc[j + 5]);
                    __nv_bfloat162 p3 = __floats2bfloat162_rn(acc[j + 6], acc[j + 7]);
                    o.x = *reinterpret_cast<uint32_t*>(&p0);
                    o.y = *reinterpret_cast<uint32_t*>(&p1);
                    o.z = *reinterpret_cast<uint32_t*>(&p2);
                    o.w = *reinterpret_cast<uint32_t*>(&p3);
                    *reinterpret_cast<uint4*>(dst + j) = o;
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

extern "C" __global__ void __launch_bounds__(Fp8Cfg<256>::kThreads, 1)
tb200_k_gemm_fp8_bs_n256(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const float* sa, const float* sb, __nv_bfloat16* out, int M, int N, int K, int64_t ldo) {
    gemm_fp8_body<256>(&tmap_a, &tmap_b, sa, sb, out, M, N, K, ldo);
}
extern "C" __global__ void __launch_bounds__(Fp8Cfg<128>::kThreads, 1)
tb200_k_gemm_fp8_bs_n128(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const float* sa, const float* sb, __nv_bfloat16* out, int M, int N, int K, int64_t ldo) {
    gemm_fp8_body<128>(&tmap_a, &tmap_b, sa, sb, out, M, N, K, ldo);
}

TB200_DEFINE_STATUS_HOOKS(gemm_fp8)

template <int BN, typename Kern>
static int launch_fp8(Kern kern, const void* a, const float* sa, const void* b, const float* sb, void* out, int64_t m,
                      int64_t n, int64_t k, int64_t ldo, cudaStream_t st) {
    using Cfg = Fp8Cfg<BN>;
    static bool attr_set[64] = {false};
    int dev = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    CUtensorMap ta, tb;
    int rc = encode_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m, k, k, kBM, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k, k, BN, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    const int64_t tiles = ((m + kBM - 1) / kBM) * (n / BN);
    const int grid = static_cast<int>(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(ta, tb, sa, sb, static_cast<__nv_bfloat16*>(out),
                                                        static_cast<int>(m), static_cast<int>(n), static_cast<int>(k), ldo);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_gemm_fp8_blockscaled(const void* a, const float* sa, const void* b, const float* sb, void* out,
                                          int64_t m, int64_t n, int64_t k, int64_t ldo, void* stream) {
    clear_error();
    if (!a || !sa || !b || !sb || !out) return fail(TB200_ERR_ARG, "gemm_fp8_blockscaled: null pointer");
    if (m <= 0 || n <= 0 || k <= 0) return fail(TB200_ERR_ARG, "gemm_fp8_blockscaled: non-positive size m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    if (n % 128 != 0 || k % 128 != 0)
        return fail(TB200_ERR_ARG, "gemm_fp8_blockscaled: n=%lld and k=%lld must be multiples of 128", (long long)n, (long long)k);
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(TB200_ERR_UNSUPPORTED, "gemm_fp8_blockscaled: dimension too large");
    if (ldo < n || ldo % 8 != 0) return fail(TB200_ERR_ALIGN, "gemm_fp8_blockscaled: ldo=%lld must be >= n and a multiple of 8", (long long)ldo);
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return fail(TB200_ERR_ALIGN, "gemm_fp8_blockscaled: a, b, out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // 256-wide tiles halve shared-memory traffic per flop; use them when they still fill the SMs.
    const int64_t tiles256 = ((m + kBM - 1) / kBM) * (n / 256);
    if (n % 256 == 0 && tiles256 >= num_sms())
        return launch_fp8<256>(tb200_k_gemm_fp8_bs_n256, a, sa, b, sb, out, m, n, k, ldo, st);
    return launch_fp8<128>(tb200_k_gemm_fp8_bs_n128, a, sa, b, sb, out, m, n, k, ldo, st);
}
