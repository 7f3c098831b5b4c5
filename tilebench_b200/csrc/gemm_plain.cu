// Plain GEMM out[M, N] = a[M, K] . b[K, N] for the reference operator matmul_fp32_fp16_fp8
// (tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27), both operands row-major as
// the reference's generator makes them (tilebench/data/tensors.py:416-436):
//   fp16  x fp16  -> fp16   tcgen05 kind::f16,    fp32 accumulation
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

namespace tb200 {
namespace {

constexpr int kPlBM = 128;
constexpr int kPlStages = 4;
constexpr int kPlGroupM = 16;

enum PlainKind : int { PK_F16 = 0, PK_TF32 = 1, PK_F8 = 2 };

template <int KIND> struct PlainTraits;
template <> struct PlainTraits<PK_F16> {
    using In = __half;
    using Out = __half;
    static constexpr int kFmt = 0;          // f16
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
__device__ __forceinline__ void pl_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == PK_F16) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate) : "memory");
    } else if constexpr (KIND == PK_TF32) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
                     "r"(idesc), "r"(accumulate) : "memory");
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
        if (lane == 0) {
            constexpr uint32_t idesc = pl_idesc(PlainTraits<KIND>::kFmt, kPlBM, BN);
            uint32_t it = 0, tile_cnt = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_cnt) {
                const uint32_t acc = tile_cnt & 1;
                if (!mbar_wait(&bar_aempty[acc], ((tile_cnt >> 1) & 1) ^ 1, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S;
                    if (!mbar_wait(&bar_full[s], (it / S) & 1, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // a: +32 bytes along K inside the swizzle atom; b: the next kKInst rows of k
                        pl_mma<KIND>(d_tmem, a_desc + 2 * k, pl_desc_mn_sw128<KIND == PK_TF32>(b_addr + k * Cfg::kKInst * 128, Cfg::kAtomBytes),
                                     idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(&bar_empty[s]);
                }
                if (ok) tc_commit(&bar_afull[acc]);
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

TB200_DEFINE_STATUS_HOOKS(gemm_plain)

template <int KIND, int BN, typename Kern>
static int launch_plain(Kern kern, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int64_t ldo,
                        cudaStream_t st) {
    using Cfg = PlainCfg<KIND, BN>;
    static bool attr_set[64] = {false};
    int dev = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    const CUtensorMapDataType dt = KIND == PK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
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

extern "C" int tb200_matmul_plain(const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int dtype,
                                  int64_t ldo, void* stream) {
    clear_error();
    if (!a || !b || !out) return fail(TB200_ERR_ARG, "matmul_plain: null pointer");
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(TB200_ERR_ARG, "matmul_plain: non-positive size m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    if (dtype != TB200_DT_F32 && dtype != TB200_DT_F16 && dtype != TB200_DT_F8E4M3)
        return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: dtype %d is not one of F32 (tf32 math), F16, F8E4M3", dtype);
    const int elem = dtype == TB200_DT_F32 ? 4 : (dtype == TB200_DT_F16 ? 2 : 1);
    const int64_t bk = 128 / elem;
    if (k % bk != 0 || n % 128 != 0)
        return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: k=%lld must be a multiple of %lld and n=%lld of 128", (long long)k, (long long)bk, (long long)n);
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(TB200_ERR_UNSUPPORTED, "matmul_plain: dimension too large");
    if (ldo < n || (ldo * elem) % 16 != 0) return fail(TB200_ERR_ALIGN, "matmul_plain: ldo=%lld must be >= n with 16-byte aligned rows", (long long)ldo);
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return fail(TB200_ERR_ALIGN, "matmul_plain: a, b, out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t tiles256 = ((m + kPlBM - 1) / kPlBM) * (n / 256);
    const bool wide = n % 256 == 0 && 2 * tiles256 > num_sms();
    if (dtype == TB200_DT_F16)
        return wide ? launch_plain<PK_F16, 256>(tb200_k_gemm_f16_n256, a, b, out, m, n, k, ldo, st)
                    : launch_plain<PK_F16, 128>(tb200_k_gemm_f16_n128, a, b, out, m, n, k, ldo, st);
    if (dtype == TB200_DT_F32)
        return wide ? launch_plain<PK_TF32, 256>(tb200_k_gemm_tf32_n256, a, b, out, m, n, k, ldo, st)
                    : launch_plain<PK_TF32, 128>(tb200_k_gemm_tf32_n128, a, b, out, m, n, k, ldo, st);
    return wide ? launch_plain<PK_F8, 256>(tb200_k_gemm_f8_n256, a, b, out, m, n, k, ldo, st)
                : launch_plain<PK_F8, 128>(tb200_k_gemm_f8_n128, a, b, out, m, n, k, ldo, st);
}
