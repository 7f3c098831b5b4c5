// Decode-sized W4A16 (m <= 16), streaming form: one persistent CTA per SM, every warp its own TMA ring.
//
// The weight stream (n * k / 2 bytes) is all that matters at this size, and it only runs at HBM speed when
// enough bytes are in flight: bandwidth x latency is about 35 KB per SM on this part.  Register-staged loads
// cannot hold that much, so the packed rows travel by TMA: a work unit is 8 weight rows over the whole K,
// owned by ONE warp (no cross-warp reduction, no workspace, fixed summation order), and the warp keeps a ring
// of kStages boxes of [8 rows x 128 bytes] (256 values of k each, 128-byte swizzle) in flight for itself —
// lane 0 re-arms a slot and issues the next box as soon as the warp has read it.  13 warps x 6 KB per SM for
// the benchmark shape.
//
// The arithmetic is warp-level mma.sync.m16n8k16 (fp16 in, fp32 accumulate) with the activations as the
// 16-row operand and the 8 weight rows as the 8-column operand.  K order inside an MMA is free as long as both
// operands agree, which is used twice:
//   * a lane reads 16 contiguous packed bytes (one LDS.128, bank-conflict free under the swizzle because
//     operand column g sits in box row g/2 (+4 for odd g)), and unpacks each 32-bit word of 8 nibbles with
//     (w >> 4i) & 0x000f000f | 0x64006400 — one shift and one LOP3 per PAIR, the pair being nibbles (i, i+4);
//   * the activations are laid out once per CTA in shared memory in exactly that order ([k0, k0+4, k0+1, k0+5,
//     k0+2, k0+6, k0+3, k0+7] per word, word-major, rows XOR-swizzled against bank conflicts), so one LDS.128
//     is the A fragment of two MMA steps.
// Weights are rounded to fp16 after scaling — fp16((q - zp) * s), one rounding, the value the dequant kernel
// and the tensor-memory GEMM produce.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kRgWarps = 16;
constexpr int kRgThreads = 32 * kRgWarps;
constexpr int kRgBoxBytes = 8 * 128;          // one ring slot: 8 rows x 128 packed bytes = 256 k
constexpr int kRgStageK = 256;

template <int MPAD> struct RingCfg {
    static constexpr int kStages = MPAD == 8 ? 6 : 5;
    static constexpr int kRingBytes = kRgWarps * kStages * kRgBoxBytes;
    static constexpr int kBarBytes = kRgWarps * kStages * 8;
    // activations: (k / 8) words x MPAD rows x 16 bytes
    static constexpr int act_bytes(int kpad) { return kpad / 8 * MPAD * 16; }
    static constexpr int smem_bytes(int kpad) { return 1024 + kRingBytes + act_bytes(kpad) + kBarBytes; }
};
constexpr int kRgMaxSmem = 232448;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// nibbles (i, i + 4) of `w` (already shifted right by 4i) -> fp16 pair ((q - zp) * s), one rounding each
__device__ __forceinline__ uint32_t rg_pair(uint32_t w_shifted, __half2 bias, __half2 s2) {
    uint32_t h;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h) : "r"(w_shifted));
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h), bias), s2);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

template <int MPAD>
__device__ __forceinline__ void gemv_ring_body(const CUtensorMap* __restrict__ tmap_w, const __half* __restrict__ a,
                                               const __half* __restrict__ scales, __half* __restrict__ out, int M, int K, int kpad,
                                               int groups_per_row, int group128, int64_t ldo, int64_t col_offset,
                                               float zp_plus_1024, int units, int warps_used) {
    using Cfg = RingCfg<MPAD>;
    constexpr int ST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring_all = smem;
    uint8_t* act = smem + Cfg::kRingBytes;
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(act + Cfg::act_bytes(kpad));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* ring = ring_all + warp * ST * kRgBoxBytes;
    uint64_t* bars = bars_all + warp * ST;
    const int n_st = kpad / kRgStageK;                       // boxes per unit
    // this warp's units: u = blockIdx.x + gridDim.x * (warp + warps_used * i)
    const int first_unit = blockIdx.x + gridDim.x * warp;
    const int unit_stride = gridDim.x * warps_used;
    const int my_units = (warp < warps_used && first_unit < units) ? (units - first_unit + unit_stride - 1) / unit_stride : 0;
    const uint32_t total = static_cast<uint32_t>(my_units) * n_st;   // boxes this warp consumes, in order

    if (lane == 0) {
        for (int s = 0; s < ST; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        if (warp == 0) tma_prefetch_desc(tmap_w);
    }
    __syncwarp();
    auto issue = [&](uint32_t idx) {       // box number idx of this warp's stream (lane 0 only)
        const int ui = idx / n_st, st = idx - ui * n_st;
        const int s = idx % ST;
        mbar_expect_tx(&bars[s], kRgBoxBytes);
        tma_load_2d(ring + s * kRgBoxBytes, tmap_w, &bars[s], st * 128, (first_unit + ui * unit_stride) * 8);
    };
    if (lane == 0)
        for (uint32_t i = 0; i < static_cast<uint32_t>(ST) && i < total; ++i) issue(i);

    // ---- activations into shared memory, in fragment order (all threads; overlaps the first boxes' flight) ----
    {
        const int words = kpad / 8;
        const int kwords = K / 8;
        for (int idx = threadIdx.x; idx < words * MPAD; idx += kRgThreads) {
            const int m = idx / words, w = idx - m * words;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < M && w < kwords) {
                const uint4 r = __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(m) * K) + w);
                // halves k0..k0+7 -> [k0, k0+4 | k0+1, k0+5 | k0+2, k0+6 | k0+3, k0+7]
                v.x = __byte_perm(r.x, r.z, 0x5410);
                v.y = __byte_perm(r.x, r.z, 0x7632);
                v.z = __byte_perm(r.y, r.w, 0x5410);
                v.w = __byte_perm(r.y, r.w, 0x7632);
            }
            const int sw = 2 * ((w >> 2) & 3);                 // the lane column (t) that reads this word, times two
            const int row = (m & 8) | ((m & 7) ^ sw);
            *reinterpret_cast<uint4*>(act + (static_cast<size_t>(w) * MPAD + row) * 16) = v;
        }
    }
    __syncthreads();
    if (my_units == 0) return;

    const __half2 bias = __float2half2_rn(zp_plus_1024);
    const int brow = (g >> 1) + ((g & 1) << 2);               // box row that holds operand column g
    const bool lo_ok = g < M, hi_ok = MPAD == 16 && g + 8 < M;
    const uint32_t act_lane = smem_u32(act) + ((g ^ (2 * t)) << 4);
    const uint32_t ring_lane = smem_u32(ring) + brow * 128;
    const int g_last = groups_per_row - 1;
    const int blocks128 = K / 128;

    uint32_t ci = 0;
    bool ok = true;
    for (int ui = 0; ui < my_units && ok; ++ui) {
        const int unit = first_unit + ui * unit_stride;
        const __half* srow = scales + static_cast<int64_t>(unit * 8 + brow) * groups_per_row;
        auto scale_of = [&](int blk) { return __ldg(srow + min(min(blk, blocks128 - 1) / group128, g_last)); };
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        // scales of the next two 128-wide blocks are fetched one box ahead of their use
        __half sc0 = scale_of(0), sc1 = scale_of(1);
        for (int st = 0; st < n_st; ++st, ++ci) {
            const int s = ci % ST;
            const __half nx0 = scale_of(2 * st + 2), nx1 = scale_of(2 * st + 3);
            if (!mbar_wait(&bars[s], (ci / ST) & 1, ST_WAIT_SMEM_FULL, st)) { ok = false; break; }
            const uint32_t box = ring_lane + s * kRgBoxBytes;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 wv = lds128(box + (((t + 4 * h) ^ brow) << 4));
                const __half2 s2 = __half2half2(h == 0 ? sc0 : sc1);
                const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
                const uint32_t abase = act_lane + static_cast<uint32_t>((st * 32 + h * 16 + 4 * t) * MPAD) * 16;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 al = make_uint4(0u, 0u, 0u, 0u), ah = make_uint4(0u, 0u, 0u, 0u);
                    if (lo_ok) al = lds128(abase + j * MPAD * 16);
                    if (hi_ok) ah = lds128(abase + j * MPAD * 16 + 128);
                    const uint32_t w = wd[j];
                    const uint32_t b0 = rg_pair(w, bias, s2), b1 = rg_pair(w >> 4, bias, s2);
                    const uint32_t b2 = rg_pair(w >> 8, bias, s2), b3 = rg_pair(w >> 12, bias, s2);
                    mma16816(acc, al.x, ah.x, al.y, ah.y, b0, b1);
                    mma16816(acc, al.z, ah.z, al.w, ah.w, b2, b3);
                }
            }
            sc0 = nx0; sc1 = nx1;
            __syncwarp();                                       // every lane has read the slot
            if (lane == 0 && ci + ST < total) issue(ci + ST);
        }
        if (!ok) break;
        // accumulator: (m = g + 8 * (r >> 1), operand column c = 2t + (r & 1)) -> weight row of that column
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int m = g + 8 * (r >> 1);
            const int c = 2 * t + (r & 1);
            const int nrow = (c >> 1) + ((c & 1) << 2);
            if (m < M) out[static_cast<int64_t>(m) * ldo + col_offset + unit * 8 + nrow] = __float2half_rn(acc[r]);
        }
    }
    if (!ok && lane == 0) {   // give boxes already in flight a bounded chance to land before the warp exits
        for (uint32_t i = ci + 1; i < total && i < ci + ST; ++i) (void)mbar_wait(&bars[i % ST], (i / ST) & 1, ST_WAIT_SMEM_FULL, -1);
    }
}

extern "C" __global__ void __launch_bounds__(kRgThreads, 1)
tb200_k_gemv_w4a16_ring_m8(const __grid_constant__ CUtensorMap tmap_w, const __half* a, const __half* scales, __half* out, int M,
                           int K, int kpad, int gpr, int group128, int64_t ldo, int64_t col_offset, float zp1024, int units,
                           int warps_used) {
    gemv_ring_body<8>(&tmap_w, a, scales, out, M, K, kpad, gpr, group128, ldo, col_offset, zp1024, units, warps_used);
}
extern "C" __global__ void __launch_bounds__(kRgThreads, 1)
tb200_k_gemv_w4a16_ring_m16(const __grid_constant__ CUtensorMap tmap_w, const __half* a, const __half* scales, __half* out, int M,
                            int K, int kpad, int gpr, int group128, int64_t ldo, int64_t col_offset, float zp1024, int units,
                            int warps_used) {
    gemv_ring_body<16>(&tmap_w, a, scales, out, M, K, kpad, gpr, group128, ldo, col_offset, zp1024, units, warps_used);
}

TB200_DEFINE_STATUS_HOOKS(gemv_ring)

namespace tb200 {

bool gemv_ring_fits(int64_t m, int64_t k) {
    const int64_t kpad = (k + kRgStageK - 1) / kRgStageK * kRgStageK;
    if (kpad > (1 << 20)) return false;
    return (m <= 8 ? RingCfg<8>::smem_bytes(static_cast<int>(kpad)) : RingCfg<16>::smem_bytes(static_cast<int>(kpad))) <= kRgMaxSmem;
}

// Host launcher used by tb200_gemm_w4a16 for m <= 16 when the activations fit in shared memory beside the
// rings (arguments already validated there; wp must be 16-byte aligned with a row pitch of k / 2 bytes).
int launch_gemv_w4a16_ring(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                           int64_t group, int zero_point, int64_t ldo, int64_t col_offset, cudaStream_t st) {
    const int kpad = static_cast<int>((k + kRgStageK - 1) / kRgStageK * kRgStageK);
    const int units = static_cast<int>(n / 8);
    const int sms = num_sms();
    const int grid = units < sms ? units : sms;
    int warps_used = (units + grid - 1) / grid;
    if (warps_used > kRgWarps) warps_used = kRgWarps;
    CUtensorMap tw;
    int rc = encode_tmap_2d(&tw, wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k / 2, k / 2, 8, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    static PerDeviceInt attr8, attr16;
    const float zp1024 = 1024.0f + static_cast<float>(zero_point);
    if (m <= 8) {
        const int smem = RingCfg<8>::smem_bytes(kpad);
        rc = ensure_max_smem(attr8, reinterpret_cast<const void*>(tb200_k_gemv_w4a16_ring_m8), kRgMaxSmem);
        if (rc != TB200_OK) return rc;
        tb200_k_gemv_w4a16_ring_m8<<<grid, kRgThreads, smem, st>>>(tw, static_cast<const __half*>(a), static_cast<const __half*>(scales),
                                                                  static_cast<__half*>(out), static_cast<int>(m), static_cast<int>(k), kpad,
                                                                  static_cast<int>(k / group), static_cast<int>(group / 128), ldo, col_offset,
                                                                  zp1024, units, warps_used);
    } else {
        const int smem = RingCfg<16>::smem_bytes(kpad);
        rc = ensure_max_smem(attr16, reinterpret_cast<const void*>(tb200_k_gemv_w4a16_ring_m16), kRgMaxSmem);
        if (rc != TB200_OK) return rc;
        tb200_k_gemv_w4a16_ring_m16<<<grid, kRgThreads, smem, st>>>(tw, static_cast<const __half*>(a), static_cast<const __half*>(scales),
                                                                   static_cast<__half*>(out), static_cast<int>(m), static_cast<int>(k), kpad,
                                                                   static_cast<int>(k / group), static_cast<int>(group / 128), ldo, col_offset,
                                                                   zp1024, units, warps_used);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

}  // namespace tb200
