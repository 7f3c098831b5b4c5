// Decode-sized W4A16 (m <= 16): weight streaming bound by HBM, not by the tensor pipe.
//
// With at most 16 activation rows the tcgen05 pipeline spends its time on hand-offs, so this shape
// gets its own kernel: every warp streams packed int4 rows straight from global memory with 128-bit
// loads, unpacks them in registers and feeds warp-level mma.sync.m16n8k16 (fp32 accumulate) with the
// activations as the 16-row operand.  No shared-memory staging, no split-K workspace, no second
// kernel: one CTA owns 32 weight rows, its 8 warps split K, and their partial sums are added in warp
// order through shared memory (deterministic).
//
// K order inside an MMA is free as long as both operands agree, so the operands are loaded in the
// order that makes every load contiguous: lane (g, t) of a warp (g = lane / 4, t = lane % 4) reads
// the 16 packed bytes [16t, 16t + 16) of weight row g of a tile — k = 32t .. 32t + 31 of the current
// 128-wide group — and in MMA step j (0..7) supplies k = 32t + 4j + {0,1} as the fragment's
// (2t, 2t+1) slots and k + {2,3} as its (2t+8, 2t+9) slots.  The activation fragment of the same lane
// is then 8 contiguous bytes of rows g and g + 8 at the same k, served by L1 (the whole [16, K]
// activation matrix is re-read by every warp and stays cached).
//
// Weights are rounded to fp16 after scaling — (q - zp) * s with one rounding, exactly the value the
// dequant kernel and the tensor-memory GEMM produce — so the result differs from theirs only by the
// fp32 summation order.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kGvWarps = 8;        // K is split over the warps of a CTA
constexpr int kGvThreads = 32 * kGvWarps;

// nibbles (2i, 2i+1) of the 16-bit field `x` -> fp16 pair ((q - zp) * s), one rounding
__device__ __forceinline__ uint32_t gv_pair(uint32_t x, uint32_t x_shr4, uint32_t sel, __half2 bias, __half2 s2) {
    uint32_t w = __byte_perm(x, x_shr4, sel);
    uint32_t h;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h) : "r"(w));
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h), bias), s2);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace
}  // namespace tb200

using namespace tb200;

// TILES = n8 tiles per warp (a CTA owns 8 * TILES weight rows).  More tiles reuse each activation
// fragment more often (L1 traffic per weight byte falls as 8 / TILES bytes), fewer tiles need fewer
// registers, so more CTAs are resident and more loads are in flight: 1 for m = 1, 4 for m up to 16.
// DEPTH = 128-wide K blocks of weights in flight per warp.
template <int TILES, int DEPTH>
__device__ __forceinline__ void gemv_w4a16_body(const __half* __restrict__ a, const uint8_t* __restrict__ wp,
                                                const __half* __restrict__ scales, __half* __restrict__ out, int M, int K,
                                                int groups_per_row, int group128, int64_t ldo, int64_t col_offset,
                                                float zp_plus_1024) {
    constexpr int ROWS = 8 * TILES;
    __shared__ float red[kGvWarps][32][TILES * 4 + 1];   // [warp][lane][tile * 4 + reg], padded against bank conflicts
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int G = K / 128;                       // 128-wide K blocks; this warp takes [gb, ge)
    const int gb = static_cast<int>(static_cast<int64_t>(warp) * G / kGvWarps);
    const int ge = static_cast<int>(static_cast<int64_t>(warp + 1) * G / kGvWarps);
    const __half2 bias = __float2half2_rn(zp_plus_1024);
    const int64_t wpitch = K / 2;
    // activation rows of this lane; rows >= M read as zero
    const bool lo_ok = g < M, hi_ok = g + 8 < M;
    const __half* a_lo = a + static_cast<int64_t>(lo_ok ? g : 0) * K + 32 * t;
    const __half* a_hi = a + static_cast<int64_t>(hi_ok ? g + 8 : 0) * K + 32 * t;
    const uint8_t* w_lane = wp + static_cast<int64_t>(n0 + g) * wpitch + 16 * t;
    const __half* s_lane = scales + static_cast<int64_t>(n0 + g) * groups_per_row;

    float acc[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[i][r] = 0.f;

    // ring of DEPTH blocks: slot u holds block (base + u); a slot is refilled as soon as it is consumed
    uint4 wq[DEPTH][TILES];
    __half sc[DEPTH][TILES];
    auto load_block = [&](int blk, uint4 (&w)[TILES], __half (&s)[TILES]) {
#pragma unroll
        for (int i = 0; i < TILES; ++i) {
            w[i] = __ldg(reinterpret_cast<const uint4*>(w_lane + static_cast<int64_t>(8 * i) * wpitch + blk * 64));
            s[i] = __ldg(s_lane + static_cast<int64_t>(8 * i) * groups_per_row + blk / group128);
        }
    };
#pragma unroll
    for (int u = 0; u < DEPTH; ++u)
        if (gb + u < ge) load_block(gb + u, wq[u], sc[u]);

    for (int base = gb; base < ge; base += DEPTH) {
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) {
            const int blk = base + u;
            if (blk >= ge) break;
            const int k0 = blk * 128;
            __half2 s2[TILES];
            uint4 wcur[TILES];
#pragma unroll
            for (int i = 0; i < TILES; ++i) { s2[i] = __half2half2(sc[u][i]); wcur[i] = wq[u][i]; }
            if (blk + DEPTH < ge) load_block(blk + DEPTH, wq[u], sc[u]);   // refill the slot just read
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint2 alo = make_uint2(0u, 0u), ahi = make_uint2(0u, 0u);
                if (lo_ok) alo = *reinterpret_cast<const uint2*>(a_lo + k0 + 4 * j);
                if (hi_ok) ahi = *reinterpret_cast<const uint2*>(a_hi + k0 + 4 * j);
                const uint32_t af[4] = {alo.x, ahi.x, alo.y, ahi.y};
#pragma unroll
                for (int i = 0; i < TILES; ++i) {
                    const uint32_t word = j < 2 ? wcur[i].x : (j < 4 ? wcur[i].y : (j < 6 ? wcur[i].z : wcur[i].w));
                    const uint32_t x = (j & 1) ? (word >> 16) : (word & 0xFFFFu);      // four nibbles: k + 0..3
                    const uint32_t xs = x >> 4;
                    const uint32_t b0 = gv_pair(x, xs, 0x0400, bias, s2[i]);           // (k+0, k+1)
                    const uint32_t b1 = gv_pair(x, xs, 0x0501, bias, s2[i]);           // (k+2, k+3)
                    mma16816(acc[i], af, b0, b1);
                }
            }
        }
    }

    // partial sums of the 8 warps, added in warp order
#pragma unroll
    for (int i = 0; i < TILES; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[warp][lane][i * 4 + r] = acc[i][r];
    __syncthreads();
    // accumulator fragment: tile i, lane (g, t), register r holds (m = g + 8 * (r >> 1), n = 8i + 2t + (r & 1))
    for (int o = threadIdx.x; o < 16 * ROWS; o += kGvThreads) {
        const int m = o / ROWS, n = o % ROWS;
        if (m >= M) continue;
        const int i = n >> 3, tt = (n & 7) >> 1, r = ((m >> 3) << 1) | (n & 1), ln = ((m & 7) << 2) | tt;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kGvWarps; ++w) sum += red[w][ln][i * 4 + r];
        out[static_cast<int64_t>(m) * ldo + col_offset + n0 + n] = __float2half_rn(sum);
    }
}

extern "C" __global__ void __launch_bounds__(kGvThreads, 2)
tb200_k_gemv_w4a16_t4(const __half* a, const uint8_t* wp, const __half* scales, __half* out, int M, int K, int gpr,
                      int group128, int64_t ldo, int64_t col_offset, float zp1024) {
    gemv_w4a16_body<4, 2>(a, wp, scales, out, M, K, gpr, group128, ldo, col_offset, zp1024);
}
extern "C" __global__ void __launch_bounds__(kGvThreads, 3)
tb200_k_gemv_w4a16_t2(const __half* a, const uint8_t* wp, const __half* scales, __half* out, int M, int K, int gpr,
                      int group128, int64_t ldo, int64_t col_offset, float zp1024) {
    gemv_w4a16_body<2, 3>(a, wp, scales, out, M, K, gpr, group128, ldo, col_offset, zp1024);
}
extern "C" __global__ void __launch_bounds__(kGvThreads, 4)
tb200_k_gemv_w4a16_t1(const __half* a, const uint8_t* wp, const __half* scales, __half* out, int M, int K, int gpr,
                      int group128, int64_t ldo, int64_t col_offset, float zp1024) {
    gemv_w4a16_body<1, 4>(a, wp, scales, out, M, K, gpr, group128, ldo, col_offset, zp1024);
}

namespace tb200 {

// Host launcher used by tb200_gemm_w4a16 for m <= 16 (arguments already validated there).
int launch_gemv_w4a16(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                      int64_t group, int zero_point, int64_t ldo, int64_t col_offset, cudaStream_t st) {
    const int tiles = m <= 2 ? 1 : (m <= 8 ? 2 : 4);
    const unsigned grid = static_cast<unsigned>(n / (8 * tiles));
    auto kern = tiles == 1 ? tb200_k_gemv_w4a16_t1 : (tiles == 2 ? tb200_k_gemv_w4a16_t2 : tb200_k_gemv_w4a16_t4);
    kern<<<grid, kGvThreads, 0, st>>>(static_cast<const __half*>(a), static_cast<const uint8_t*>(wp),
                                      static_cast<const __half*>(scales), static_cast<__half*>(out), static_cast<int>(m),
                                      static_cast<int>(k), static_cast<int>(k / group), static_cast<int>(group / 128), ldo,
                                      col_offset, 1024.0f + static_cast<float>(zero_point));
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

}  // namespace tb200
