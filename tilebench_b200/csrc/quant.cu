// FP8 e4m3 block quantiser (the step before the block-scaled GEMM): per [block_rows x 128] block
// scale = amax / 448 (1 for an all-zero block), q = e4m3(clamp(x / scale, +-448)), round to nearest even.
// Streaming and HBM-bound: 4 B read, 1 B written per element.
//   tb200_k_quant_fp8_1x128     half a warp per 1 x 128 block (activations): 8 elements per lane, 256-bit loads
//   tb200_k_quant_fp8_128x128   one CTA per 128 x 128 block (weights): 128 threads, one column strip each
//   tb200_k_quant_int4_g128     int4 group packing (the producer of the int4 dequant / W4A16 operands): half a
//                               warp per group of 128, 256-bit loads
// Every operation is an IEEE fp32 one (division by __fdiv_rn), so the result is bit-identical to the
// same formula evaluated with PyTorch ops.
#include "common.cuh"

#include <cuda_fp8.h>
#include <cuda_fp16.h>

namespace tb200 {
namespace {
constexpr float kFp8Max = 448.0f;

// four fp32 -> four e4m3 bytes; the two-value form compiles to the hardware cvt.rn.satfinite.e4m3x2.f32
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}
__device__ __forceinline__ float clamp448(float v) { return fminf(fmaxf(v, -kFp8Max), kFp8Max); }
}  // namespace
}  // namespace tb200

using namespace tb200;

// Half a warp per 1 x 128 block: each lane loads 8 consecutive floats with one 256-bit load and stores its
// 8 codes with one 64-bit store, so a warp quantises two consecutive blocks per pass.
extern "C" __global__ void __launch_bounds__(256)
tb200_k_quant_fp8_1x128(const float* __restrict__ x, uint2* __restrict__ q, float* __restrict__ scales,
                        int64_t total_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    const int64_t pairs = (total_blocks + 1) / 2;
    for (int64_t pr = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); pr < pairs; pr += warps) {
        const int64_t blk = 2 * pr + (lane >> 4);
        const bool valid = blk < total_blocks;                  // odd block count: the upper half-warp idles once
        float v[8];
        if (valid) {
            uint32_t r[8];
            asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "l"(x + blk * 128 + (lane & 15) * 8));
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within the half-warp
        const float s = amax > 0.f ? __fdiv_rn(amax, kFp8Max) : 1.0f;
        uint2 o;
        o.x = pack_e4m3x4(clamp448(__fdiv_rn(v[0], s)), clamp448(__fdiv_rn(v[1], s)), clamp448(__fdiv_rn(v[2], s)),
                          clamp448(__fdiv_rn(v[3], s)));
        o.y = pack_e4m3x4(clamp448(__fdiv_rn(v[4], s)), clamp448(__fdiv_rn(v[5], s)), clamp448(__fdiv_rn(v[6], s)),
                          clamp448(__fdiv_rn(v[7], s)));
        if (valid) {
            q[blk * 16 + (lane & 15)] = o;
            if ((lane & 15) == 0) scales[blk] = s;
        }
    }
}

// grid = (cols / 128, rows / 128); thread t owns 4 columns (t % 32) of 32 rows (t / 32).
extern "C" __global__ void __launch_bounds__(128)
tb200_k_quant_fp8_128x128(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                          int64_t cols) {
    __shared__ float wmax[4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * 128 + warp * 32;
    const int64_t col0 = static_cast<int64_t>(blockIdx.x) * 128 + lane * 4;
    float4 v[32];
    float amax = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        v[r] = __ldg(reinterpret_cast<const float4*>(x + (row0 + r) * cols + col0));
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[r].x), fabsf(v[r].y)), fmaxf(fabsf(v[r].z), fabsf(v[r].w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) wmax[warp] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
    const float s = amax > 0.f ? __fdiv_rn(amax, kFp8Max) : 1.0f;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        *reinterpret_cast<uint32_t*>(q + (row0 + r) * cols + col0) =
            pack_e4m3x4(clamp448(__fdiv_rn(v[r].x, s)), clamp448(__fdiv_rn(v[r].y, s)), clamp448(__fdiv_rn(v[r].z, s)),
                        clamp448(__fdiv_rn(v[r].w, s)));
    }
    if (threadIdx.x == 0) scales[static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x] = s;
}

// int4 group quantiser, group = 128, zero point 8:  s = fp16(amax / 7) (1 if that is zero),
// q = clamp(rint(x / float(s)) + 8, 0, 15), two values per byte with the even k in the low nibble —
// the layout tb200_dequant_int4_group and tb200_gemm_w4a16 read.  Each lane loads 8 consecutive floats
// (one 256-bit load); 16 lanes cover one group, so a warp quantises two consecutive groups per pass and
// writes 2 x 64 packed bytes.  IEEE division and rint: bit-identical to the same formula in PyTorch.
extern "C" __global__ void __launch_bounds__(256)
tb200_k_quant_int4_g128(const float* __restrict__ x, uint32_t* __restrict__ wp, __half* __restrict__ scales,
                        int64_t total_groups) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    const int64_t pairs = (total_groups + 1) / 2;
    for (int64_t pr = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); pr < pairs; pr += warps) {
        const int64_t grp = 2 * pr + (lane >> 4);
        const bool valid = grp < total_groups;                  // odd group count: the upper half-warp idles once
        float v[8];
        if (valid) {
            uint32_t r[8];
            asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "l"(x + grp * 128 + (lane & 15) * 8));
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within the half-warp
        __half s16 = __float2half_rn(__fdiv_rn(amax, 7.0f));
        if (__half2float(s16) == 0.f) s16 = __float2half_rn(1.0f);
        const float s = __half2float(s16);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float q = fminf(fmaxf(rintf(__fdiv_rn(v[i], s)) + 8.0f, 0.0f), 15.0f);
            packed |= static_cast<uint32_t>(static_cast<int>(q)) << (4 * i);
        }
        if (valid) {
            wp[grp * 16 + (lane & 15)] = packed;
            if ((lane & 15) == 0) scales[grp] = s16;
        }
    }
}

extern "C" int tb200_quantize_fp8_block(const float* x, void* q, float* scales, int64_t rows, int64_t cols,
                                        int block_rows, void* stream) {
    clear_error();
    if (!x || !q || !scales) return fail(TB200_ERR_ARG, "quantize_fp8_block: null pointer");
    if (rows <= 0 || cols <= 0 || cols % 128 != 0)
        return fail(TB200_ERR_ARG, "quantize_fp8_block: rows=%lld, cols=%lld (cols must be a positive multiple of 128)", (long long)rows, (long long)cols);
    if (block_rows != 1 && block_rows != 128) return fail(TB200_ERR_UNSUPPORTED, "quantize_fp8_block: block_rows %d (1 or 128)", block_rows);
    if (block_rows == 128 && rows % 128 != 0) return fail(TB200_ERR_ARG, "quantize_fp8_block: rows=%lld must be a multiple of 128 for 128x128 blocks", (long long)rows);
    if ((reinterpret_cast<uintptr_t>(x) & 31u) || (reinterpret_cast<uintptr_t>(q) & 7u))
        return fail(TB200_ERR_ALIGN, "quantize_fp8_block: x must be 32-byte and q 8-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (block_rows == 1) {
        const int64_t blocks = rows * (cols / 128);
        int64_t grid = ((blocks + 1) / 2 + 7) / 8;
        const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
        if (grid > cap) grid = cap;
        tb200_k_quant_fp8_1x128<<<static_cast<unsigned>(grid), 256, 0, st>>>(x, static_cast<uint2*>(q), scales, blocks);
    } else {
        if (cols / 128 > 0x7fffffff || rows / 128 > 65535) return fail(TB200_ERR_UNSUPPORTED, "quantize_fp8_block: matrix too large");
        dim3 grid(static_cast<unsigned>(cols / 128), static_cast<unsigned>(rows / 128));
        tb200_k_quant_fp8_128x128<<<grid, 128, 0, st>>>(x, static_cast<uint8_t*>(q), scales, cols);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_quantize_int4_group(const float* x, void* wp, void* scales, int64_t n, int64_t k, int64_t group,
                                         int zero_point, void* stream) {
    clear_error();
    if (!x || !wp || !scales) return fail(TB200_ERR_ARG, "quantize_int4_group: null pointer");
    if (n <= 0 || k <= 0) return fail(TB200_ERR_ARG, "quantize_int4_group: non-positive size n=%lld k=%lld", (long long)n, (long long)k);
    if (group != 128 || zero_point != 8)
        return fail(TB200_ERR_UNSUPPORTED, "quantize_int4_group: group=%lld zero_point=%d (only 128 / 8 are built)", (long long)group, zero_point);
    if (k % 128 != 0) return fail(TB200_ERR_ARG, "quantize_int4_group: k=%lld must be a multiple of the group size 128", (long long)k);
    if ((reinterpret_cast<uintptr_t>(x) & 31u) || (reinterpret_cast<uintptr_t>(wp) & 3u) || (reinterpret_cast<uintptr_t>(scales) & 1u))
        return fail(TB200_ERR_ALIGN, "quantize_int4_group: x must be 32-byte, wp 4-byte and scales 2-byte aligned");
    const int64_t groups = n * (k / 128);
    int64_t grid = ((groups + 1) / 2 + 7) / 8;
    const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    if (grid > cap) grid = cap;
    tb200_k_quant_int4_g128<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, static_cast<uint32_t*>(wp), static_cast<__half*>(scales), groups);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}
