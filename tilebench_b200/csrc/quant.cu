// FP8 e4m3 block quantiser (the step before the block-scaled GEMM): per [block_rows x 128] block
// scale = amax / 448 (1 for an all-zero block), q = e4m3(clamp(x / scale, +-448)), round to nearest even.
// Streaming and HBM-bound: 4 B read, 1 B written per element.
//   tb200_k_quant_fp8_1x128     one warp per 1 x 128 block (activations): 4 elements per lane
//   tb200_k_quant_fp8_128x128   one CTA per 128 x 128 block (weights): 128 threads, one column strip each
// Every operation is an IEEE fp32 one (division by __fdiv_rn), so the result is bit-identical to the
// same formula evaluated with PyTorch ops.
#include "common.cuh"

#include <cuda_fp8.h>

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

extern "C" __global__ void __launch_bounds__(256)
tb200_k_quant_fp8_1x128(const float4* __restrict__ x, uint32_t* __restrict__ q, float* __restrict__ scales,
                        int64_t total_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t blk = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < total_blocks;
         blk += warps) {
        const float4 v = __ldg(x + blk * 32 + lane);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float s = amax > 0.f ? __fdiv_rn(amax, kFp8Max) : 1.0f;
        q[blk * 32 + lane] = pack_e4m3x4(clamp448(__fdiv_rn(v.x, s)), clamp448(__fdiv_rn(v.y, s)),
                                         clamp448(__fdiv_rn(v.z, s)), clamp448(__fdiv_rn(v.w, s)));
        if (lane == 0) scales[blk] = s;
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

extern "C" int tb200_quantize_fp8_block(const float* x, void* q, float* scales, int64_t rows, int64_t cols,
                                        int block_rows, void* stream) {
    clear_error();
    if (!x || !q || !scales) return fail(TB200_ERR_ARG, "quantize_fp8_block: null pointer");
    if (rows <= 0 || cols <= 0 || cols % 128 != 0)
        return fail(TB200_ERR_ARG, "quantize_fp8_block: rows=%lld, cols=%lld (cols must be a positive multiple of 128)", (long long)rows, (long long)cols);
    if (block_rows != 1 && block_rows != 128) return fail(TB200_ERR_UNSUPPORTED, "quantize_fp8_block: block_rows %d (1 or 128)", block_rows);
    if (block_rows == 128 && rows % 128 != 0) return fail(TB200_ERR_ARG, "quantize_fp8_block: rows=%lld must be a multiple of 128 for 128x128 blocks", (long long)rows);
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3u)) return fail(TB200_ERR_ALIGN, "quantize_fp8_block: x must be 16-byte and q 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (block_rows == 1) {
        const int64_t blocks = rows * (cols / 128);
        int64_t grid = (blocks + 7) / 8;
        const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
        if (grid > cap) grid = cap;
        tb200_k_quant_fp8_1x128<<<static_cast<unsigned>(grid), 256, 0, st>>>(reinterpret_cast<const float4*>(x),
                                                                              static_cast<uint32_t*>(q), scales, blocks);
    } else {
        if (cols / 128 > 0x7fffffff || rows / 128 > 65535) return fail(TB200_ERR_UNSUPPORTED, "quantize_fp8_block: matrix too large");
        dim3 grid(static_cast<unsigned>(cols / 128), static_cast<unsigned>(rows / 128));
        tb200_k_quant_fp8_128x128<<<grid, 128, 0, st>>>(x, static_cast<uint8_t*>(q), scales, cols);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}
