// Streaming dequantisation kernels for sm_100a (HBM-bound):
//   tb200_k_dequant_int4_group   packed int4 + fp16 group scales   -> fp16
//   tb200_k_dequant_int8_rowwise int8 + fp32 row scale (+ post-mul) -> fp16 / bf16
//   tb200_k_weight_dequant_*     float X * S[i/T, j/T]              -> same dtype
// Shape of every vector kernel: a persistent grid (a multiple of the SM count) strides over
// 16-byte output chunks; each thread first issues UNROLL independent loads, then unpacks in
// registers and writes one 128-bit store per chunk, so every warp-level load and store is a
// single contiguous segment.  Kernels are extern "C" so profilers list them by a bare name.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// Launch shape of the streaming kernels: a grid that gives every CTA the same number of passes, sized against the
// SM's thread slots rather than against what is resident at once.  (Measured: capping the grid at the kernel's
// real occupancy — two CTAs per SM for the deep-unroll kernels — so that a single resident wave loops over all
// passes took the headline from 6.24 to 5.60 TB/s; the hardware's CTA scheduler refilling SMs as CTAs retire
// spreads the tail better than a fixed assignment does.)
inline unsigned grid_for(uint64_t work_items, int threads, int unroll) {
    uint64_t per_cta = static_cast<uint64_t>(threads) * unroll;
    uint64_t need = (work_items + per_cta - 1) / per_cta;
    uint64_t sms = static_cast<uint64_t>(num_sms());
    uint64_t cap = sms * (2048 / threads);
    if (need < 1) need = 1;
    if (need < 4 * sms) {
        // small inputs: spread the items over more CTAs (up to four per SM) instead of unrolling inside few of them;
        // the kernels skip the unroll steps that fall beyond the end, so any grid is valid
        uint64_t one_each = (work_items + threads - 1) / threads;
        uint64_t spread = one_each < 4 * sms ? one_each : 4 * sms;
        return static_cast<unsigned>(spread > need ? spread : need);
    }
    if (need <= cap) return static_cast<unsigned>(need);
    uint64_t passes = (need + cap - 1) / cap;
    return static_cast<unsigned>((need + passes - 1) / passes);
}
#define TB200_GRID_FOR(kern, work, threads, unroll) grid_for(work, threads, unroll)

// Two nibbles of one byte -> half2 (low nibble first), exact:  h = 0x6400 | q  is 1024 + q.
__device__ __forceinline__ __half2 nib_pair_to_half2(uint32_t lo_src, uint32_t hi_src, uint32_t sel) {
    // byte `sel&7` of lo_src lands in bits 0-7, the same byte of hi_src (= lo_src >> 4) in bits 16-23
    uint32_t w = __byte_perm(lo_src, hi_src, sel);
    uint32_t h;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h) : "r"(w));  // (w & m) | c
    return *reinterpret_cast<__half2*>(&h);
}

// 256-bit global accesses (sm_100): one instruction moves 32 bytes per thread, 1 KB per warp.  The
// streaming kernels below are bound by HBM, and HBM efficiency on this part rises with the bytes each
// thread has in flight and with stores that cover whole 32-byte sectors in one instruction.
__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ void stg256(void* p, const uint32_t (&r)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]),
                 "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
constexpr int kWideUnroll = 8;     // 256-bit loads in flight per thread
constexpr int kWideUnroll4 = 4;    // the int4 kernel writes 4x what it reads: fewer chunks, same output in flight

}  // namespace
}  // namespace tb200

using namespace tb200;

// out[r, c] = fp16((q - zp) * s[r, c/group]);  one thread-chunk = 4 packed bytes = 8 outputs.
template <int kUnroll>
__device__ __forceinline__ void dequant_int4_group_body(const uint32_t* __restrict__ wp, const __half* __restrict__ scales,
                                                        __half* __restrict__ out, uint32_t chunks_per_row,
                                                        uint32_t group_chunks, uint32_t groups_per_row,
                                                        uint64_t total_chunks, int64_t ldo, float zp_plus_1024) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    const __half2 bias = __float2half2_rn(zp_plus_1024);  // 1024 + zero_point, exact for 0..15
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * kUnroll) {
        uint32_t packed[kUnroll];
        __half sc[kUnroll];
        uint64_t off[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) {
                uint64_t row = c / chunks_per_row;
                uint32_t cc = static_cast<uint32_t>(c - row * chunks_per_row);
                packed[u] = __ldg(wp + c);
                sc[u] = __ldg(scales + row * groups_per_row + cc / group_chunks);
                off[u] = row * static_cast<uint64_t>(ldo) + static_cast<uint64_t>(cc) * 8;
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const uint32_t lo = packed[u], hi = packed[u] >> 4;
                const __half2 s2 = __half2half2(sc[u]);
                __half2 v[4];
                // selector: result byte0 = byte i of lo, byte2 = byte i of hi (index 4+i); others masked
                v[0] = nib_pair_to_half2(lo, hi, 0x0400);
                v[1] = nib_pair_to_half2(lo, hi, 0x0501);
                v[2] = nib_pair_to_half2(lo, hi, 0x0602);
                v[3] = nib_pair_to_half2(lo, hi, 0x0703);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = __hmul2(__hsub2(v[i], bias), s2);  // exact int, one rounding
                *reinterpret_cast<uint4*>(out + off[u]) = *reinterpret_cast<uint4*>(v);
            }
        }
    }
}

extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int4_group(const uint32_t* wp, const __half* scales, __half* out, uint32_t cpr, uint32_t gc,
                           uint32_t gpr, uint64_t total, int64_t ldo, float zp1024) {
    dequant_int4_group_body<4>(wp, scales, out, cpr, gc, gpr, total, ldo, zp1024);
}

// Wide variant: one thread-chunk = 16 packed bytes (one 128-bit load) = 32 outputs written by two
// 256-bit stores.  Needs k % 32 == 0, group % 32 == 0 and 32-byte aligned output rows.
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int4_group_wide(const uint4* __restrict__ wp, const __half* __restrict__ scales, __half* __restrict__ out,
                                uint32_t chunks_per_row, uint32_t group_chunks, uint32_t groups_per_row,
                                uint64_t total_chunks, int64_t ldo, float zp_plus_1024) {
    constexpr int U = kWideUnroll4;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    const __half2 bias = __float2half2_rn(zp_plus_1024);
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * U) {
        uint4 packed[U];
        __half sc[U];
        uint64_t off[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const uint64_t row = c / chunks_per_row;
                const uint32_t cc = static_cast<uint32_t>(c - row * chunks_per_row);
                packed[u] = __ldg(wp + c);
                sc[u] = __ldg(scales + row * groups_per_row + cc / group_chunks);
                off[u] = row * static_cast<uint64_t>(ldo) + static_cast<uint64_t>(cc) * 32;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const __half2 s2 = __half2half2(sc[u]);
                const uint32_t words[4] = {packed[u].x, packed[u].y, packed[u].z, packed[u].w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t o[8];
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const uint32_t lo = words[2 * h + w], hi = lo >> 4;
                        __half2 v[4];
                        v[0] = nib_pair_to_half2(lo, hi, 0x0400);
                        v[1] = nib_pair_to_half2(lo, hi, 0x0501);
                        v[2] = nib_pair_to_half2(lo, hi, 0x0602);
                        v[3] = nib_pair_to_half2(lo, hi, 0x0703);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[i] = __hmul2(__hsub2(v[i], bias), s2);          // exact int, one rounding
                            o[4 * w + i] = *reinterpret_cast<uint32_t*>(&v[i]);
                        }
                    }
                    stg256(out + off[u] + 16 * h, o);
                }
            }
        }
    }
}
// Any even k, any group that divides k: one output element per thread.
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int4_group_scalar(const uint8_t* __restrict__ wp, const __half* __restrict__ scales,
                                  __half* __restrict__ out, int64_t n, int64_t k, int64_t group, int zp,
                                  int64_t ldo) {
    const int64_t total = n * k;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        int64_t r = i / k, c = i - r * k;
        uint32_t b = wp[r * (k / 2) + c / 2];
        int q = (c & 1) ? (b >> 4) : (b & 15);
        float s = __half2float(scales[r * (k / group) + c / group]);
        out[r * ldo + c] = __float2half_rn(static_cast<float>(q - zp) * s);
    }
}

namespace {
// Exact int8 -> float without a convert instruction: place (b ^ 0x80) in the low mantissa byte of
// 2^23, giving 2^23 + b + 128, then subtract 2^23 + 128.
__device__ __forceinline__ float s8_to_float(uint32_t flipped, uint32_t byte_sel) {
    uint32_t bits = __byte_perm(flipped, 0x4B000000u, 0x7540u | byte_sel);
    return __uint_as_float(bits) - 8388736.0f;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}
}  // namespace

// out[r, c] = cast((float(w) * scale[r]) [* post]);  one thread-chunk = 8 int8 = 16 output bytes.
template <bool BF16, bool POST>
__device__ __forceinline__ void dequant_int8_rowwise_body(const uint2* __restrict__ w, const float* __restrict__ scale,
                                                          uint4* __restrict__ out, uint32_t chunks_per_row,
                                                          uint64_t total_chunks, float post) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * kUnroll) {
        uint2 raw[kUnroll];
        float sc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) {
                raw[u] = __ldg(w + c);
                sc[u] = __ldg(scale + c / chunks_per_row);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const uint32_t x0 = raw[u].x ^ 0x80808080u, x1 = raw[u].y ^ 0x80808080u;
                float f[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    f[i] = s8_to_float(x0, i);
                    f[4 + i] = s8_to_float(x1, i);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    f[i] = __fmul_rn(f[i], sc[u]);              // first fp32 rounding
                    if (POST) f[i] = __fmul_rn(f[i], post);     // second fp32 rounding (reference order)
                }
                uint4 o;
                o.x = pack2<BF16>(f[0], f[1]);
                o.y = pack2<BF16>(f[2], f[3]);
                o.z = pack2<BF16>(f[4], f[5]);
                o.w = pack2<BF16>(f[6], f[7]);
                out[c] = o;
            }
        }
    }
}

extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int8_rowwise_bf16(const uint2* w, const float* scale, uint4* out, uint32_t cpr, uint64_t total,
                                  float post) {
    dequant_int8_rowwise_body<true, false>(w, scale, out, cpr, total, post);
}
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int8_rowwise_f16(const uint2* w, const float* scale, uint4* out, uint32_t cpr, uint64_t total,
                                 float post) {
    dequant_int8_rowwise_body<false, false>(w, scale, out, cpr, total, post);
}
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int8_rowwise_bf16_post(const uint2* w, const float* scale, uint4* out, uint32_t cpr,
                                       uint64_t total, float post) {
    dequant_int8_rowwise_body<true, true>(w, scale, out, cpr, total, post);
}
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int8_rowwise_f16_post(const uint2* w, const float* scale, uint4* out, uint32_t cpr,
                                      uint64_t total, float post) {
    dequant_int8_rowwise_body<false, true>(w, scale, out, cpr, total, post);
}

// Wide variant: one thread-chunk = 32 int8 (one 256-bit load) = 64 output bytes (two 256-bit stores).
// Needs cols % 32 == 0 and 32-byte aligned w and out.
template <bool BF16, bool POST, int U>
__device__ __forceinline__ void dequant_int8_rowwise_wide_body(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                                               uint8_t* __restrict__ out, uint32_t chunks_per_row,
                                                               uint64_t total_chunks, float post) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * U) {
        uint32_t raw[U][8];
        float sc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
                ldg256(w + c * 32, raw[u]);
                sc[u] = __ldg(scale + c / chunks_per_row);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t o[8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t x = raw[u][4 * h + q] ^ 0x80808080u;
                        float f[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            f[i] = __fmul_rn(s8_to_float(x, i), sc[u]);          // first fp32 rounding
                            if (POST) f[i] = __fmul_rn(f[i], post);              // second fp32 rounding (reference order)
                        }
                        o[2 * q] = pack2<BF16>(f[0], f[1]);
                        o[2 * q + 1] = pack2<BF16>(f[2], f[3]);
                    }
                    stg256(out + c * 64 + 32 * h, o);
                }
            }
        }
    }
}
// kWideUnroll chunks in flight per thread for large inputs; 2 for mid-sized ones, where the deep variant
// would leave SMs without a CTA.
#define TB200_INT8_WIDE(name, BF16, POST, U)                                                                        \
    extern "C" __global__ void __launch_bounds__(kThreads)                                                         \
    name(const uint8_t* w, const float* scale, uint8_t* out, uint32_t cpr, uint64_t total, float post) {           \
        dequant_int8_rowwise_wide_body<BF16, POST, U>(w, scale, out, cpr, total, post);                            \
    }
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_bf16_wide, true, false, kWideUnroll)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_f16_wide, false, false, kWideUnroll)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_bf16_post_wide, true, true, kWideUnroll)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_f16_post_wide, false, true, kWideUnroll)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_bf16_wide2, true, false, 2)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_f16_wide2, false, false, 2)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_bf16_post_wide2, true, true, 2)
TB200_INT8_WIDE(tb200_k_dequant_int8_rowwise_f16_post_wide2, false, true, 2)

// Any cols: one element per thread.
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_dequant_int8_rowwise_scalar(const int8_t* __restrict__ w, const float* __restrict__ scale, void* out,
                                    int64_t rows, int64_t cols, int bf16, int use_post, float post) {
    const int64_t total = rows * cols;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        float v = __fmul_rn(static_cast<float>(w[i]), scale[i / cols]);
        if (use_post) v = __fmul_rn(v, post);
        if (bf16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
        else      reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
    }
}

// Y = X * S[i/T, j/T].  16-bit types: the fp32 product of two 11-bit (8-bit) significands is exact,
// so multiply in fp32 and round once — identical to a correctly rounded native multiply.
namespace {
template <int DT> struct Vec16;  // 16-byte chunk traits
template <> struct Vec16<TB200_DT_F32> {
    static constexpr int kElems = 4;
    // load_raw / scale: the load is issued with nothing depending on it, the conversion happens where the value is
    // used — a dependent instruction right behind the load would hold back the data loads queued after it
    __device__ static uint32_t load_raw(const void* s, uint64_t i) { return __float_as_uint(__ldg(reinterpret_cast<const float*>(s) + i)); }
    __device__ static float scale(uint32_t raw) { return __uint_as_float(raw); }
    __device__ static uint4 mul(uint4 x, float s) {
        float* f = reinterpret_cast<float*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __fmul_rn(f[i], s);
        return x;
    }
};
template <> struct Vec16<TB200_DT_F16> {
    static constexpr int kElems = 8;
    __device__ static uint32_t load_raw(const void* s, uint64_t i) { return __ldg(reinterpret_cast<const unsigned short*>(s) + i); }
    __device__ static float scale(uint32_t raw) { return __half2float(__ushort_as_half(static_cast<unsigned short>(raw))); }
    // one HMUL2 per two elements: a correctly rounded fp16 product, i.e. the exact fp32 product rounded once
    __device__ static uint4 mul(uint4 x, float s) {
        __half2* h = reinterpret_cast<__half2*>(&x);
        const __half2 s2 = __float2half2_rn(s);                 // s came from an fp16 value: exact
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __hmul2(h[i], s2);
        return x;
    }
};
template <> struct Vec16<TB200_DT_BF16> {
    static constexpr int kElems = 8;
    __device__ static uint32_t load_raw(const void* s, uint64_t i) { return __ldg(reinterpret_cast<const unsigned short*>(s) + i); }
    __device__ static float scale(uint32_t raw) { return __uint_as_float(raw << 16); }      // bf16 -> fp32 is a 16-bit shift
    // one bf16x2 multiply per two elements (correctly rounded: the exact fp32 product rounded once)
    __device__ static uint4 mul(uint4 x, float s) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
        const __nv_bfloat162 s2 = __float2bfloat162_rn(s);      // s came from a bf16 value: exact
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __hmul2(h[i], s2);
        return x;
    }
};

template <int DT>
__device__ __forceinline__ void weight_dequant_body(const uint4* __restrict__ x, const void* __restrict__ s,
                                                    uint4* __restrict__ y, uint32_t chunks_per_row,
                                                    uint32_t tile_chunks, uint32_t tile_rows, uint32_t s_cols,
                                                    uint64_t total_chunks) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * kUnroll) {
        uint4 raw[kUnroll];
        uint32_t sc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) {
                uint64_t row = c / chunks_per_row;
                uint32_t cc = static_cast<uint32_t>(c - row * chunks_per_row);
                raw[u] = __ldg(x + c);
                sc[u] = Vec16<DT>::load_raw(s, (row / tile_rows) * s_cols + cc / tile_chunks);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint64_t c = base + u * stride;
            if (c < total_chunks) y[c] = Vec16<DT>::mul(raw[u], Vec16<DT>::scale(sc[u]));
        }
    }
}

// Wide variant: one thread-chunk = 32 bytes in, 32 bytes out (256-bit load and store); the scale is
// constant over a chunk because the tile width is a multiple of the chunk width.
template <int DT, int U>
__device__ __forceinline__ void weight_dequant_wide_body(const uint8_t* __restrict__ x, const void* __restrict__ s,
                                                         uint8_t* __restrict__ y, uint32_t chunks_per_row,
                                                         uint32_t tile_chunks, uint32_t tile_rows, uint32_t s_cols,
                                                         uint64_t total_chunks) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    for (uint64_t base = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; base < total_chunks;
         base += stride * U) {
        uint32_t raw[U][8];
        uint32_t sc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const uint64_t row = c / chunks_per_row;
                const uint32_t cc = static_cast<uint32_t>(c - row * chunks_per_row);
                ldg256(x + c * 32, raw[u]);
                sc[u] = Vec16<DT>::load_raw(s, (row / tile_rows) * s_cols + cc / tile_chunks);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t c = base + u * stride;
            if (c < total_chunks) {
                const float scale = Vec16<DT>::scale(sc[u]);
                const uint4 lo = Vec16<DT>::mul(make_uint4(raw[u][0], raw[u][1], raw[u][2], raw[u][3]), scale);
                const uint4 hi = Vec16<DT>::mul(make_uint4(raw[u][4], raw[u][5], raw[u][6], raw[u][7]), scale);
                const uint32_t o[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                stg256(y + c * 32, o);
            }
        }
    }
}
}  // namespace

#define TB200_WDQ_WIDE(name, DT, U)                                                                                 \
    extern "C" __global__ void __launch_bounds__(kThreads)                                                         \
    name(const uint8_t* x, const void* s, uint8_t* y, uint32_t cpr, uint32_t tc, uint32_t tr, uint32_t sc,         \
         uint64_t total) {                                                                                         \
        weight_dequant_wide_body<DT, U>(x, s, y, cpr, tc, tr, sc, total);                                          \
    }
TB200_WDQ_WIDE(tb200_k_weight_dequant_f32_wide, TB200_DT_F32, kWideUnroll)
TB200_WDQ_WIDE(tb200_k_weight_dequant_f16_wide, TB200_DT_F16, kWideUnroll)
TB200_WDQ_WIDE(tb200_k_weight_dequant_bf16_wide, TB200_DT_BF16, kWideUnroll)
TB200_WDQ_WIDE(tb200_k_weight_dequant_f32_wide2, TB200_DT_F32, 2)
TB200_WDQ_WIDE(tb200_k_weight_dequant_f16_wide2, TB200_DT_F16, 2)
TB200_WDQ_WIDE(tb200_k_weight_dequant_bf16_wide2, TB200_DT_BF16, 2)

extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_weight_dequant_f32(const uint4* x, const void* s, uint4* y, uint32_t cpr, uint32_t tc, uint32_t tr,
                           uint32_t sc, uint64_t total) {
    weight_dequant_body<TB200_DT_F32>(x, s, y, cpr, tc, tr, sc, total);
}
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_weight_dequant_f16(const uint4* x, const void* s, uint4* y, uint32_t cpr, uint32_t tc, uint32_t tr,
                           uint32_t sc, uint64_t total) {
    weight_dequant_body<TB200_DT_F16>(x, s, y, cpr, tc, tr, sc, total);
}
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_weight_dequant_bf16(const uint4* x, const void* s, uint4* y, uint32_t cpr, uint32_t tc, uint32_t tr,
                            uint32_t sc, uint64_t total) {
    weight_dequant_body<TB200_DT_BF16>(x, s, y, cpr, tc, tr, sc, total);
}

// Any m, n, tile: one element per thread.
extern "C" __global__ void __launch_bounds__(kThreads)
tb200_k_weight_dequant_scalar(const void* __restrict__ x, const void* __restrict__ s, void* __restrict__ y,
                              int64_t m, int64_t n, int64_t tile, int64_t s_cols, int dtype) {
    const int64_t total = m * n;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        int64_t r = i / n, c = i - r * n;
        int64_t si = (r / tile) * s_cols + c / tile;
        if (dtype == TB200_DT_F32) {
            reinterpret_cast<float*>(y)[i] =
                __fmul_rn(reinterpret_cast<const float*>(x)[i], reinterpret_cast<const float*>(s)[si]);
        } else if (dtype == TB200_DT_F16) {
            float v = __fmul_rn(__half2float(reinterpret_cast<const __half*>(x)[i]),
                                __half2float(reinterpret_cast<const __half*>(s)[si]));
            reinterpret_cast<__half*>(y)[i] = __float2half_rn(v);
        } else {
            float v = __fmul_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]),
                                __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(s)[si]));
            reinterpret_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
extern "C" int tb200_dequant_int4_group(const void* wp, const void* scales, void* out, int64_t n, int64_t k,
                                        int64_t group, int zero_point, int64_t ldo, void* stream) {
    clear_error();
    if (!wp || !scales || !out) return fail(TB200_ERR_ARG, "dequant_int4_group: null pointer");
    if (n < 0 || k < 0) return fail(TB200_ERR_ARG, "dequant_int4_group: negative size n=%lld k=%lld", (long long)n, (long long)k);
    if (group <= 0 || (k % 2) != 0 || (k % group) != 0)
        return fail(TB200_ERR_ARG, "dequant_int4_group: k=%lld must be even and a multiple of group=%lld", (long long)k, (long long)group);
    if (zero_point < 0 || zero_point > 15) return fail(TB200_ERR_ARG, "dequant_int4_group: zero_point %d outside 0..15", zero_point);
    if (ldo < k) return fail(TB200_ERR_ARG, "dequant_int4_group: ldo=%lld < k=%lld", (long long)ldo, (long long)k);
    if (n == 0 || k == 0) return TB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = (group % 8 == 0) && (ldo % 8 == 0) && aligned16(out) &&
                     ((reinterpret_cast<uintptr_t>(wp) & 3u) == 0) && (k / 8 < (1ll << 32));
    const bool wide = (group % 32 == 0) && (ldo % 16 == 0) && ((reinterpret_cast<uintptr_t>(out) & 31u) == 0) &&
                      aligned16(wp) && (k / 32 < (1ll << 32));
    if (wide) {
        const uint64_t total = static_cast<uint64_t>(n) * static_cast<uint64_t>(k / 32);
        const unsigned grid = TB200_GRID_FOR(tb200_k_dequant_int4_group_wide, total, kThreads, kWideUnroll4);
        tb200_k_dequant_int4_group_wide<<<grid, kThreads, 0, st>>>(
            static_cast<const uint4*>(wp), static_cast<const __half*>(scales), static_cast<__half*>(out),
            static_cast<uint32_t>(k / 32), static_cast<uint32_t>(group / 32), static_cast<uint32_t>(k / group), total,
            ldo, 1024.0f + static_cast<float>(zero_point));
    } else if (vec) {
        uint64_t total = static_cast<uint64_t>(n) * static_cast<uint64_t>(k / 8);
        unsigned grid = TB200_GRID_FOR(tb200_k_dequant_int4_group, total, kThreads, kUnroll);
        tb200_k_dequant_int4_group<<<grid, kThreads, 0, st>>>(
            static_cast<const uint32_t*>(wp), static_cast<const __half*>(scales), static_cast<__half*>(out),
            static_cast<uint32_t>(k / 8), static_cast<uint32_t>(group / 8), static_cast<uint32_t>(k / group), total,
            ldo, 1024.0f + static_cast<float>(zero_point));
    } else {
        unsigned grid = TB200_GRID_FOR(tb200_k_dequant_int4_group_scalar, static_cast<uint64_t>(n) * k, kThreads, 1);
        tb200_k_dequant_int4_group_scalar<<<grid, kThreads, 0, st>>>(
            static_cast<const uint8_t*>(wp), static_cast<const __half*>(scales), static_cast<__half*>(out), n, k,
            group, zero_point, ldo);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_dequant_int8_rowwise(const void* w, const float* scale, void* out, int64_t rows, int64_t cols,
                                          int out_dtype, int use_post, float post, void* stream) {
    clear_error();
    if (!w || !scale || !out) return fail(TB200_ERR_ARG, "dequant_int8_rowwise: null pointer");
    if (rows < 0 || cols < 0) return fail(TB200_ERR_ARG, "dequant_int8_rowwise: negative size");
    if (out_dtype != TB200_DT_F16 && out_dtype != TB200_DT_BF16)
        return fail(TB200_ERR_UNSUPPORTED, "dequant_int8_rowwise: out_dtype %d (want F16 or BF16)", out_dtype);
    if (rows == 0 || cols == 0) return TB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = out_dtype == TB200_DT_BF16;
    const bool vec = (cols % 8 == 0) && aligned16(out) && ((reinterpret_cast<uintptr_t>(w) & 7u) == 0) &&
                     (cols / 8 < (1ll << 32));
    const bool wide = (cols % 32 == 0) && ((reinterpret_cast<uintptr_t>(out) & 31u) == 0) &&
                      ((reinterpret_cast<uintptr_t>(w) & 31u) == 0) && (cols / 32 < (1ll << 32));
    const uint64_t wide_total = static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols / 32);
    const uint64_t sms = static_cast<uint64_t>(num_sms());
    if (wide && wide_total >= sms * kThreads * 2) {
        // deep variant once it still gives every SM two CTAs, else two chunks per thread
        const bool deep = wide_total >= 2 * sms * kThreads * kWideUnroll;
        auto kern = deep ? (bf16 ? (use_post ? tb200_k_dequant_int8_rowwise_bf16_post_wide : tb200_k_dequant_int8_rowwise_bf16_wide)
                                 : (use_post ? tb200_k_dequant_int8_rowwise_f16_post_wide : tb200_k_dequant_int8_rowwise_f16_wide))
                         : (bf16 ? (use_post ? tb200_k_dequant_int8_rowwise_bf16_post_wide2 : tb200_k_dequant_int8_rowwise_bf16_wide2)
                                 : (use_post ? tb200_k_dequant_int8_rowwise_f16_post_wide2 : tb200_k_dequant_int8_rowwise_f16_wide2));
        const unsigned grid = TB200_GRID_FOR(kern, wide_total, kThreads, deep ? kWideUnroll : 2);
        kern<<<grid, kThreads, 0, st>>>(static_cast<const uint8_t*>(w), scale, static_cast<uint8_t*>(out),
                                        static_cast<uint32_t>(cols / 32), wide_total, post);
    } else if (vec) {
        uint64_t total = static_cast<uint64_t>(rows) * static_cast<uint64_t>(cols / 8);
        auto kern = bf16 ? (use_post ? tb200_k_dequant_int8_rowwise_bf16_post : tb200_k_dequant_int8_rowwise_bf16)
                         : (use_post ? tb200_k_dequant_int8_rowwise_f16_post : tb200_k_dequant_int8_rowwise_f16);
        unsigned grid = TB200_GRID_FOR(kern, total, kThreads, kUnroll);
        kern<<<grid, kThreads, 0, st>>>(static_cast<const uint2*>(w), scale, static_cast<uint4*>(out),
                                        static_cast<uint32_t>(cols / 8), total, post);
    } else {
        unsigned grid = TB200_GRID_FOR(tb200_k_dequant_int8_rowwise_scalar, static_cast<uint64_t>(rows) * cols, kThreads, 1);
        tb200_k_dequant_int8_rowwise_scalar<<<grid, kThreads, 0, st>>>(static_cast<const int8_t*>(w), scale, out,
                                                                       rows, cols, bf16 ? 1 : 0, use_post, post);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_weight_dequant_block(const void* x, const void* s, void* y, int64_t m, int64_t n, int64_t tile,
                                          int dtype, void* stream) {
    clear_error();
    if (!x || !s || !y) return fail(TB200_ERR_ARG, "weight_dequant_block: null pointer");
    if (m < 0 || n < 0 || tile <= 0) return fail(TB200_ERR_ARG, "weight_dequant_block: bad size m=%lld n=%lld tile=%lld", (long long)m, (long long)n, (long long)tile);
    if (dtype != TB200_DT_F32 && dtype != TB200_DT_F16 && dtype != TB200_DT_BF16)
        return fail(TB200_ERR_UNSUPPORTED, "weight_dequant_block: dtype %d", dtype);
    if (m == 0 || n == 0) return TB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t s_cols = (n + tile - 1) / tile;
    const int elems = dtype == TB200_DT_F32 ? 4 : 8;
    const bool vec = (n % elems == 0) && (tile % elems == 0) && aligned16(x) && aligned16(y) &&
                     (n / elems < (1ll << 32)) && (tile < (1ll << 32)) && (s_cols < (1ll << 32));
    const bool wide = (n % (2 * elems) == 0) && (tile % (2 * elems) == 0) && ((reinterpret_cast<uintptr_t>(x) & 31u) == 0) &&
                      ((reinterpret_cast<uintptr_t>(y) & 31u) == 0) && (n / (2 * elems) < (1ll << 32)) &&
                      (tile < (1ll << 32)) && (s_cols < (1ll << 32));
    const uint64_t wide_total = static_cast<uint64_t>(m) * static_cast<uint64_t>(n / (2 * elems));
    const uint64_t sms = static_cast<uint64_t>(num_sms());
    if (wide && wide_total >= sms * kThreads * 2) {
        const bool deep = wide_total >= 2 * sms * kThreads * kWideUnroll;
        auto kern = deep ? (dtype == TB200_DT_F32 ? tb200_k_weight_dequant_f32_wide
                            : dtype == TB200_DT_F16 ? tb200_k_weight_dequant_f16_wide : tb200_k_weight_dequant_bf16_wide)
                         : (dtype == TB200_DT_F32 ? tb200_k_weight_dequant_f32_wide2
                            : dtype == TB200_DT_F16 ? tb200_k_weight_dequant_f16_wide2 : tb200_k_weight_dequant_bf16_wide2);
        const unsigned grid = TB200_GRID_FOR(kern, wide_total, kThreads, deep ? kWideUnroll : 2);
        kern<<<grid, kThreads, 0, st>>>(static_cast<const uint8_t*>(x), s, static_cast<uint8_t*>(y),
                                        static_cast<uint32_t>(n / (2 * elems)), static_cast<uint32_t>(tile / (2 * elems)),
                                        static_cast<uint32_t>(tile), static_cast<uint32_t>(s_cols), wide_total);
    } else if (vec) {
        uint64_t total = static_cast<uint64_t>(m) * static_cast<uint64_t>(n / elems);
        auto kern = dtype == TB200_DT_F32 ? tb200_k_weight_dequant_f32
                    : dtype == TB200_DT_F16 ? tb200_k_weight_dequant_f16 : tb200_k_weight_dequant_bf16;
        unsigned grid = TB200_GRID_FOR(kern, total, kThreads, kUnroll);
        kern<<<grid, kThreads, 0, st>>>(static_cast<const uint4*>(x), s, static_cast<uint4*>(y),
                                        static_cast<uint32_t>(n / elems), static_cast<uint32_t>(tile / elems),
                                        static_cast<uint32_t>(tile), static_cast<uint32_t>(s_cols), total);
    } else {
        unsigned grid = TB200_GRID_FOR(tb200_k_weight_dequant_scalar, static_cast<uint64_t>(m) * n, kThreads, 1);
        tb200_k_weight_dequant_scalar<<<grid, kThreads, 0, st>>>(x, s, y, m, n, tile, s_cols, dtype);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}
