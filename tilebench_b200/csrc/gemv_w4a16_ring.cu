// Decode-sized W4A16 (m <= 16), streaming form: one persistent CTA per SM, every warp its own TMA ring.
//
// The weight stream (n * k / 2 bytes) is all that matters at this size, and it only runs at HBM speed when
// enough bytes are in flight: bandwidth x latency is about 35 KB per SM on this part.  Register-staged loads
// cannot hold that much, so the packed rows travel by TMA: a work unit is 16 weight rows over the whole K,
// owned by a PAIR of warps (each takes one half of K; the upper half hands its partial sums to the lower one
// through shared memory, so the summation order is fixed and no workspace is needed), and each warp keeps a
// ring of boxes of [16 rows x 128 bytes] (256 values of k, 128-byte swizzle) in flight for itself — lane 0
// re-arms a slot and issues the next box as soon as the warp has read it.
//
// The arithmetic is warp-level mma.sync.m16n8k16 (fp16 in, fp32 accumulate) with the 16 WEIGHT rows as the
// 16-row operand and up to 8 activation rows as the 8-column operand (a second MMA covers rows 8..15).  What
// shaped the loop, measured with the profiler's pipe counters on earlier forms of this kernel: it is bound by
// instruction issue, not by memory (the same time with the weights resident in L2), and more than half of the
// instructions were register moves and per-box bookkeeping.  Hence:
//   * the unpacked weights are the operand whose four registers are COMPUTED (no moves to line them up), and
//     the activations are the operand that comes straight out of one LDS.128 as two aligned register pairs;
//   * K order inside an MMA is free as long as both operands agree: a lane reads 16 contiguous packed bytes
//     (one LDS.128 per row, bank-conflict free under the swizzle because operand rows g / g + 8 sit in box rows
//     g/2 (+4 for odd g) and that + 8), and a 32-bit word of 8 nibbles is unpacked as the pairs (i, i + 4):
//     (w & 0x000f000f) | 0x6400 is 1024 + q, (w & 0x00f000f0) | 0x6400 is 1024 + 16 q, and the same two masks
//     on w >> 8 — one shift and four LOP3 per word; "- zero point" is one exact HADD2 resp. HFMA2 (x / 16 - 64
//     - zp), the scale one HMUL2 with a single rounding;
//   * the activations are laid out once per CTA in shared memory in exactly that order ([k0, k0+4, k0+1, k0+5,
//     k0+2, k0+6, k0+3, k0+7] per word, word-major, rows XOR-swizzled against bank conflicts); rows beyond m
//     are zeros, so the loop loads unconditionally;
//   * nothing on the streaming path divides: box, slot, phase and scale-group indices advance by increments.
// Weights are rounded to fp16 after scaling — fp16((q - zp) * s), one rounding, the value the dequant kernel
// and the tensor-memory GEMM produce.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kRgWarps = 14;                  // 7 pairs; pair p uses named barrier p + 1
constexpr int kRgThreads = 32 * kRgWarps;
constexpr int kRgRows = 16;                   // weight rows per unit
constexpr int kRgBoxBytes = kRgRows * 128;    // one ring slot: 16 rows x 128 packed bytes = 256 k
constexpr int kRgStageK = 256;

template <int MPAD> struct RingCfg {
    static constexpr int kStages = MPAD == 8 ? 5 : 2;
    static constexpr int kAcc = MPAD == 8 ? 4 : 8;                      // fp32 sums per lane
    static constexpr int kRingBytes = kRgWarps * kStages * kRgBoxBytes;
    static constexpr int kBarBytes = kRgWarps * kStages * 8;
    static constexpr int kRedBytes = (kRgWarps / 2) * 2 * 32 * kAcc * 4;   // per pair: two buffers of kAcc floats per lane
    // activations: (k / 8) words x MPAD rows x 16 bytes
    static constexpr int act_bytes(int kpad) { return kpad / 8 * MPAD * 16; }
    static constexpr int smem_bytes(int kpad) { return 1024 + kRingBytes + kRedBytes + act_bytes(kpad) + kBarBytes; }
};
constexpr int kRgMaxSmem = 232448;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One packed word (nibbles n0..n7 at bits 4i) -> four fp16 pairs (n_i, n_{i+4}), i = 0..3, each fp16((q - zp) * s).
// bias_lo = 1024 + zp (for 1024 + q), bias_hi = -(64 + zp) (for (1024 + 16 q) / 16): both subtractions are exact.
__device__ __forceinline__ void unpack_word(uint32_t w, __half2 bias_lo, __half2 bias_hi, __half2 sixteenth, __half2 s2,
                                            uint32_t& p0, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
    const uint32_t w8 = w >> 8;
    uint32_t h0, h1, h2, h3;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h0) : "r"(w));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(h1) : "r"(w));
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h2) : "r"(w8));
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(h3) : "r"(w8));
    const __half2 v0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h0), bias_lo), s2);
    const __half2 v1 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&h1), sixteenth, bias_hi), s2);
    const __half2 v2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h2), bias_lo), s2);
    const __half2 v3 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&h3), sixteenth, bias_hi), s2);
    p0 = *reinterpret_cast<const uint32_t*>(&v0);
    p1 = *reinterpret_cast<const uint32_t*>(&v1);
    p2 = *reinterpret_cast<const uint32_t*>(&v2);
    p3 = *reinterpret_cast<const uint32_t*>(&v3);
}

template <int OFF>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

template <int MPAD>
__device__ __forceinline__ void gemv_ring_body(const CUtensorMap* __restrict__ tmap_w, const __half* __restrict__ a,
                                               const __half* __restrict__ scales, __half* __restrict__ out, int M, int K, int kpad,
                                               int groups_per_row, int group128, int64_t ldo, int64_t col_offset, float zp,
                                               int units, int pairs_used) {
    using Cfg = RingCfg<MPAD>;
    constexpr int ST = Cfg::kStages;
    constexpr int NACC = Cfg::kAcc;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring_all = smem;
    float* red_all = reinterpret_cast<float*>(smem + Cfg::kRingBytes);
    uint8_t* act = smem + Cfg::kRingBytes + Cfg::kRedBytes;
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(act + Cfg::act_bytes(kpad));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rt_zero = static_cast<uint32_t>(K) >> 31;    // 0, but not known to be before the kernel runs
    const int g = lane >> 2, t = lane & 3;
    const int pair = warp >> 1, kh = warp & 1;                // kh: which half of K this warp sums
    uint8_t* ring = ring_all + warp * ST * kRgBoxBytes;
    uint64_t* bars = bars_all + warp * ST;
    const int n_st = kpad / kRgStageK;                       // boxes per unit over the whole K
    const int box_lo = (kh * n_st) >> 1, box_hi = ((kh + 1) * n_st) >> 1;
    const int my_boxes = box_hi - box_lo;                     // per unit (0 for the lower half when n_st == 1)
    // this pair's units: u = blockIdx.x + gridDim.x * (pair + pairs_used * i)
    const int first_unit = blockIdx.x + gridDim.x * pair;
    const int unit_stride = gridDim.x * pairs_used;
    const int my_units = (pair < pairs_used && first_unit < units) ? (units - first_unit + unit_stride - 1) / unit_stride : 0;
    const uint32_t total = static_cast<uint32_t>(my_units) * my_boxes;   // boxes this warp consumes, in order

    if (lane == 0) {
        for (int s = 0; s < ST; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        if (warp == 0) tma_prefetch_desc(tmap_w);
    }
    __syncwarp();
    // The warp's stream of boxes: (unit 0, box lo), ... (unit 0, box hi - 1), (unit 1, box lo), ...  Lane 0 runs ST
    // boxes ahead of the consumer.
    uint32_t issued = 0;
    int iss_x = box_lo * 128, iss_y = first_unit * kRgRows, iss_slot = 0;
    // `landed` is a zero derived (in hardware) from words just loaded out of the slot being refilled: the copy's
    // coordinate depends on it, so the refill cannot be issued while those loads are still in flight.
    auto issue = [&](uint32_t landed = 0u) {                    // lane 0 only
        mbar_expect_tx(&bars[iss_slot], kRgBoxBytes);
        tma_load_2d(ring + iss_slot * kRgBoxBytes, tmap_w, &bars[iss_slot], iss_x + static_cast<int>(landed), iss_y);
        ++issued;
        iss_slot = iss_slot + 1 == ST ? 0 : iss_slot + 1;
        iss_x += 128;
        if (iss_x == box_hi * 128) { iss_x = box_lo * 128; iss_y += unit_stride * kRgRows; }
    };
    if (lane == 0)
        while (issued < static_cast<uint32_t>(ST) && issued < total) issue();

    // ---- activations into shared memory, in fragment order (all threads; overlaps the first boxes' flight) ----
    // Rows m >= M (up to MPAD) and words beyond K are written as zeros, so the MMA loop loads unconditionally.
    {
        const int words = kpad / 8;
        const int kwords = K / 8;
        auto put = [&](int m, int w, uint4 r) {
            uint4 v;                                           // halves k0..k0+7 -> [k0, k0+4 | k0+1, k0+5 | k0+2, k0+6 | k0+3, k0+7]
            v.x = __byte_perm(r.x, r.z, 0x5410);
            v.y = __byte_perm(r.x, r.z, 0x7632);
            v.z = __byte_perm(r.y, r.w, 0x5410);
            v.w = __byte_perm(r.y, r.w, 0x7632);
            const int sw = 2 * ((w >> 2) & 3);                 // the lane column (t) that reads this word, times two
            const int row = (m & 8) | ((m & 7) ^ sw);
            *reinterpret_cast<uint4*>(act + (static_cast<size_t>(w) * MPAD + row) * 16) = v;
        };
        // real rows: eight independent loads in flight per thread, so their latency is paid once per batch
        constexpr int U = 8;
        const int real = M * kwords;
        for (int base = threadIdx.x; base < real; base += kRgThreads * U) {
            uint4 r[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * kRgThreads;
                if (idx < real) {
                    const int m = idx / kwords, w = idx - m * kwords;
                    r[u] = __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(m) * K) + w);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * kRgThreads;
                if (idx < real) {
                    const int m = idx / kwords;
                    put(m, idx - m * kwords, r[u]);
                }
            }
        }
        // zero rows m >= M, and the words beyond K of every row
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        for (int idx = threadIdx.x; idx < (MPAD - M) * words; idx += kRgThreads) put(M + idx / words, idx % words, zero);
        for (int idx = threadIdx.x; idx < M * (words - kwords); idx += kRgThreads) put(idx / (words - kwords), kwords + idx % (words - kwords), zero);
    }
    __syncthreads();
    if (my_units == 0) return;                                  // whole pairs leave together: no one waits for them

    const __half2 bias_lo = __float2half2_rn(1024.0f + zp);     // 1024 + q       -> q - zp
    const __half2 bias_hi = __float2half2_rn(-(64.0f + zp));    // (1024 + 16 q) / 16 = 64 + q -> q - zp
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    const int brow = (g >> 1) + ((g & 1) << 2);               // box rows brow and brow + 8 hold operand rows g and g + 8
    constexpr uint32_t kActStage = 32u * MPAD * 16u;            // bytes of activation words per box (32 words)
    const uint32_t act_lane = smem_u32(act) + ((g ^ (2 * t)) << 4) + static_cast<uint32_t>(4 * t * MPAD) * 16 +
                              static_cast<uint32_t>(box_lo) * kActStage;
    const uint32_t woff0 = brow * 128 + ((t ^ brow) << 4), woff1 = brow * 128 + (((t + 4) ^ brow) << 4);
    const uint32_t ring_base = smem_u32(ring);
    const int g_last = groups_per_row - 1;
    const int fg0 = min((2 * box_lo) / group128, g_last), fin0 = (2 * box_lo) % group128;
    float* red = red_all + (pair * 2 * 32 + lane) * NACC;       // [buffer][lane][NACC] of this pair

    int slot = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int ui = 0; ui < my_units; ++ui) {
        const int unit = first_unit + ui * unit_stride;
        const __half* srow = scales + static_cast<int64_t>(unit * kRgRows + brow) * groups_per_row;
        const int64_t hi_row = static_cast<int64_t>(8) * groups_per_row;
        // running group index of the next 128-wide block whose scales are fetched (two blocks per box)
        int fg = fg0, fin = fin0;
        auto next_scales = [&](__half& lo, __half& hi) {
            lo = __ldg(srow + fg);                               // plain loads: nothing may depend on them before their use
            hi = __ldg(srow + hi_row + fg);
            if (++fin == group128) { fin = 0; fg = fg < g_last ? fg + 1 : g_last; }
        };
        // two accumulator chains (the two MMA steps of a word), added at the end: halves the dependent chain
        // (for 9..16 activation rows the two row sets already give two chains; one accumulator each keeps registers down)
        constexpr int NACC1 = MPAD == 8 ? NACC : 4;
        float acc0[NACC], acc1[NACC1];
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc0[i] = 0.f;
#pragma unroll
        for (int i = 0; i < NACC1; ++i) acc1[i] = 0.f;
        __half sl[2], sh[2], nl[2], nh[2];                      // scales of the current box, and of the next one
        next_scales(sl[0], sh[0]);
        next_scales(sl[1], sh[1]);
        uint32_t a_addr = act_lane;
        for (int st = 0; st < my_boxes && ok; ++st) {
            next_scales(nl[0], nh[0]);
            next_scales(nl[1], nh[1]);
            if (!mbar_wait(&bars[slot], phase, ST_WAIT_SMEM_FULL, st)) { ok = false; break; }
            const uint32_t box = ring_base + slot * kRgBoxBytes;
            uint32_t touched = 0u;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 wl = lds128<0>(box + (h == 0 ? woff0 : woff1));
                const uint4 wh = lds128<1024>(box + (h == 0 ? woff0 : woff1));
                touched ^= wl.x ^ wh.x;
                const __half2 s_lo = __half2half2(sl[h]), s_hi = __half2half2(sh[h]);
                const uint32_t wdl[4] = {wl.x, wl.y, wl.z, wl.w}, wdh[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t l0, l1, l2, l3, u0, u1, u2, u3;
                    unpack_word(wdl[j], bias_lo, bias_hi, sixteenth, s_lo, l0, l1, l2, l3);
                    unpack_word(wdh[j], bias_lo, bias_hi, sixteenth, s_hi, u0, u1, u2, u3);
                    const uint32_t aoff = a_addr + static_cast<uint32_t>((h * 16 + j) * MPAD) * 16;
                    const uint4 b = lds128<0>(aoff);
                    // step A: k-slots (k0, k0+4 | k0+1, k0+5); step B: (k0+2, k0+6 | k0+3, k0+7)
                    if (MPAD == 8) {
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc0[0]), l0, u0, l1, u1, b.x, b.y);
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc1[0]), l2, u2, l3, u3, b.z, b.w);
                    } else {
                        const uint4 b8 = lds128<128>(aoff);         // activation rows 8..15
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc0[0]), l0, u0, l1, u1, b.x, b.y);
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc0[4]), l0, u0, l1, u1, b8.x, b8.y);
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc0[0]), l2, u2, l3, u3, b.z, b.w);
                        mma16816(*reinterpret_cast<float(*)[4]>(&acc0[4]), l2, u2, l3, u3, b8.z, b8.w);
                    }
                }
            }
            sl[0] = nl[0]; sl[1] = nl[1]; sh[0] = nh[0]; sh[1] = nh[1];
            a_addr += kActStage;
            // The slot may be refilled only when the four loads from it have LANDED in registers; following them in
            // program order is not enough (the copy could be issued while they are in flight, and the unpack
            // arithmetic may be moved across it).  The loaded words are ANDed with a zero that only exists at run time
            // (a literal zero would be folded away by the assembler), so the result is a zero the hardware can form
            // only once the loads have returned; a warp's load completes as a unit, so lane 0's registers speak for all.
            const uint32_t landed = touched & rt_zero;
            __syncwarp();                                       // every lane has read the slot
            if (lane == 0 && issued < total) issue(landed);     // refill it: the slot just read is the next to fill
            if (++slot == ST) { slot = 0; phase ^= 1; }
        }
        // upper half -> shared memory; lower half adds it (own sum first) and writes the unit's outputs.  One named
        // barrier per unit and two buffers: the upper warp can be a unit ahead, never two.  A warp whose wait ran
        // out still takes part, so its partner is not left waiting.
        float* slot_red = red + (ui & 1) * 32 * NACC;
        auto own = [&](int i) { return MPAD == 8 ? acc0[i] + acc1[i % NACC1] : acc0[i]; };
        if (kh == 1) {
#pragma unroll
            for (int i = 0; i < NACC; i += 4)
                *reinterpret_cast<float4*>(slot_red + i) = make_float4(own(i), own(i + 1), own(i + 2), own(i + 3));
        }
        asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
        if (kh == 0) {
            // accumulator register r of set q: (operand row g + 8 * (r >> 1), activation row m = 8 q + 2t + (r & 1))
#pragma unroll
            for (int q = 0; q < NACC / 4; ++q) {
                const float4 up = *reinterpret_cast<const float4*>(slot_red + 4 * q);
                const float upv[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int m = 8 * q + 2 * t + (r & 1);
                    const int nrow = brow + 8 * (r >> 1);
                    const float sum = own(4 * q + r) + upv[r];
                    if (m < M) out[static_cast<int64_t>(m) * ldo + col_offset + unit * kRgRows + nrow] = __float2half_rn(sum);
                }
            }
        }
    }
    if (!ok && lane == 0) {   // give boxes already in flight a bounded chance to land before the warp exits
        for (int i = 0; i < ST; ++i) (void)mbar_wait_limit(&bars[i], i < slot ? phase ^ 1 : phase, ST_WAIT_SMEM_FULL, -1, 1ll << 22);
    }
}

extern "C" __global__ void __launch_bounds__(kRgThreads, 1)
tb200_k_gemv_w4a16_ring_m8(const __grid_constant__ CUtensorMap tmap_w, const __half* a, const __half* scales, __half* out, int M,
                           int K, int kpad, int gpr, int group128, int64_t ldo, int64_t col_offset, float zp, int units,
                           int pairs_used) {
    gemv_ring_body<8>(&tmap_w, a, scales, out, M, K, kpad, gpr, group128, ldo, col_offset, zp, units, pairs_used);
}
extern "C" __global__ void __launch_bounds__(kRgThreads, 1)
tb200_k_gemv_w4a16_ring_m16(const __grid_constant__ CUtensorMap tmap_w, const __half* a, const __half* scales, __half* out, int M,
                            int K, int kpad, int gpr, int group128, int64_t ldo, int64_t col_offset, float zp, int units,
                            int pairs_used) {
    gemv_ring_body<16>(&tmap_w, a, scales, out, M, K, kpad, gpr, group128, ldo, col_offset, zp, units, pairs_used);
}

TB200_DEFINE_STATUS_HOOKS(gemv_ring)

namespace tb200 {

bool gemv_ring_fits(int64_t m, int64_t k) {
    const int64_t kpad = (k + kRgStageK - 1) / kRgStageK * kRgStageK;
    if (kpad > (1 << 20)) return false;
    return (m <= 8 ? RingCfg<8>::smem_bytes(static_cast<int>(kpad)) : RingCfg<16>::smem_bytes(static_cast<int>(kpad))) <= kRgMaxSmem;
}

// Host launcher used by tb200_gemm_w4a16 for m <= 16 when the activations fit in shared memory beside the
// rings (arguments already validated there; n is a multiple of 128, wp 16-byte aligned with a row pitch of
// k / 2 bytes).
int launch_gemv_w4a16_ring(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                           int64_t group, int zero_point, int64_t ldo, int64_t col_offset, cudaStream_t st) {
    const int kpad = static_cast<int>((k + kRgStageK - 1) / kRgStageK * kRgStageK);
    const int units = static_cast<int>(n / kRgRows);
    const int sms = num_sms();
    const int grid = units < sms ? units : sms;
    int pairs_used = (units + grid - 1) / grid;        // pairs of warps that get work: one unit per pair and round
    if (pairs_used > kRgWarps / 2) pairs_used = kRgWarps / 2;
    CUtensorMap tw;
    int rc = encode_tmap_2d(&tw, wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k / 2, k / 2, kRgRows, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    static PerDeviceInt attr8, attr16;
    const float zp = static_cast<float>(zero_point);
    if (m <= 8) {
        const int smem = RingCfg<8>::smem_bytes(kpad);
        rc = ensure_max_smem(attr8, reinterpret_cast<const void*>(tb200_k_gemv_w4a16_ring_m8), kRgMaxSmem);
        if (rc != TB200_OK) return rc;
        tb200_k_gemv_w4a16_ring_m8<<<grid, kRgThreads, smem, st>>>(tw, static_cast<const __half*>(a), static_cast<const __half*>(scales),
                                                                  static_cast<__half*>(out), static_cast<int>(m), static_cast<int>(k), kpad,
                                                                  static_cast<int>(k / group), static_cast<int>(group / 128), ldo, col_offset,
                                                                  zp, units, pairs_used);
    } else {
        const int smem = RingCfg<16>::smem_bytes(kpad);
        rc = ensure_max_smem(attr16, reinterpret_cast<const void*>(tb200_k_gemv_w4a16_ring_m16), kRgMaxSmem);
        if (rc != TB200_OK) return rc;
        tb200_k_gemv_w4a16_ring_m16<<<grid, kRgThreads, smem, st>>>(tw, static_cast<const __half*>(a), static_cast<const __half*>(scales),
                                                                   static_cast<__half*>(out), static_cast<int>(m), static_cast<int>(k), kpad,
                                                                   static_cast<int>(k / group), static_cast<int>(group / 128), ldo, col_offset,
                                                                   zp, units, pairs_used);
    }
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

}  // namespace tb200
