// int8 x packed-2-bit GEMM for sm_100a:  out[m, n] = sum_k a[m, k] * B[k, n]  (int32, exact), where
// B[i * Kb + kb, n] = ((b[kb, n] >> 2i) & 3) - 1 for i = 0..3 and Kb = K / 4: every byte of the packed
// operand carries four weights of the same column, a quarter of K apart
// (tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19).
//
// K may be visited in any order as long as both operands agree, so the kernel walks the PACKED rows:
// a stage holds 64 packed rows of b ([64 x BN] bytes, as stored) and, for each of the four bit fields
// i, the matching [128 x 64] slice of a (columns i * Kb + kb0 ..), 256 values of k in all.  Unpacking
// a byte tile yields four int8 planes that keep the packed tile's shape — n stays the contiguous
// index — and tcgen05.mma reads such a tile directly as an MN-major operand: no transpose anywhere.
//
// Warp roles (512 threads, one persistent CTA per SM):
//   warp 0       TMA producer: four [128 x 64 B] boxes of a (64-byte swizzle) and one [64 x BN] box of b
//   warps 1, 2   MMA issuers: warp 1 takes the first 32 packed rows of every stage, warp 2 the second
//                32; per plane one tcgen05.mma kind::i8 (M = 128, N = BN, K = 32), each issuer into its
//                own TMEM accumulator — integer addition is associative, the epilogue adds the two
//   warps 4..11  unpack: shared-memory packed bytes -> planes in the 128-byte-swizzled MN-major operand
//                layout.  Four groups of two warps, each with its own two-plane buffer: group g turns
//                the packed rows of sub-step g / 2 into planes 2 (g % 2) and 2 (g % 2) + 1 of every
//                stage.  One pass of a group is a latency chain (wait, load, unpack, store, proxy fence,
//                arrive, two MMAs, commit, wake-up) much longer than its arithmetic, so four chains run
//                side by side instead of eight warps walking one chain together
//   warps 12..15 row sums of a during the main loop, then the epilogue: tcgen05.ld both accumulators,
//                add, subtract the row sum, store int32 rows
//
// The "- 1" of the decode is taken out of the inner loop: sum_k a * (f - 1) = sum_k a * f - sum_k a.  The
// unpack warps, whose instruction chain paces the kernel, only shift and mask (the planes hold the raw
// fields 0..3, fed to the tensor cores as UNSIGNED 8-bit against the signed a), and the four epilogue
// warps, otherwise idle until the accumulators complete, add up their own row of every a slice from
// shared memory (dp4a against ones) and subtract that once per tile.  All of it is int32 arithmetic, so
// the result is the same number bit for bit.
// Every mbarrier wait is bounded and reports through g_status.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kI8BM = 128;
constexpr int kI8StageRows = 64;                 // packed rows per stage
constexpr int kI8SubRows = 32;                   // packed rows per MMA (K = 32 per plane)
constexpr int kI8APlaneBytes = kI8BM * kI8StageRows;            // [128 x 64 B]
constexpr int kI8ABytes = 4 * kI8APlaneBytes;

template <int BN> struct I8Cfg {
    static constexpr int kStages = BN == 256 ? 3 : 4;
    static constexpr int kPackedBytes = kI8StageRows * BN;
    static constexpr int kStageBytes = kI8ABytes + kPackedBytes;
    static constexpr int kPlaneBytes = kI8SubRows * BN;         // one unpacked plane of one sub-step
    static constexpr int kGroups = 4;                           // unpack groups = unpacked buffers
    static constexpr int kGroupWarps = 2;
    static constexpr int kGroupBufBytes = 2 * kPlaneBytes;      // two planes of one sub-step
    static constexpr int kThreads = 512;
    static constexpr int kConvertWarps = 8;
    static constexpr int kTmemCols = 2 * BN;                    // one accumulator per issuer
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kGroups * kGroupBufBytes + kBarBytes + 1024;
    static_assert(kGroups * kGroupWarps == kConvertWarps, "unpack warps");
};

// K-major operand stored with the 64-byte swizzle (rows of 64 bytes, 8-row groups 512 bytes apart)
__device__ __forceinline__ uint64_t umma_desc_k_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(512 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(4) << 61;
    return d;
}
// MN-major operand stored with the 128-byte swizzle: 128 contiguous bytes along N per row of k, rows
// 128 bytes apart, 8-row groups `1024` bytes apart (stride offset), 128-wide column blocks
// `atom_pitch` bytes apart (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t atom_pitch) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(atom_pitch >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// kind::i8 instruction descriptor: D = s32 (2 at [4,6)), A signed 8-bit (1 at [7,10)), B unsigned 8-bit
// (0 at [10,13)), A K-major, B MN-major (bit 16), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_i8(uint32_t m, uint32_t n) {
    return (2u << 4) | (1u << 7) | (0u << 10) | (1u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// four packed bytes -> field i of each as four unsigned bytes 0..3 (the "- 1" is applied per row in the
// epilogue)
__device__ __forceinline__ uint32_t unpack_field(uint32_t w, int i) {
    return (w >> (2 * i)) & 0x03030303u;
}
// sum of the sixteen signed bytes of v, added to acc
__device__ __forceinline__ int32_t add_bytes16(const uint4& v, int32_t acc) {
    acc = __dp4a(static_cast<int>(v.x), 0x01010101, acc);
    acc = __dp4a(static_cast<int>(v.y), 0x01010101, acc);
    acc = __dp4a(static_cast<int>(v.z), 0x01010101, acc);
    return __dp4a(static_cast<int>(v.w), 0x01010101, acc);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

template <int BN>
__device__ __forceinline__ void gemm_i8_body(const CUtensorMap* __restrict__ tmap_a, const CUtensorMap* __restrict__ tmap_b,
                                             int32_t* __restrict__ out, int M, int N, int K, int64_t ldo) {
    using Cfg = I8Cfg<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ubuf = smem + S * Cfg::kStageBytes;                  // [4 groups][2 planes][32 x BN]
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(ubuf + Cfg::kGroups * Cfg::kGroupBufBytes);
    uint64_t* bar_empty = bar_full + S;       // stage consumed: 2 issuer commits + 8 unpack warps + 4 row-sum warps
    uint64_t* bar_ufull = bar_empty + S;      // [4] group buffer written (the group's 2 warps)
    uint64_t* bar_ufree = bar_ufull + Cfg::kGroups;   // [4] group buffer read by its issuer's MMAs
    uint64_t* bar_afull = bar_ufree + Cfg::kGroups;   // both accumulators complete (2 issuer commits)
    uint64_t* bar_aempty = bar_afull + 1;     // both accumulators drained (4 epilogue warps)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_aempty + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int Kb = K / 4;
    const int KS = Kb / kI8StageRows;          // stages per tile
    const int tiles_m = (M + kI8BM - 1) / kI8BM;
    const int tiles_n = N / BN;
    const int tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 2 + Cfg::kConvertWarps + 4);
        }
        for (int u = 0; u < Cfg::kGroups; ++u) {
            mbar_init(&bar_ufull[u], Cfg::kGroupWarps);
            mbar_init(&bar_ufree[u], 1);
        }
        mbar_init(bar_afull, 2);
        mbar_init(bar_aempty, 4);
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
            uint32_t n = 0;                                       // stages issued so far
            uint32_t s = 0, ph = 0;                               // ring slot and phase of stage n, advanced by addition
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const int m_blk = t % tiles_m, n_blk = t / tiles_m;
                for (int ks = 0; ks < KS; ++ks, ++n, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
                    if (!mbar_wait(&bar_empty[s], ph ^ 1, ST_WAIT_SMEM_EMPTY, ks)) { ok = false; break; }
                    uint8_t* stage = smem + s * Cfg::kStageBytes;
                    const int kb0 = ks * kI8StageRows;
                    mbar_expect_tx(&bar_full[s], Cfg::kStageBytes);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        tma_load_2d(stage + i * kI8APlaneBytes, tmap_a, &bar_full[s], i * Kb + kb0, m_blk * kI8BM);
                    tma_load_2d(stage + kI8ABytes, tmap_b, &bar_full[s], n_blk * BN, kb0);
                }
            }
            if (!ok) {
                // give copies already in flight a bounded chance to land before the CTA exits
                for (int st = 0; st < S; ++st) {
                    if (n > static_cast<uint32_t>(st)) {
                        const uint32_t last = n - 1 - ((n - 1 - st) % S);
                        (void)mbar_wait(&bar_full[st], (last / S) & 1, ST_WAIT_SMEM_FULL, -1);
                    }
                }
            }
        }
    } else if (warp <= 2) {
        // ---------------- MMA issuers ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(kI8BM, BN);
            const uint32_t me = warp - 1;                         // sub-step of every stage, accumulator; groups 2 me, 2 me + 1
            const uint32_t d_tmem = tmem_base + me * BN;
            const uint32_t u_addr = smem_u32(ubuf + 2 * me * Cfg::kGroupBufBytes);
            uint32_t n = 0;                                       // stages seen so far (= own sub-steps)
            uint32_t s = 0, ph = 0;                               // ring slot and phase of stage n, advanced by addition
            uint32_t tile_cnt = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_cnt) {
                if (!mbar_wait(bar_aempty, (tile_cnt & 1) ^ 1, ST_WAIT_TMEM_EMPTY, t)) { ok = false; break; }
                tc_fence_after();
                for (int ks = 0; ks < KS; ++ks, ++n, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
                    if (!mbar_wait(&bar_full[s], ph, ST_WAIT_SMEM_FULL, ks)) { ok = false; break; }
                    const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes) + me * kI8SubRows;   // +32 B along K
#pragma unroll
                    for (int h = 0; h < 2; ++h) {                 // the two groups of this sub-step
                        if (!mbar_wait(&bar_ufull[2 * me + h], n & 1, ST_WAIT_OPERAND, ks)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int i = 2 * h; i < 2 * h + 2; ++i) {
                            umma_i8_ss(d_tmem, umma_desc_k_sw64(a_addr + i * kI8APlaneBytes),
                                       umma_desc_mn_sw128(u_addr + i * Cfg::kPlaneBytes, kI8SubRows * 128), idesc,
                                       (ks > 0 || i > 0) ? 1u : 0u);
                        }
                        tc_commit(&bar_ufree[2 * me + h]);
                    }
                    if (!ok) break;
                    tc_commit(&bar_empty[s]);
                }
                if (ok) tc_commit(bar_afull);
            }
        }
    } else if (warp >= 4 && warp < 4 + Cfg::kConvertWarps) {
        // ---------------- unpack warps ----------------
        constexpr int kChunksPerRow = BN / 16;
        constexpr int kChunks = kI8SubRows * kChunksPerRow;       // 16-byte chunks per sub-step
        constexpr int kGroupThreads = 32 * Cfg::kGroupWarps;
        constexpr int kPerThread = kChunks / kGroupThreads;
        static_assert(kPerThread >= 1, "unpack mapping");
        const int g = (warp - 4) / Cfg::kGroupWarps;              // group = buffer
        const int j = g >> 1, h = g & 1;                          // sub-step, plane pair
        const int gt = threadIdx.x - (4 + g * Cfg::kGroupWarps) * 32;
        uint8_t* dst = ubuf + g * Cfg::kGroupBufBytes;
        uint32_t n = 0;
        uint32_t s = 0, ph = 0;                                   // ring slot and phase of stage n, advanced by addition
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            for (int ks = 0; ks < KS && ok; ++ks, ++n, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
                if (!mbar_wait(&bar_full[s], ph, ST_WAIT_SMEM_FULL, ks)) { ok = false; break; }
                const uint8_t* packed = smem + s * Cfg::kStageBytes + kI8ABytes + j * kI8SubRows * BN;
                uint4 w[kPerThread];
#pragma unroll
                for (int c = 0; c < kPerThread; ++c) {
                    const int chunk = gt + c * kGroupThreads;
                    w[c] = *reinterpret_cast<const uint4*>(packed + (chunk / kChunksPerRow) * BN + (chunk % kChunksPerRow) * 16);
                }
                if (!mbar_wait(&bar_ufree[g], (n & 1) ^ 1, ST_WAIT_SMEM_EMPTY, -ks - 1)) { ok = false; break; }
#pragma unroll
                for (int c = 0; c < kPerThread; ++c) {
                    const int chunk = gt + c * kGroupThreads;
                    const int row = chunk / kChunksPerRow, col16 = chunk % kChunksPerRow;
                    const int off = (col16 >> 3) * (kI8SubRows * 128) + row * 128 + (((col16 & 7) ^ (row & 7)) << 4);
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const int i = 2 * h + p;
                        uint4 o;
                        o.x = unpack_field(w[c].x, i);
                        o.y = unpack_field(w[c].y, i);
                        o.z = unpack_field(w[c].z, i);
                        o.w = unpack_field(w[c].w, i);
                        *reinterpret_cast<uint4*>(dst + p * Cfg::kPlaneBytes + off) = o;
                    }
                }
                fence_async_smem();                               // generic-proxy writes -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bar_ufull[g]);
                    mbar_arrive(&bar_empty[s]);                   // this warp's packed bytes are in registers / consumed
                }
            }
        }
    } else if (warp >= 12) {
        // ---------------- epilogue ----------------
        const int ew = warp - 12;                                  // == warp % 4: TMEM lanes 32 * ew ..
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
        // this thread's row of an a slice: 64 bytes at row * 64, its four 16-byte chunks permuted by the
        // 64-byte swizzle (chunk ^ bits [1,3) of the row).  A sum visits them in any order; reading chunk
        // (c ^ that key) makes the eight lanes of a quarter-warp hit eight different 16-byte bank groups.
        const int row = ew * 32 + lane;
        const uint32_t row_off = row * 64, key = (row >> 1) & 3;
        uint32_t tile_cnt = 0, n = 0;
        uint32_t es = 0, eph = 0;                                 // ring slot and phase of stage n, advanced by addition
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_cnt) {
            const int m_blk = t % tiles_m, n_blk = t / tiles_m;
            const int m = m_blk * kI8BM + row;
            int32_t rs0 = 0, rs1 = 0;                              // sum_k a[m, k] (rows past M are zero-filled by TMA)
            for (int ks = 0; ks < KS; ++ks, ++n, es = (es + 1 == S ? 0 : es + 1), eph ^= (es == 0)) {
                const uint32_t s = es;
                if (!mbar_wait(&bar_full[s], eph, ST_WAIT_SMEM_FULL, ks)) { ok = false; break; }
                const uint8_t* a_row = smem + s * Cfg::kStageBytes + row_off;
                uint32_t touched = 0u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int c = 0; c < 4; c += 2) {
                        const uint4 u = *reinterpret_cast<const uint4*>(a_row + i * kI8APlaneBytes + (((c + 0) ^ key) << 4));
                        const uint4 v = *reinterpret_cast<const uint4*>(a_row + i * kI8APlaneBytes + (((c + 1) ^ key) << 4));
                        rs0 = add_bytes16(u, rs0);
                        rs1 = add_bytes16(v, rs1);
                        touched ^= u.x ^ v.x;
                    }
                }
                // The stage may be handed back only when the loads above have LANDED: an arrive that merely follows them
                // in program order can be issued while they are in flight, and the refill would overtake them.  One word
                // of every load is folded into `touched` (not the sums: their dependent chains are long, and the
                // stage would be held for their whole length); ANDed with a zero that only exists at run time (the sign bit of M;
                // a literal zero would be folded away) they give a zero the hardware can form only after the loads have
                // returned, and the barrier address depends on it.
                const uint32_t landed = touched & (static_cast<uint32_t>(M) >> 31);
                __syncwarp();
                if (lane == 0)                                    // this warp's rows of the a slices are read
                    mbar_arrive(reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(&bar_empty[s]) + landed));
            }
            if (!ok) break;
            const uint32_t rs = static_cast<uint32_t>(rs0 + rs1);
            if (!mbar_wait(bar_afull, tile_cnt & 1, ST_WAIT_TMEM_FULL, t)) { ok = false; break; }
            tc_fence_after();
            int32_t* dst = out + static_cast<int64_t>(m < M ? m : 0) * ldo + n_blk * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v0[32], v1[32];
                tmem_ld32(t_lane + c * 32, v0);
                tmem_ld32(t_lane + BN + c * 32, v1);
                tmem_wait_ld();
                if (c == BN / 32 - 1) {                            // both accumulators are in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_aempty);
                }
                if (m < M) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        int4 o;
                        o.x = static_cast<int32_t>(v0[4 * q + 0] + v1[4 * q + 0] - rs);
                        o.y = static_cast<int32_t>(v0[4 * q + 1] + v1[4 * q + 1] - rs);
                        o.z = static_cast<int32_t>(v0[4 * q + 2] + v1[4 * q + 2] - rs);
                        o.w = static_cast<int32_t>(v0[4 * q + 3] + v1[4 * q + 3] - rs);
                        *reinterpret_cast<int4*>(dst + c * 32 + 4 * q) = o;
                    }
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

extern "C" __global__ void __launch_bounds__(I8Cfg<256>::kThreads, 1)
tb200_k_gemm_i8_p2_n256(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, int32_t* out,
                        int M, int N, int K, int64_t ldo) {
    gemm_i8_body<256>(&tmap_a, &tmap_b, out, M, N, K, ldo);
}
extern "C" __global__ void __launch_bounds__(I8Cfg<128>::kThreads, 1)
tb200_k_gemm_i8_p2_n128(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, int32_t* out,
                        int M, int N, int K, int64_t ldo) {
    gemm_i8_body<128>(&tmap_a, &tmap_b, out, M, N, K, ldo);
}

TB200_DEFINE_STATUS_HOOKS(gemm_i8)

template <int BN, typename Kern>
static int launch_i8(Kern kern, const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int64_t ldo,
                     cudaStream_t st) {
    using Cfg = I8Cfg<BN>;
    static PerDeviceInt attr_set;
    {
        const int rc_attr = ensure_max_smem(attr_set, reinterpret_cast<const void*>(kern), Cfg::kSmemBytes);
        if (rc_attr != TB200_OK) return rc_attr;
    }
    CUtensorMap ta, tb;
    int rc = encode_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m, k, k, kI8BM, kI8StageRows, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k / 4, n, n, kI8StageRows, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TB200_OK) return rc;
    const int64_t tiles = ((m + kI8BM - 1) / kI8BM) * (n / BN);
    const int grid = static_cast<int>(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(ta, tb, static_cast<int32_t*>(out), static_cast<int>(m),
                                                        static_cast<int>(n), static_cast<int>(k), ldo);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_matmul_int8_packed2(const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k,
                                         int64_t ldo, void* stream) {
    clear_error();
    if (!a || !b || !out) return fail(TB200_ERR_ARG, "matmul_int8_packed2: null pointer");
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(TB200_ERR_ARG, "matmul_int8_packed2: non-positive size m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    if (k % 4 != 0) return fail(TB200_ERR_ARG, "matmul_int8_packed2: k=%lld must be a multiple of 4 (four fields per byte)", (long long)k);
    if (k % 256 != 0 || n % 128 != 0)
        return fail(TB200_ERR_UNSUPPORTED, "matmul_int8_packed2: k=%lld must be a multiple of 256 and n=%lld of 128", (long long)k, (long long)n);
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(TB200_ERR_UNSUPPORTED, "matmul_int8_packed2: dimension too large");
    if (ldo < n || ldo % 4 != 0) return fail(TB200_ERR_ALIGN, "matmul_int8_packed2: ldo=%lld must be >= n and a multiple of 4", (long long)ldo);
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return fail(TB200_ERR_ALIGN, "matmul_int8_packed2: a, b, out must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t tiles256 = ((m + kI8BM - 1) / kI8BM) * (n / 256);
    if (n % 256 == 0 && 2 * tiles256 > num_sms())
        return launch_i8<256>(tb200_k_gemm_i8_p2_n256, a, b, out, m, n, k, ldo, st);
    return launch_i8<128>(tb200_k_gemm_i8_p2_n128, a, b, out, m, n, k, ldo, st);
}
