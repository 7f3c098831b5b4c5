// W4A16 dequant-fused GEMM for sm_100a:
//   out[m, col_offset + n] = fp16( sum_k a[m,k] * fp16((q[n,k] - zp) * s[n, k/group]) ),  fp32 accumulate.
//
// The kernel computes the transposed product D^T[n, m] = W[n,:] . A[m,:] so that the *weights* are
// the tensor-memory operand of tcgen05.mma: the convert warps unpack int4 to fp16 in registers and
// write the fragments straight into TMEM with tcgen05.st — the dequantised tile never goes back
// through shared memory.  Activations arrive by TMA as the 128-byte-swizzled shared-memory operand
// with MMA-N = the activation-row tile MT (16 for decode-sized m, 64, 128, or 256 for m > 128:
// issuing a tcgen05.mma costs the issuing thread roughly 90 cycles whatever its size, so only
// N = 256 instructions (128 cycles of tensor work each) keep the tensor pipe ahead of the issuer).
//
// One persistent CTA per SM walks work items (weight tile, activation tile(s), K split).  Three
// rings decouple the roles, so the small packed-weight stream runs far ahead of the wide
// activation stream and the TMA + unpack latency stays off the MMA's critical path:
//   packed weights  smem, SW stages of [128 x 32 B] (32-byte swizzle)   TMA (warp 1)  -> convert warps
//   fp16 operand    TMEM, AST stages of 32 columns                      convert warps -> MMA
//   activations     smem, SA stages of [MT x 64] fp16 (128-byte swizzle)         TMA (warp 0) -> MMA
// Roles:
//   warp 0            activation TMA producer
//   warp 1            packed-weight TMA producer
//   warps 2..5        MMA issuers (NI of them; the rest idle).  Issuer j takes K blocks with it % NI == j:
//                     four tcgen05.mma kind::f16 (A from TMEM, B from smem, K = 16 each) into ITS OWN
//                     accumulator, then ONE tcgen05.commit: "MMAs of this K block complete" frees the
//                     activation stage and the operand stage (same barrier).  Small-N MMAs finish in
//                     fewer cycles than one thread needs to issue them, so decode-sized tiles use
//                     several issuers; private accumulators keep the summation order fixed.
//   (idle warps)      up to the next multiple of four (the following warp quads align with the TMEM lane quarters)
//   warps 4.. / 8..   convert warps (kDQ groups of 4 taking K blocks in turn): thread = weight row;
//                     2 x LDS.128 of packed nibbles -> 64 fp16 -> tcgen05.st into an operand stage
//   next 4 warps      epilogue: tcgen05.ld the finished accumulators (summed in issuer order), cast;
//                     for MT >= 128 transpose
//                     through a shared-memory tile and write it with one TMA store per 128 rows,
//                     otherwise store directly (fp32 split-K partials or fp16)
// With a K split > 1 the epilogue writes fp32 partials to the caller's workspace and a second
// kernel sums them in a fixed order (deterministic).  Every wait is bounded (see common.cuh).
#include "common.cuh"

#include <mutex>
#include <stdlib.h>

namespace tb200 {
namespace {

constexpr int kBNW = 128;      // weight rows per tile (MMA M)
constexpr int kBK = 64;        // K per stage: 64 fp16 = one 128-byte swizzle row
constexpr int kWBytes = kBNW * (kBK / 2);   // 4096 packed bytes per weight stage
constexpr int kGroupN = 16;    // tile-order grouping for L2 reuse

// MT = activation rows per work item = MMA N.  kPair: two CTAs on neighbouring SMs (a cluster of 2) share one
// work item of 256 weight rows x 256 activation rows: each converts ITS 128 weight rows into its own tensor
// memory and loads ITS 128 activation rows, and ONE thread of the leader CTA issues cta_group::2 MMAs (M = 256)
// that read both CTAs' tensor and shared memory — twice the tensor work per issued instruction, which is what
// the issuing thread of the single-CTA kernel cannot deliver fast enough, and half the activation bytes
// per SM.
template <int MT, bool kPair = false> struct W4Cfg {
    static_assert(!kPair || MT == 256, "the CTA-pair kernel exists for the 256-row tile only");
    // Convert warp groups; group g takes the K blocks with it % kDQ == g.  One group needs about 1 us per K block
    // (barrier hops, LDS, ~140 dependent ALU instructions, tcgen05.st), so two groups deliver a block every
    // ~0.5 us whatever the tile size.  The 128-row tile (one wave of CTAs) is bound by exactly that: three groups
    // were worth 12 %, a fourth another 6 % once it fitted the same 768 threads.  The 256-row tile gains 2-4 %
    // from a third group and loses it again with a fourth (80 registers per thread at 768 threads).
    static constexpr int kDQ = MT == 128 ? 4 : (MT == 256 ? 3 : 2);
    static constexpr int kActRows = kPair ? MT / 2 : MT;         // activation rows this CTA loads per K block
    static constexpr int kActStageBytes = kActRows * kBK * 2;    // one [rows x 64] fp16 activation tile
    static constexpr int kNI = MT <= 32 ? 4 : (MT <= 128 ? 2 : 1);   // MMA issuer threads, one accumulator each
    static constexpr int kNAcc = MT >= 128 ? 1 : 2;              // accumulator sets (double-buffered when they fit)
    static constexpr bool kTmaStore = MT >= 128;                 // epilogue through smem + TMA store
    static constexpr int kStoreBytes = kTmaStore ? 128 * kBNW * 2 : 0;   // [128 m x 128 n] fp16 staging tile
    static constexpr int kSA = MT <= 32 ? 16 : (MT == 64 ? 12 : (MT == 128 || kPair ? 8 : 5));   // activation stages
    // packed-weight stages: a multiple of kDQ, so that every slot is always consumed by the SAME convert group.
    // A group then meets the phases of its slots one by one.  With 8 slots and 3 groups successive uses of a
    // slot fell to different groups, and a group could test a slot's barrier two phases ahead of it — copies
    // complete out of order, so "block it - 3 has landed" does not imply "block it - 8 has" — where a
    // parity test cannot tell "phase k complete" from "phase k - 1 not yet complete": it then read the slot's old
    // bytes (seen as single output columns differing between identical calls of large problems).
    static constexpr int kSW = MT <= 32 ? 32 : (MT == 256 ? (kPair ? 9 : 6) : 16);
    // TMEM operand stages, 32 columns each: as deep as the activation ring, because both are freed by
    // the same per-K-block commit and share its barrier
    static constexpr int kAStages = kSA < 8 ? kSA : 8;
    static constexpr int kDCols = kNAcc * kNI * MT;
    static constexpr int kACol0 = kDCols;
    static constexpr int kTmemNeed = kDCols + 32 * kAStages;
    static constexpr int kTmemCols = kTmemNeed <= 32 ? 32 : kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128
                                     : kTmemNeed <= 256 ? 256 : 512;
    static constexpr int kMmaWarp0 = 2;
    // convert warps start at a multiple of four (a warp reaches the TMEM lane quarter warp % 4): right behind the
    // issuers when there are at most two of them, which is what lets the 128-row tile run four convert groups
    // in the 768 threads that held three
    static constexpr int kCvtWarp0 = kNI <= 2 ? 4 : 8;
    static constexpr int kEpiWarp0 = kCvtWarp0 + 4 * kDQ;
    static constexpr int kWarps = kEpiWarp0 + 4;
    static constexpr int kThreads = 32 * kWarps;
    static constexpr int kActRingBytes = kSA * kActStageBytes;
    static constexpr int kWRingBytes = kSW * kWBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kSmemBytes = kActRingBytes + kWRingBytes + kStoreBytes + kBarBytes + 1024;
    static_assert(kAStages <= kSA, "operand ring must not be deeper than the activation ring");
    static_assert(kSW % kDQ == 0, "each packed-weight slot must belong to one convert group");
    static_assert(kTmemNeed <= 512, "TMEM over-subscribed");
    static_assert((2 * kSA + 2 * kSW + kAStages + 4) * 8 + 8 <= kBarBytes, "barrier block too small");
    static_assert(kSmemBytes <= 232448, "over the 227 KB shared-memory limit");
};

// Output buffers of the other ranks of an N-partitioned GEMM (already offset to this rank's column
// slice): the epilogue stores every finished tile there too, so the all-gather rides on the GEMM.
constexpr int kMaxPeers = 7;
struct PeerOut {
    int count;
    int use_tma;                 // 1: the tiles go to the peers as TMA stores through PeerMaps, 0: as 128-bit stores from the epilogue threads
    __half* base[kMaxPeers];
};
// One tensor map per peer output slice (same geometry as the local one): the epilogue then hands a finished tile to
// the copy engine once per rank instead of pushing it through the NVLink with its own threads' stores.
struct PeerMaps {
    CUtensorMap m[kMaxPeers];
};

// half < 0: the item covers all MT activation rows of tile m_blk; half = 0 / 1: a 128-row half of a 256-row
// tile (tail of the persistent schedule, see Schedule below).
struct Item { int n_blk, m_blk, kb0, kb1, ks, half; };
// The persistent work list: `full` whole items (tile x K split), then 2 * tail_split half-height units that
// cover the last tail_split tiles.  When the last wave of the grid would hold at most half a grid of
// 256-row tiles, cutting them in two lets twice as many SMs share that wave (6.05 -> 6.5 instead of 7
// waves for 896 tiles on 148 SMs).  A half unit adds the same K blocks in the same order into the same
// accumulator columns, so results do not depend on where the cut falls.
struct Schedule { int tiles_n, tiles_m, splitk, KB, tail_split, items; };
__device__ __forceinline__ Schedule make_schedule(int tiles_n, int tiles_m, int splitk, int KB, int tail_split) {
    Schedule sc{tiles_n, tiles_m, splitk, KB, tail_split, tiles_n * tiles_m * splitk + tail_split};
    return sc;
}
// tiles_m counts activation tiles of MT rows.
__device__ __forceinline__ Item make_item(int w, const Schedule& sc) {
    const int tiles_n = sc.tiles_n, tiles_m = sc.tiles_m, splitk = sc.splitk, KB = sc.KB;
    int half = -1;
    const int full = tiles_n * tiles_m * splitk - sc.tail_split;      // tail_split > 0 only with splitk == 1
    if (w >= full) {
        const int j = w - full;
        w = full + (j >> 1);
        half = j & 1;
    }
    const int tile = w / splitk;
    const int ks = w - tile * splitk;
    const int per_group = kGroupN * tiles_m;
    const int g = tile / per_group;
    const int first_n = g * kGroupN;
    const int gsz = min(kGroupN, tiles_n - first_n);
    const int r = tile - g * per_group;
    Item it;
    it.n_blk = first_n + r % gsz;
    it.m_blk = r / gsz;
    it.ks = ks;
    it.half = half;
    it.kb0 = static_cast<int>(static_cast<int64_t>(ks) * KB / splitk);
    it.kb1 = static_cast<int>(static_cast<int64_t>(ks + 1) * KB / splitk);
    return it;
}

// (1024 + q) pairs -> fp16((q - zp) * s), exactly rounded once.
__device__ __forceinline__ uint32_t dq_pair(uint32_t lo, uint32_t hi, uint32_t sel, __half2 bias, __half2 s2) {
    uint32_t w = __byte_perm(lo, hi, sel);
    uint32_t h;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(h) : "r"(w));
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h), bias), s2);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

#ifdef TB200_ROLE_CYCLES
// Sums of clock64 intervals per role, CTA 0 only.  [0..6] issuer (all issuer warps): loop back edge, wait (blocking, only
// when the probe said "not ready"), fence, first MMA, probes + slot arithmetic, remaining MMAs + commit, K blocks;
// [8..13] convert warps of TMEM lane quarter 0 (one per group): wait for the packed stage, loads + unpack + release,
// wait for the operand slot, tcgen05.st + arrive, loop overhead between visits, visits; [16] cycles from kernel start to
// the end of CTA 0's epilogue, [17] work items of CTA 0, [18] cycles the issuer spent between items.
__device__ unsigned long long g_w4_role_cycles[32];
extern "C" int tb200_w4a16_role_cycles(unsigned long long* host32, int clear) {
    if (cudaMemcpyFromSymbol(host32, g_w4_role_cycles, sizeof(unsigned long long) * 32) != cudaSuccess) return 1;
    if (clear) {
        unsigned long long z[32] = {};
        if (cudaMemcpyToSymbol(g_w4_role_cycles, z, sizeof(z)) != cudaSuccess) return 1;
    }
    return 0;
}
#define TB200_RC_ADD(slot, v) atomicAdd(&g_w4_role_cycles[slot], static_cast<unsigned long long>(v))
#endif

template <int MT, bool kPair = false>
__device__ __forceinline__ void gemm_w4a16_body(const CUtensorMap* __restrict__ tmap_act, const CUtensorMap* __restrict__ tmap_act_half,
                                                const CUtensorMap* __restrict__ tmap_w, const CUtensorMap* __restrict__ tmap_out,
                                                const __half* __restrict__ scales, __half* __restrict__ out,
                                                float* __restrict__ ws, int M, int N, int K, int groups_per_row,
                                                int kb_per_group, int64_t ldo, int64_t col_offset, int splitk,
                                                float zp_plus_1024, int tma_store, int tail_split, const PeerOut& peers,
                                                const PeerMaps* __restrict__ peer_maps) {
    using Cfg = W4Cfg<MT, kPair>;
    constexpr int SA = Cfg::kSA;
    constexpr int SW = Cfg::kSW;
    constexpr int AST = Cfg::kAStages;
    constexpr int DQ = Cfg::kDQ;
    constexpr int NACC = Cfg::kNAcc;
    constexpr int NI = Cfg::kNI;
    // With equally deep activation and operand rings a K block uses the same slot in both, so ONE barrier per
    // slot collects the activation copy (expect-tx arrival of the producer) and the four convert warps: the
    // issuer waits on, and probes, a single barrier per K block.
    constexpr bool kMerged = SA == AST;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* act_ring = smem;
    uint8_t* w_ring = smem + Cfg::kActRingBytes;
    uint8_t* store_tile = w_ring + Cfg::kWRingBytes;
    uint64_t* bar_afull = reinterpret_cast<uint64_t*>(store_tile + Cfg::kStoreBytes);
    uint64_t* bar_done = bar_afull + SA;      // MMAs of a K block complete: activation stage and operand stage free
    uint64_t* bar_wfull = bar_done + SA;      // packed-weight stage: TMA landed
    uint64_t* bar_wempty = bar_wfull + SW;    //                      convert warps have read it
    uint64_t* bar_ofull = bar_wempty + SW;    // TMEM operand stage written by the convert warps
    uint64_t* bar_dfull = bar_ofull + AST;    // accumulator complete
    uint64_t* bar_dempty = bar_dfull + 2;     // accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_dempty + 2);

    // The warp index and the tensor-memory base are the same in every lane; passing them through a shuffle tells
    // the compiler so, and everything derived from them (roles, ring slots, descriptors, loop counters) can live
    // in uniform registers — which is where the MMA and TMA instructions take their operands from.
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int KB = K / kBK;
    // CTA pair: the work list is walked by pairs; an item's n_blk counts 256-row weight tiles and CTA `rank`
    // of the pair owns the 128-row half n_blk * 2 + rank
    const int rank = kPair ? static_cast<int>(cluster_ctarank()) : 0;
    const int w_first = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int w_step = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int tiles_n = N / (kPair ? 2 * kBNW : kBNW);
    const int tiles_m = (M + MT - 1) / MT;
    const Schedule sched = make_schedule(tiles_n, tiles_m, splitk, KB, MT == 256 ? tail_split : 0);
    const int items = sched.items;
    auto item_of = [&](int w) {
        Item im = make_item(w, sched);
        if (kPair) im.n_blk = im.n_blk * 2 + rank;
        return im;
    };
    // accumulator of an item and how often it was used before (phase of its barriers)
    auto acc_of = [](uint32_t item_cnt) { return NACC == 1 ? 0 : static_cast<int>(item_cnt & 1); };
    auto acc_use = [](uint32_t item_cnt) { return NACC == 1 ? item_cnt : (item_cnt >> 1); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) { mbar_init(&bar_afull[s], kMerged ? (kPair ? 9 : 5) : 1); mbar_init(&bar_done[s], 1); }
        for (int s = 0; s < SW; ++s) { mbar_init(&bar_wfull[s], 1); mbar_init(&bar_wempty[s], 4); }
        for (int s = 0; s < AST; ++s) mbar_init(&bar_ofull[s], 4);
        for (int b = 0; b < 2; ++b) { mbar_init(&bar_dfull[b], NI); mbar_init(&bar_dempty[b], kPair ? 8 : 4); }
        mbar_fence_init();
        tma_prefetch_desc(tmap_act);
        if (MT == 256 && tail_split > 0) tma_prefetch_desc(tmap_act_half);
        tma_prefetch_desc(tmap_w);
        if (Cfg::kTmaStore && tma_store) tma_prefetch_desc(tmap_out);
    }
    static_assert(!kPair || kMerged, "the pair kernel uses the merged slot barrier");
    if (warp == 2) {
        if constexpr (kPair) { tmem_alloc_pair(tmem_slot, Cfg::kTmemCols); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();   // the other CTA's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    TB200_RC(const long long rc_start = clock64(); const bool rc_on = blockIdx.x == 0;)

    if (warp == 0) {
        // ---------------- activation TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int w = w_first; w < items && ok; w += w_step) {
                const Item im = item_of(w);
                for (int kb = im.kb0; kb < im.kb1; ++kb, ++it) {
                    const int s = it % SA;
                    if (!mbar_wait(&bar_done[s], ((it / SA) & 1) ^ 1, ST_WAIT_SMEM_EMPTY, kb)) { ok = false; break; }
                    if constexpr (kPair) {
                        // this CTA's half of the item's activation rows (128, or 64 of a half-height unit); the bytes
                        // of both CTAs are counted on the leader's barrier
                        const bool hu = im.half >= 0;
                        const uint32_t bytes = hu ? Cfg::kActStageBytes / 2 : Cfg::kActStageBytes;
                        const int row0 = hu ? im.m_blk * MT + im.half * 128 + rank * 64 : im.m_blk * MT + rank * 128;
                        if (rank == 0) mbar_expect_tx(&bar_afull[s], 2 * bytes);
                        tma_load_2d_pair(act_ring + s * Cfg::kActStageBytes, hu ? tmap_act_half : tmap_act, &bar_afull[s], kb * kBK, row0);
                    } else if (MT == 256 && im.half >= 0) {      // 128-row unit: the upper or lower half of the stage's box
                        mbar_expect_tx(&bar_afull[s], Cfg::kActStageBytes / 2);
                        tma_load_2d(act_ring + s * Cfg::kActStageBytes, tmap_act_half, &bar_afull[s], kb * kBK, im.m_blk * MT + im.half * 128);
                    } else {
                        mbar_expect_tx(&bar_afull[s], Cfg::kActStageBytes);
                        tma_load_2d(act_ring + s * Cfg::kActStageBytes, tmap_act, &bar_afull[s], kb * kBK, im.m_blk * MT);
                    }
                }
            }
            if (!ok) {   // give copies already in flight a bounded chance to land before the CTA exits
                for (int s = 0; s < SA; ++s) {
                    if (it > static_cast<uint32_t>(s)) {
                        uint32_t last = it - 1 - ((it - 1 - s) % SA);
                        // (short limit: with the merged barrier the phase also needs the convert warps, which
                        // may have left already)
                        (void)mbar_wait_limit(&bar_afull[s], (last / SA) & 1, ST_WAIT_SMEM_FULL, -1, 1ll << 22);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- packed-weight TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int w = w_first; w < items && ok; w += w_step) {
                const Item im = item_of(w);
                for (int kb = im.kb0; kb < im.kb1; ++kb, ++it) {
                    const int s = it % SW;
                    if (!mbar_wait(&bar_wempty[s], ((it / SW) & 1) ^ 1, ST_WAIT_SMEM_EMPTY, -kb - 1)) { ok = false; break; }
                    mbar_expect_tx(&bar_wfull[s], kWBytes);
                    tma_load_2d(w_ring + s * kWBytes, tmap_w, &bar_wfull[s], kb * (kBK / 2), im.n_blk * kBNW);
                }
            }
            if (!ok) {
                for (int s = 0; s < SW; ++s) {
                    if (it > static_cast<uint32_t>(s)) {
                        uint32_t last = it - 1 - ((it - 1 - s) % SW);
                        (void)mbar_wait(&bar_wfull[s], (last / SW) & 1, ST_WAIT_SMEM_FULL, -2);
                    }
                }
            }
        }
    } else if (warp >= Cfg::kMmaWarp0 && warp < Cfg::kMmaWarp0 + NI && rank == 0) {
        // ---------------- MMA issuers (CTA pair: in the leader CTA only) ----------------
        // The issuing thread is the pacemaker of the large tiles (four MMAs of 128 tensor-pipe cycles each per
        // K block leave it about 500 cycles for everything), so its loop carries no division, no branch
        // that is not needed and no wait that can be avoided: the K blocks of issuer `me` are the running
        // counts me, me + NI, ... across work items; ring slots and phases advance by addition; the shared-
        // memory descriptor is a base plus a slot offset; and the barriers of the NEXT block are probed
        // (non-blocking) between the first and second MMA of the current one, so the blocking wait
        // is skipped whenever the convert warps and the activation copies are ahead.
        // The WHOLE warp walks the loop (waits, probes, slot arithmetic are warp-uniform); only the MMAs and the
        // commits are issued by lane 0.  Running the loop inside an `if (lane == 0)` region instead made every
        // branch of the lone thread cost 100-250 cycles (measured with the cycle counter: 257 cycles for the loop's
        // back edge, 95 for a not-taken `if`), which alone held the 256-row tile to about half the tensor rate.
        {
            const bool leader = lane == 0;
            const uint32_t me = warp - Cfg::kMmaWarp0;
            constexpr uint32_t kMmaM = kPair ? 2 * kBNW : kBNW;           // weight rows per MMA (both CTAs of a pair)
            constexpr uint32_t idesc_full = umma_idesc(0, 0, kMmaM, MT);  // f16 x f16 -> f32, N = MT
            constexpr uint32_t idesc_half = umma_idesc(0, 0, kMmaM, 128); // N = 128 for a half unit of the 256-row tile
            constexpr uint32_t kStageDesc = Cfg::kActStageBytes >> 4;     // one activation stage in descriptor units
            static_assert(NI <= SA && NI <= AST, "an issuer advances by NI slots per K block");
            const uint64_t b_desc0 = umma_desc_sw128(smem_u32(act_ring));
            const uint32_t a_tmem0 = tmem_base + Cfg::kACol0;
            uint32_t my_it = me;                 // running count of my next K block
            uint32_t sa = me, pa = 0;            // its activation slot and phase
            uint32_t so = me, po = 0;            // its operand slot and phase
            uint32_t it0 = 0, item_cnt = 0;
            bool ready = false;                  // my next block's barriers were seen complete already
            bool ok = true;
            TB200_RC(long long rc[7] = {0, 0, 0, 0, 0, 0, 0}; long long rc_prev = 0, rc_item = 0, rc_between = 0;)
            for (int w = w_first; w < items && ok; w += w_step, ++item_cnt) {
                const Item im = item_of(w);
                const uint32_t it_end = it0 + static_cast<uint32_t>(im.kb1 - im.kb0);
                const int acc = acc_of(item_cnt);
                const uint32_t idesc = (MT == 256 && im.half >= 0) ? idesc_half : idesc_full;
                const uint32_t d_tmem = tmem_base + (acc * NI + me) * MT;
                // the accumulator set must have been drained before this item's first MMA overwrites it
                if (!mbar_wait(&bar_dempty[acc], (acc_use(item_cnt) & 1) ^ 1, ST_WAIT_TMEM_EMPTY, w)) { ok = false; break; }
                uint32_t accumulate = 0u;
                TB200_RC(if (rc_item) rc_between += clock64() - rc_item; rc_prev = 0;)
                while (my_it < it_end) {
                    TB200_RC(const long long q0 = clock64(); if (rc_prev) rc[0] += q0 - rc_prev;)
                    if (!ready) {
                        const int kb = im.kb0 + static_cast<int>(my_it - it0);
                        if (!kMerged && !mbar_wait(&bar_ofull[so], po, ST_WAIT_OPERAND, kb)) { ok = false; break; }
                        if (!mbar_wait(&bar_afull[sa], pa, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                    }
                    TB200_RC(const long long q1 = clock64();)
                    tc_fence_after();
                    TB200_RC(const long long q2 = clock64();)
                    const uint32_t a_tmem = a_tmem0 + so * 32;
                    const uint64_t b_desc = b_desc0 + sa * kStageDesc;
                    uint64_t* const done = &bar_done[sa];
                    sa += NI; if (sa >= static_cast<uint32_t>(SA)) { sa -= SA; pa ^= 1; }
                    so += NI; if (so >= static_cast<uint32_t>(AST)) { so -= AST; po ^= 1; }
                    // 16 fp16 of K = 8 TMEM columns of the operand, 32 bytes of the swizzled smem row
                    if constexpr (kPair) {
                        if (leader) umma_f16_ts_pair(d_tmem, a_tmem, b_desc, idesc, accumulate);
                    } else {
                        umma_f16_ts_if(leader, d_tmem, a_tmem, b_desc, idesc, accumulate);
                    }
                    TB200_RC(const long long q3 = clock64();)
                    const bool next_o = kMerged ? true : mbar_test_wait(&bar_ofull[so], po);
                    const bool next_a = mbar_test_wait(&bar_afull[sa], pa);
                    TB200_RC(asm volatile("" ::"r"(static_cast<int>(next_o)), "r"(static_cast<int>(next_a)) : "memory"); const long long q4 = clock64();)
                    if constexpr (kPair) {
                        if (leader) {
#pragma unroll
                            for (int k = 1; k < kBK / 16; ++k) umma_f16_ts_pair(d_tmem, a_tmem + 8 * k, b_desc + 2 * k, idesc, 1u);
                            tc_commit_pair(done, 0x3);   // arrives in both CTAs of the pair
                        }
                    } else {
                        // predicated, not branched: only lane 0's instructions take effect
#pragma unroll
                        for (int k = 1; k < kBK / 16; ++k) umma_f16_ts_if(leader, d_tmem, a_tmem + 8 * k, b_desc + 2 * k, idesc, 1u);
                        // "MMAs of this K block complete": frees the activation slot and the operand slot
                        tc_commit_if(leader, done);
                    }
                    accumulate = 1u;
                    // (per lane, no warp vote: the lanes agree in practice, and a vote would have to wait for lanes whose
                    // bounded wait gave up in the rare case that others' succeeded)
                    ready = next_o && next_a;
                    my_it += NI;
                    TB200_RC(const long long q5 = clock64(); rc[1] += q1 - q0; rc[2] += q2 - q1; rc[3] += q3 - q2; rc[4] += q4 - q3;
                             rc[5] += q5 - q4; rc[6] += 1; rc_prev = q5;)
                }
                TB200_RC(rc_item = clock64();)
                if (ok && leader) {                   // one arrival per issuer; every issuer had >= 1 K block
                    if constexpr (kPair) tc_commit_pair(&bar_dfull[acc], 0x3);
                    else tc_commit(&bar_dfull[acc]);
                }
                it0 = it_end;
            }
            TB200_RC(if (rc_on && leader) { for (int i = 0; i < 7; ++i) TB200_RC_ADD(i, rc[i]);
                                            if (me == 0) { TB200_RC_ADD(17, item_cnt); TB200_RC_ADD(18, rc_between); } })
        }
    } else if (warp >= Cfg::kCvtWarp0 && warp < Cfg::kEpiWarp0) {
        // ---------------- convert warps: packed int4 (smem) -> fp16 operand (TMEM) ----------------
        const int grp = (warp - Cfg::kCvtWarp0) >> 2;    // which K blocks this group takes (it % DQ == grp)
        const int lane_grp = warp & 3;
        const int row = lane_grp * 32 + lane;            // weight row inside the tile == TMEM lane
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + Cfg::kACol0;
        const __half2 bias = __float2half2_rn(zp_plus_1024);
        // physical offset of this row's two 16-byte chunks under the 32-byte TMA swizzle
        const uint32_t swz = ((row >> 2) & 1) << 4;
        const uint32_t off0 = row * 32 + (0u ^ swz), off1 = row * 32 + (16u ^ swz);
        const uint32_t rt_zero = static_cast<uint32_t>(M) >> 31;   // 0, but not known to be before the kernel runs
        const int g_last = groups_per_row - 1;
        // scale of this thread's weight row for K block kb (clamped into the row, so look-ahead never leaves it)
        // (K blocks per scale group are a power of two for every group size in use: a shift instead of a division)
        const int kbpg_shift = (kb_per_group & (kb_per_group - 1)) == 0 ? 31 - __clz(kb_per_group) : -1;
        auto scale_kb = [&](const __half* srow, int kb) {
            const int g = kbpg_shift >= 0 ? kb >> kbpg_shift : kb / kb_per_group;
            return __ldg(srow + min(g, g_last));
        };
        auto scale_row = [&](const Item& im) {
            return scales + static_cast<int64_t>(im.n_blk * kBNW + row) * groups_per_row;
        };
        // Scales travel in a three-deep queue indexed by this group's VISITS (K blocks kb, kb + DQ, kb + 2 DQ):
        // a value is loaded two visits before it is used and only moved between registers a whole visit
        // after its load was issued, so no instruction waits on a load in flight whatever the ratio of
        // DQ to the K blocks per scale group.  The first three of the next work item are fetched while
        // the current one runs.
        // This group's K blocks are the running counts grp, grp + DQ, ... across work items; ring slots and
        // phases advance by addition (no division and no skipped iterations in the loop).
        static_assert(DQ <= SW && DQ <= AST && DQ <= SA, "a convert group advances by DQ slots per visit");
        uint32_t my_it = grp;                            // running count of my next K block
        uint32_t sw = grp, phw = 0;                      // its packed-weight slot and phase
        uint32_t os = grp;                               // its operand slot
        // "MMAs complete" slot and phase of the block that used operand slot os before (running count
        // my_it - AST), meaningful from the first visit with my_it >= AST on
        uint32_t first_reuse = grp;
        while (first_reuse < static_cast<uint32_t>(AST)) first_reuse += DQ;
        uint32_t sd = (first_reuse - AST) % SA, pd = ((first_reuse - AST) / SA) & 1;
        __half s0, s1, s2, n0 = __half(), n1 = __half(), n2 = __half();
        if (w_first < items) {
            const Item im = item_of(w_first);
            const __half* srow = scale_row(im);
            const int kbf = im.kb0 + grp;
            n0 = scale_kb(srow, kbf); n1 = scale_kb(srow, kbf + DQ); n2 = scale_kb(srow, kbf + 2 * DQ);
        }
        uint32_t it0 = 0;
        bool ok = true;
        TB200_RC(long long rc[6] = {0, 0, 0, 0, 0, 0}; long long rc_prev = 0;)
        for (int w = w_first; w < items && ok; w += w_step) {
            const Item im = item_of(w);
            const uint32_t it_end = it0 + static_cast<uint32_t>(im.kb1 - im.kb0);
            const __half* srow = scale_row(im);
            s0 = n0; s1 = n1; s2 = n2;
            if (w + w_step < items) {
                const Item nx = item_of(w + w_step);
                const __half* nrow = scale_row(nx);
                const uint32_t rem = it_end > my_it ? it_end - my_it : 0u;
                const uint32_t my_next = my_it + (rem + DQ - 1) / DQ * DQ;      // my first K block past this item
                const int kbf = nx.kb0 + static_cast<int>(my_next - it_end);
                n0 = scale_kb(nrow, kbf); n1 = scale_kb(nrow, kbf + DQ); n2 = scale_kb(nrow, kbf + 2 * DQ);
            }
            for (; my_it < it_end; my_it += DQ) {
                const int kb = im.kb0 + static_cast<int>(my_it - it0);
                const __half s_cur = s0;
                s0 = s1; s1 = s2; s2 = scale_kb(srow, kb + 3 * DQ);
                TB200_RC(const long long q0 = clock64(); if (rc_prev) rc[4] += q0 - rc_prev;)
                if (!mbar_wait(&bar_wfull[sw], phw, ST_WAIT_SMEM_FULL, kb)) { ok = false; break; }
                TB200_RC(const long long q1 = clock64();)
                const uint8_t* wt = w_ring + sw * kWBytes;
                const uint4 p0 = *reinterpret_cast<const uint4*>(wt + off0);
                const uint4 p1 = *reinterpret_cast<const uint4*>(wt + off1);
                const __half2 s2h = __half2half2(s_cur);
                uint32_t frag[32];
                const uint32_t pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t lo = pw[i], hi = pw[i] >> 4;
                    frag[4 * i + 0] = dq_pair(lo, hi, 0x0400, bias, s2h);
                    frag[4 * i + 1] = dq_pair(lo, hi, 0x0501, bias, s2h);
                    frag[4 * i + 2] = dq_pair(lo, hi, 0x0602, bias, s2h);
                    frag[4 * i + 3] = dq_pair(lo, hi, 0x0703, bias, s2h);
                }
                // The packed stage may be released only when p0 / p1 have LANDED in registers.  An arrive that merely
                // follows the two loads in program order can be issued while they are still in flight, and the TMA
                // refill then overtakes them: a few weight rows of one K block come from the wrong block (seen as
                // run-to-run differences in single output columns, about one call in ten of a 7168-tile problem).
                // Placing the arrive after the unpack is not enough either — compiler and hardware are free to
                // move register arithmetic across it — so the barrier address is made to DEPEND on the loaded
                // words: they are ANDed with a zero that only exists at run time (the sign bit of M; a literal zero
                // would be folded away by the assembler), which the hardware can compute only once both 128-bit loads
                // have returned (a warp's load completes as a unit, so lane 0 suffices).
                const uint32_t landed = (p0.x ^ p1.x) & rt_zero;
                __syncwarp();
                if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(&bar_wempty[sw]) + landed));
                TB200_RC(asm volatile("" ::"r"(frag[0]), "r"(frag[15]), "r"(frag[31]) : "memory"); const long long q2 = clock64();)
                if (my_it >= static_cast<uint32_t>(AST)) {   // the MMAs that last read this operand stage
                    if (!mbar_wait(&bar_done[sd], pd, ST_WAIT_OPERAND, -kb - 1)) { ok = false; break; }
                    sd += DQ; if (sd >= static_cast<uint32_t>(SA)) { sd -= SA; pd ^= 1; }
                }
                TB200_RC(const long long q3 = clock64();)
                tc_fence_after();
                tmem_st32(t_lane + os * 32, frag);
                tmem_wait_st();                                  // warp-collective: every lane's stores have completed
                tc_fence_before();
                if (lane == 0) {
                    if constexpr (kPair) mbar_arrive_leader(&bar_afull[os]);
                    else mbar_arrive(kMerged ? &bar_afull[os] : &bar_ofull[os]);
                }
                sw += DQ; if (sw >= static_cast<uint32_t>(SW)) { sw -= SW; phw ^= 1; }
                os += DQ; if (os >= static_cast<uint32_t>(AST)) os -= AST;
                TB200_RC(const long long q4 = clock64(); rc[0] += q1 - q0; rc[1] += q2 - q1; rc[2] += q3 - q2; rc[3] += q4 - q3;
                         rc[5] += 1; rc_prev = q4;)
            }
            it0 = it_end;
        }
        TB200_RC(if (rc_on && lane == 0 && lane_grp == 0) for (int i = 0; i < 6; ++i) TB200_RC_ADD(8 + i, rc[i]);)
    } else if (warp >= Cfg::kEpiWarp0) {
        // ---------------- epilogue warps ----------------
        const int lane_grp = warp & 3;
        const int row = lane_grp * 32 + lane;
        const int epi_tid = threadIdx.x - Cfg::kEpiWarp0 * 32;
        constexpr int kChunk = MT >= 32 ? 32 : 16;
        uint32_t item_cnt = 0, it0 = 0;
        bool ok = true;
        bool store_pending = false;
        for (int w = w_first; w < items && ok; w += w_step, ++item_cnt) {
            const Item im = item_of(w);
            const int acc = acc_of(item_cnt);
            // issuer i wrote its accumulator in this item iff one of the item's K blocks (global
            // numbers it0 .. it0 + len - 1) is congruent to i modulo NI
            const uint32_t len = static_cast<uint32_t>(im.kb1 - im.kb0);
            const uint32_t first_issuer = it0 % NI;
            it0 += len;
            auto issuer_active = [&](int i) { return len >= static_cast<uint32_t>(NI) || ((i + NI - first_issuer) % NI) < len; };
            if (!mbar_wait(&bar_dfull[acc], acc_use(item_cnt) & 1, ST_WAIT_TMEM_FULL, w)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + acc * NI * MT;
            const int64_t n = static_cast<int64_t>(im.n_blk) * kBNW + row;
            // v[] = sum over the issuers' private accumulators, always in issuer order
            auto load_sum = [&](uint32_t col, auto& v) {
                constexpr int W = sizeof(v) / sizeof(v[0]);
                if constexpr (W == 32) tmem_ld32(t_lane + col, v); else tmem_ld16(t_lane + col, v);
                tmem_wait_ld();
                if (NI > 1 && !issuer_active(0)) {
#pragma unroll
                    for (int j = 0; j < W; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int i = 1; i < NI; ++i) {
                    if (!issuer_active(i)) continue;
                    uint32_t u[W];
                    if constexpr (W == 32) tmem_ld32(t_lane + i * MT + col, u); else tmem_ld16(t_lane + i * MT + col, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < W; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                }
            };
            if (Cfg::kTmaStore && tma_store) {
                // D^T holds [n = lane][m = column]; the output wants rows of n.  Each thread writes its
                // column of a [128 m x 128 n] fp16 tile in shared memory (a warp writes 64 contiguous
                // bytes per m), and one TMA store per 128 rows of m moves the tile out, clipped at M.
                __half* tile = reinterpret_cast<__half*>(store_tile);
                const int passes = (MT == 256 && im.half >= 0) ? 1 : MT / 128;   // 128-row passes over the accumulator
                const int first_half = im.half >= 0 ? im.half : 0;
#pragma unroll 1
                for (int h = 0; h < passes; ++h) {
                    const int row0 = im.m_blk * MT + (first_half + h) * 128;
                    if (row0 >= M) break;
                    if (store_pending) {                     // the previous store must have read the tile
                        if (epi_tid == 0) tma_store_wait_read<0>();
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        store_pending = false;
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        load_sum(h * 128 + c * 32, v);
                        if (h == passes - 1 && c == 3) {     // accumulator fully read: release it
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) { if constexpr (kPair) mbar_arrive_leader(&bar_dempty[acc]); else mbar_arrive(&bar_dempty[acc]); }
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) tile[(c * 32 + j) * kBNW + row] = __float2half_rn(__uint_as_float(v[j]));
                    }
                    fence_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (epi_tid == 0) {
                        tma_store_2d(tmap_out, tile, im.n_blk * kBNW, row0);
                        if (peers.use_tma)      // the same tile to every other rank, in the same bulk group (plain stores, no multicast)
                            for (int p = 0; p < peers.count; ++p) tma_store_2d(&peer_maps->m[p], tile, im.n_blk * kBNW, row0);
                        tma_store_commit();
                    }
                    store_pending = true;
                    if (peers.count > 0 && !peers.use_tma) {
                        // the same tile to every other rank: 16 threads write one 256-byte row, 128-bit stores
                        const int rows_valid = min(128, M - row0);
                        for (int p = 0; p < peers.count; ++p) {
                            __half* dst = peers.base[p] + static_cast<int64_t>(row0) * ldo + im.n_blk * kBNW;
                            for (int idx = epi_tid; idx < rows_valid * 16; idx += 128) {
                                const int r = idx >> 4, c = idx & 15;
                                const uint4 v = *reinterpret_cast<const uint4*>(tile + r * kBNW + c * 8);
                                *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * ldo + c * 8) = v;
                            }
                        }
                    }
                }
                // an item whose last pass lies beyond M never reached the release above
                if (im.m_blk * MT + (first_half + passes - 1) * 128 >= M) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { if constexpr (kPair) mbar_arrive_leader(&bar_dempty[acc]); else mbar_arrive(&bar_dempty[acc]); }
                }
            } else {
                const int unit_rows = (MT == 256 && im.half >= 0) ? 128 : MT;
                const int unit_row0 = im.m_blk * MT + (im.half > 0 ? 128 : 0);
#pragma unroll
                for (int c = 0; c < MT / kChunk; ++c) {
                    const int m0 = unit_row0 + c * kChunk;
                    if (c * kChunk < unit_rows && m0 < M) {
                        uint32_t v[kChunk];
                        load_sum(c * kChunk, v);
                        if (splitk == 1) {
                            __half* dst = out + col_offset + n;
#pragma unroll
                            for (int j = 0; j < kChunk; ++j)
                                if (m0 + j < M) dst[static_cast<int64_t>(m0 + j) * ldo] = __float2half_rn(__uint_as_float(v[j]));
                        } else {
                            float* dst = ws + static_cast<int64_t>(im.ks) * M * N + n;
#pragma unroll
                            for (int j = 0; j < kChunk; ++j)
                                if (m0 + j < M) dst[static_cast<int64_t>(m0 + j) * N] = __uint_as_float(v[j]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { if constexpr (kPair) mbar_arrive_leader(&bar_dempty[acc]); else mbar_arrive(&bar_dempty[acc]); }
            }
        }
        if (store_pending && epi_tid == 0) tma_store_wait<0>();   // global writes complete before exit
        TB200_RC(if (rc_on && epi_tid == 0) TB200_RC_ADD(16, clock64() - rc_start);)
        if (peers.count > 0) __threadfence_system();              // peer stores visible beyond this GPU
    }

    // (pair: neither CTA may leave while the other can still read its shared or tensor memory or signal its barriers)
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();
    tc_fence_after();
    if (warp == 2) {
        __syncwarp();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
        else tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

#define TB200_W4_KERNEL(MT)                                                                                        \
    extern "C" __global__ void __launch_bounds__(W4Cfg<MT>::kThreads, 1) tb200_k_gemm_w4a16_m##MT(                 \
        const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_act_half,           \
        const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_out,                  \
        const __half* scales, __half* out, float* ws, int M, int N, int K, int gpr, int kbpg, int64_t ldo,         \
        int64_t col_offset, int splitk, float zp1024, int tma_store, int tail_split, const PeerOut peers,          \
        const __grid_constant__ PeerMaps peer_maps) {                                                              \
        gemm_w4a16_body<MT>(&tmap_act, &tmap_act_half, &tmap_w, &tmap_out, scales, out, ws, M, N, K, gpr, kbpg,    \
                            ldo, col_offset, splitk, zp1024, tma_store, tail_split, peers, &peer_maps);            \
    }
TB200_W4_KERNEL(16)
TB200_W4_KERNEL(64)
TB200_W4_KERNEL(128)
TB200_W4_KERNEL(256)

// CTA-pair form of the 256-row tile (see W4Cfg): a cluster of two CTAs per 256 x 256 work item.
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W4Cfg<256, true>::kThreads, 1) tb200_k_gemm_w4a16_pair(
    const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_act_half,
    const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_out, const __half* scales,
    __half* out, float* ws, int M, int N, int K, int gpr, int kbpg, int64_t ldo, int64_t col_offset, int splitk,
    float zp1024, int tma_store, int tail_split, const PeerOut peers, const __grid_constant__ PeerMaps peer_maps) {
    gemm_w4a16_body<256, true>(&tmap_act, &tmap_act_half, &tmap_w, &tmap_out, scales, out, ws, M, N, K, gpr, kbpg, ldo,
                               col_offset, splitk, zp1024, tma_store, tail_split, peers, &peer_maps);
}

// out[m, col_offset + n] = fp16( ws[0][m][n] + ws[1][m][n] + ... ) — fixed order, 4 columns per thread.
extern "C" __global__ void __launch_bounds__(256)
tb200_k_splitk_reduce_f16(const float* __restrict__ ws, __half* __restrict__ out, int64_t M, int64_t N, int splitk,
                          int64_t ldo, int64_t col_offset) {
    const int64_t n4 = N / 4;
    const int64_t total = M * n4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t m = i / n4, c = (i - m * n4) * 4;
        float4 acc = __ldg(reinterpret_cast<const float4*>(ws + m * N + c));
        for (int s = 1; s < splitk; ++s) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(ws + (static_cast<int64_t>(s) * M + m) * N + c));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
        __half* dst = out + m * ldo + col_offset + c;
        if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = o;
        } else {
            dst[0] = __low2half(lo); dst[1] = __high2half(lo); dst[2] = __low2half(hi); dst[3] = __high2half(hi);
        }
    }
}

TB200_DEFINE_STATUS_HOOKS(gemm_w4a16)

namespace {

// Activation-row tile (= MMA N).  17..64 rows: the 64-row tile with split-K only pays when there are few weight
// tiles to spread (n / 128 under half the SM count); otherwise the 128-row tile in one wave is faster although
// most of its MMA is padding, because the kernel is paced by the weight conversion, not by the MMA (measured at
// n = 14336, k = 4096: 34-44 us split against 27.5 us unsplit).
int pick_mt(int64_t m, int64_t n) {
    if (m <= 16) return 16;
    if (m <= 64) return (n / kBNW) * 2 > num_sms() ? 128 : 64;
    return m <= 128 ? 128 : 256;
}

// Shapes of at most kGemvMaxM activation rows go to the streaming mma.sync kernel (gemv_w4a16.cu).
constexpr int64_t kGemvMaxM = 16;
bool use_gemv(int64_t m, int64_t group) { return m <= kGemvMaxM && group % 128 == 0; }

// K split for the small-tile shapes (17 <= m <= 64), where there are fewer weight tiles than SMs:
// pick the split that fills whole waves of SMs best.  Every split keeps at least 4 K blocks, which
// also guarantees each MMA issuer thread its own block.
int pick_splitk(int64_t m, int64_t n, int64_t k) {
    const int mt = pick_mt(m, n);
    // m <= 16 never splits K: with group a multiple of 128 those shapes take the streaming kernel, and with
    // any other group the tensor-memory kernel runs unsplit, so that the workspace query (which does not
    // know the group) can promise "no workspace" for every decode-sized call
    if (mt > 64 || m <= kGemvMaxM) return 1;
    const int64_t tiles = (n / kBNW) * ((m + mt - 1) / mt);
    const int sms = num_sms();
    const int64_t KB = k / kBK;
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= 16; ++s) {
        if (KB / s < 4) break;
        const int64_t items = tiles * s;
        const int64_t waves = (items + sms - 1) / sms;
        const double eff = static_cast<double>(items) / static_cast<double>(waves * sms);
        if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    return best;
}

// Tensor maps of the peers' output slices ([m, n] fp16 at peers.base[p], row pitch ldo; 128 x 128 boxes like the local one).
int encode_peer_maps(PeerMaps* pm, const PeerOut& peers, int64_t m, int64_t n, int64_t ldo) {
    memset(pm, 0, sizeof(*pm));
    if (!peers.use_tma) return TB200_OK;
    for (int p = 0; p < peers.count; ++p) {
        const int rc = encode_tmap_2d(&pm->m[p], peers.base[p], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, n, ldo * 2, 128, kBNW,
                                      CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != TB200_OK) return rc;
    }
    return TB200_OK;
}

template <int MT, typename Kern>
int launch_w4(Kern kern, const void* a, const void* wp, const void* scales, void* out, float* ws, int64_t m, int64_t n,
              int64_t k, int64_t group, int zp, int64_t ldo, int64_t col_offset, int splitk, const PeerOut& peers,
              cudaStream_t st) {
    using Cfg = W4Cfg<MT>;
    static PerDeviceInt attr_set;
    {
        const int rc_attr = ensure_max_smem(attr_set, reinterpret_cast<const void*>(kern), Cfg::kSmemBytes);
        if (rc_attr != TB200_OK) return rc_attr;
    }
    CUtensorMap ta, tw, to;
    int rc = encode_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, k, k * 2, MT, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tw, wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k / 2, k / 2, kBNW, kBK / 2, CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc != TB200_OK) return rc;
    // TMA-store epilogue: the rank's output slice [m, n] at out + col_offset with row pitch ldo.  It needs a
    // 16-byte aligned base and pitch; otherwise the kernel stores from registers.
    __half* out_slice = static_cast<__half*>(out) + col_offset;
    int tma_store = Cfg::kTmaStore && splitk == 1 && aligned16(out_slice) && (ldo % 8 == 0);
    if (peers.count > 0 && !tma_store)
        return fail(TB200_ERR_UNSUPPORTED, "gemm_w4a16_gather: the fused gather needs m > 64 and 16-byte aligned output slices");
    if (tma_store) {
        rc = encode_tmap_2d(&to, out_slice, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, n, ldo * 2, 128, kBNW, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != TB200_OK) return rc;
    } else {
        to = ta;   // unused by the kernel
    }
    int64_t items = (n / kBNW) * ((m + MT - 1) / MT) * splitk;
    // 256-row tiles: when the last wave of the persistent grid would be at most half full, its tiles are cut
    // into two 128-row units each (see Schedule).  TB200_W4_TAIL=0 turns the cut off (tests compare both).
    int tail_split = 0;
    CUtensorMap tah = ta;
    if (MT == 256 && splitk == 1) {
        const int64_t rem = items % num_sms();
        const char* knob = getenv("TB200_W4_TAIL");
        if (rem > 0 && 2 * rem <= num_sms() && !(knob && knob[0] == '0')) {
            tail_split = static_cast<int>(rem);
            rc = encode_tmap_2d(&tah, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, k, k * 2, 128, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != TB200_OK) return rc;
        }
    }
    items += tail_split;
    PeerMaps pm;
    rc = encode_peer_maps(&pm, peers, m, n, ldo);
    if (rc != TB200_OK) return rc;
    const int grid = static_cast<int>(items < num_sms() ? items : num_sms());
    kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(ta, tah, tw, to, static_cast<const __half*>(scales), static_cast<__half*>(out), ws,
                                                        static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),
                                                        static_cast<int>(k / group), static_cast<int>(group / kBK), ldo,
                                                        col_offset, splitk, 1024.0f + static_cast<float>(zp), tma_store, tail_split, peers, pm);
    TB200_CUDA_TRY(cudaGetLastError());
    if (splitk > 1) {
        const int64_t total = m * (n / 4);
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
        if (blocks > cap) blocks = cap;
        tb200_k_splitk_reduce_f16<<<static_cast<unsigned>(blocks), 256, 0, st>>>(ws, static_cast<__half*>(out), m, n, splitk, ldo,
                                                                                 col_offset);
        TB200_CUDA_TRY(cudaGetLastError());
    }
    return TB200_OK;
}

// Launch of the CTA-pair kernel (m > 128, n a multiple of 256, no K split): as many pairs as can be resident at once
// (one CTA per SM, two SMs per pair), never more than there are work items.  The tail of the persistent schedule is
// cut into half-height units exactly like the single-CTA kernel's, counted in pairs.
int launch_w4_pair(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                   int64_t group, int zp, int64_t ldo, int64_t col_offset, const PeerOut& peers, cudaStream_t st) {
    using Cfg = W4Cfg<256, true>;
    static PerDeviceInt max_pairs_tab;
    int dev = 0;
    {
        const int rc_dev = current_device(&dev);
        if (rc_dev != TB200_OK) return rc_dev;
    }
    int max_pairs = max_pairs_tab.v[dev].load(std::memory_order_acquire);
    if (max_pairs == 0) {
        TB200_CUDA_TRY(cudaFuncSetAttribute(tb200_k_gemm_w4a16_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(num_sms() & ~1), 1, 1);
        cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        int clusters = 0;
        TB200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, tb200_k_gemm_w4a16_pair, &cfg));
        if (clusters < 1) return fail(TB200_ERR_UNSUPPORTED, "gemm_w4a16: no CTA pair fits on this device");
        max_pairs = clusters;
        max_pairs_tab.v[dev].store(clusters, std::memory_order_release);
    }
    CUtensorMap ta, tah, tw, to;
    // this CTA's half of the activation rows of a unit: 128 of 256, or 64 of a 128-row half unit
    int rc = encode_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, k, k * 2, 128, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tah, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, k, k * 2, 64, kBK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TB200_OK) return rc;
    rc = encode_tmap_2d(&tw, wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k / 2, k / 2, kBNW, kBK / 2, CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc != TB200_OK) return rc;
    __half* out_slice = static_cast<__half*>(out) + col_offset;
    rc = encode_tmap_2d(&to, out_slice, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, m, n, ldo * 2, 128, kBNW, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TB200_OK) return rc;
    int64_t items = (n / (2 * kBNW)) * ((m + 255) / 256);
    int tail_split = 0;
    {
        const int64_t rem = items % max_pairs;
        const char* knob = getenv("TB200_W4_TAIL");
        if (rem > 0 && 2 * rem <= max_pairs && !(knob && knob[0] == '0')) tail_split = static_cast<int>(rem);
    }
    items += tail_split;
    PeerMaps pm;
    rc = encode_peer_maps(&pm, peers, m, n, ldo);
    if (rc != TB200_OK) return rc;
    const int pairs = static_cast<int>(items < max_pairs ? items : max_pairs);
    tb200_k_gemm_w4a16_pair<<<2 * pairs, Cfg::kThreads, Cfg::kSmemBytes, st>>>(
        ta, tah, tw, to, static_cast<const __half*>(scales), static_cast<__half*>(out), nullptr, static_cast<int>(m),
        static_cast<int>(n), static_cast<int>(k), static_cast<int>(k / group), static_cast<int>(group / kBK), ldo, col_offset, 1,
        1024.0f + static_cast<float>(zp), 1, tail_split, peers, pm);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

// The pair kernel needs whole 256-row weight tiles and the TMA-store epilogue (16-byte aligned slice and pitch).
bool pair_usable(const void* out, int64_t n, int64_t ldo, int64_t col_offset) {
    return n % (2 * kBNW) == 0 && ldo % 8 == 0 && aligned16(static_cast<const __half*>(out) + col_offset);
}

}  // namespace

extern "C" size_t tb200_gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k <= 0 || n % kBNW != 0 || k % 128 != 0) return 0;
    if (m <= kGemvMaxM) return 0;                 // streaming kernel or unsplit tensor-memory kernel: no scratch
    const int s = pick_splitk(m, n, k);
    return s > 1 ? static_cast<size_t>(s) * m * n * sizeof(float) : 0;
}

namespace {
int gemm_w4a16_impl(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                    int64_t group, int zero_point, int64_t ldo, int64_t col_offset, void* workspace,
                    size_t workspace_bytes, const PeerOut& peers, void* stream) {
    clear_error();
    if (!a || !wp || !scales || !out) return fail(TB200_ERR_ARG, "gemm_w4a16: null pointer");
    if (m <= 0 || n <= 0 || k <= 0) return fail(TB200_ERR_ARG, "gemm_w4a16: non-positive size m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    if (n % kBNW != 0) return fail(TB200_ERR_ARG, "gemm_w4a16: n=%lld must be a multiple of 128", (long long)n);
    if (group <= 0 || group % kBK != 0 || k % group != 0 || k % 128 != 0)
        return fail(TB200_ERR_ARG, "gemm_w4a16: k=%lld must be a multiple of 128 and of group=%lld, group a multiple of 64", (long long)k, (long long)group);
    if (zero_point < 0 || zero_point > 15) return fail(TB200_ERR_ARG, "gemm_w4a16: zero_point %d outside 0..15", zero_point);
    if (col_offset < 0 || ldo < col_offset + n) return fail(TB200_ERR_ARG, "gemm_w4a16: ldo=%lld < col_offset+n=%lld", (long long)ldo, (long long)(col_offset + n));
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return fail(TB200_ERR_UNSUPPORTED, "gemm_w4a16: dimension too large");
    if (!aligned16(a) || !aligned16(wp)) return fail(TB200_ERR_ALIGN, "gemm_w4a16: a and wp must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (use_gemv(m, group) && peers.count == 0) {
        // decode-sized m: the TMA-ring streaming kernel when the activations fit beside the rings in shared
        // memory, else the register-staged one (TB200_GEMV_VARIANT=stream forces the latter; tests compare both)
        const char* knob = getenv("TB200_GEMV_VARIANT");
        const bool want_stream = knob && knob[0] == 's';
        if (!want_stream && gemv_ring_fits(m, k))
            return launch_gemv_w4a16_ring(a, wp, scales, out, m, n, k, group, zero_point, ldo, col_offset, st);
        return launch_gemv_w4a16(a, wp, scales, out, m, n, k, group, zero_point, ldo, col_offset, st);
    }
    const int splitk = pick_splitk(m, n, k);
    float* ws = nullptr;
    if (splitk > 1) {
        const size_t need = static_cast<size_t>(splitk) * m * n * sizeof(float);
        if (!workspace || workspace_bytes < need)
            return fail(TB200_ERR_WORKSPACE, "gemm_w4a16: needs %zu workspace bytes, got %zu", need, workspace ? workspace_bytes : 0);
        if (!aligned16(workspace)) return fail(TB200_ERR_ALIGN, "gemm_w4a16: workspace must be 16-byte aligned");
        ws = static_cast<float*>(workspace);
    }
    switch (pick_mt(m, n)) {
        case 16:  return launch_w4<16>(tb200_k_gemm_w4a16_m16, a, wp, scales, out, ws, m, n, k, group, zero_point, ldo, col_offset, splitk, peers, st);
        case 64:  return launch_w4<64>(tb200_k_gemm_w4a16_m64, a, wp, scales, out, ws, m, n, k, group, zero_point, ldo, col_offset, splitk, peers, st);
        case 128: return launch_w4<128>(tb200_k_gemm_w4a16_m128, a, wp, scales, out, ws, m, n, k, group, zero_point, ldo, col_offset, splitk, peers, st);
        default: {
            // TB200_W4_VARIANT = "pair" | "single" overrides the choice (a tuning and test aid)
            const char* knob = getenv("TB200_W4_VARIANT");
            const bool want_pair = knob && knob[0] == 'p';
            if (want_pair && pair_usable(out, n, ldo, col_offset))
                return launch_w4_pair(a, wp, scales, out, m, n, k, group, zero_point, ldo, col_offset, peers, st);
            return launch_w4<256>(tb200_k_gemm_w4a16_m256, a, wp, scales, out, ws, m, n, k, group, zero_point, ldo, col_offset, splitk, peers, st);
        }
    }
}
}  // namespace

extern "C" int tb200_gemm_w4a16(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n,
                                int64_t k, int64_t group, int zero_point, int64_t ldo, int64_t col_offset,
                                void* workspace, size_t workspace_bytes, void* stream) {
    return gemm_w4a16_impl(a, wp, scales, out, m, n, k, group, zero_point, ldo, col_offset, workspace, workspace_bytes,
                           PeerOut{}, stream);
}

extern "C" int tb200_gemm_w4a16_gather(const void* a, const void* wp_local, const void* scales_local,
                                       void* const* out_ptrs, int world, int rank, int64_t m, int64_t n_local, int64_t k,
                                       int64_t group, int zero_point, int64_t ldo, void* stream) {
    clear_error();
    if (!out_ptrs || world < 1 || world > kMaxPeers + 1 || rank < 0 || rank >= world)
        return fail(TB200_ERR_ARG, "gemm_w4a16_gather: bad world=%d rank=%d (1..%d ranks)", world, rank, kMaxPeers + 1);
    if (ldo < static_cast<int64_t>(world) * n_local)
        return fail(TB200_ERR_ARG, "gemm_w4a16_gather: ldo=%lld < world*n_local=%lld", (long long)ldo, (long long)(world * n_local));
    const int64_t col_offset = static_cast<int64_t>(rank) * n_local;
    PeerOut peers{};
    for (int r = 0; r < world; ++r)
        if (!out_ptrs[r]) return fail(TB200_ERR_ARG, "gemm_w4a16_gather: null output pointer for rank %d", r);
    // peers in the order rank + 1, rank + 2, ... (mod world): at any moment the ranks then store to DIFFERENT
    // destinations instead of all starting with rank 0
    for (int i = 1; i < world; ++i) {
        const int r = (rank + i) % world;
        __half* base = static_cast<__half*>(out_ptrs[r]) + col_offset;
        if (!aligned16(base)) return fail(TB200_ERR_ALIGN, "gemm_w4a16_gather: peer output slices must be 16-byte aligned");
        peers.base[peers.count++] = base;
    }
    // TB200_W4_GATHER=stores: the epilogue threads' own 128-bit peer stores instead of TMA stores (a tuning and test aid)
    const char* gk = getenv("TB200_W4_GATHER");
    peers.use_tma = (gk && gk[0] == 's') ? 0 : 1;
    return gemm_w4a16_impl(a, wp_local, scales_local, out_ptrs[rank], m, n_local, k, group, zero_point, ldo, col_offset,
                           nullptr, 0, peers, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the split-K partial sums live in a fixed array inside the library image.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = TB200_W4A16_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) float g_w4a16_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of g_w4a16_scratch, resolved once per device.  In host code the array's name is
// only a handle for the runtime; the pointer a kernel can use comes from cudaGetSymbolAddress.
int static_scratch_ptr(float** out) {
    static float* cached[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TB200_ERR_UNSUPPORTED, "gemm_w4a16_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_w4a16_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_w4a16_scratch)");
        cached[dev] = static_cast<float*>(p);
    }
    *out = cached[dev];
    return TB200_OK;
}
}  // namespace

extern "C" size_t tb200_gemm_w4a16_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int tb200_gemm_w4a16_static(const void* a, const void* wp, const void* scales, void* out, int64_t m,
                                       int64_t n, int64_t k, int64_t group, int zero_point, int64_t ldo,
                                       int64_t col_offset, void* stream) {
    clear_error();
    const size_t need = tb200_gemm_w4a16_workspace_bytes(m, n, k);
    if (need > kStaticScratchBytes)
        return fail(TB200_ERR_WORKSPACE,
                    "gemm_w4a16_static: m=%lld n=%lld k=%lld needs %zu scratch bytes, the built-in array holds %zu; "
                    "use tb200_gemm_w4a16 with a caller workspace",
                    (long long)m, (long long)n, (long long)k, need, kStaticScratchBytes);
    float* ws = nullptr;
    if (need > 0) {
        int rc = static_scratch_ptr(&ws);
        if (rc != TB200_OK) return rc;
    }
    return tb200_gemm_w4a16(a, wp, scales, out, m, n, k, group, zero_point, ldo, col_offset, ws, need, stream);
}
