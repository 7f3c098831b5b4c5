// Shared host/device helpers for the tb200 library: error reporting, the device status word,
// and thin inline-PTX wrappers for the sm_100a features the GEMM kernels use (mbarrier, TMA,
// tcgen05 MMA / TMEM).  Every wait is bounded: after a fixed number of polls it records a code in
// the status word and gives up, so a protocol bug shows as an error code, never as a hung GPU.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <atomic>

#include "../../include/tb200.h"

namespace tb200 {

// ---- host side -------------------------------------------------------------------------------
int  fail(int code, const char* fmt, ...);          // stores the message, returns code
void clear_error();
int  cuda_fail(cudaError_t e, const char* what);    // TB200_ERR_CUDA with the runtime's text
int  num_sms();                                     // SM count of the current device (cached per device)

// Per-device one-time set-up slots for launchers (thread-safe: two host threads making their first call
// together both see a consistent value).  kMaxDevices bounds the device index; larger indices are refused.
constexpr int kMaxDevices = 64;
struct PerDeviceInt {
    std::atomic<int> v[kMaxDevices];
};
// Current device index, or TB200_ERR_UNSUPPORTED (message set) when it does not fit the per-device tables.
int current_device(int* dev);
// Raises the dynamic shared-memory limit of `kern` on the current device the first time it is called there.
int ensure_max_smem(PerDeviceInt& done, const void* kern, int bytes);

#define TB200_CUDA_TRY(expr)                                              \
    do {                                                                  \
        cudaError_t e__ = (expr);                                         \
        if (e__ != cudaSuccess) return ::tb200::cuda_fail(e__, #expr);    \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Codes written to the device status word (detail = where).
enum : int {
    ST_OK = 0,
    ST_WAIT_SMEM_FULL = 1,   // consumer waited for a TMA stage that never landed
    ST_WAIT_SMEM_EMPTY = 2,  // producer waited for a stage the MMA never released
    ST_WAIT_TMEM_FULL = 3,   // drain warps waited for an accumulator that never completed
    ST_WAIT_TMEM_EMPTY = 4,  // MMA waited for an accumulator buffer that was never drained
    ST_WAIT_OPERAND = 5,     // MMA waited for a TMEM operand stage the convert warps never filled
    ST_WAIT_SELFTEST = 6,    // the self-test kernel's wait on a barrier nobody arrives on (expected to run out)
};

// The status word lives in the library image (one copy per translation unit that launches
// waiting kernels): no allocation.  read_status_words()/clear_status_words() in api.cu visit all.
#ifdef __CUDACC__
static __device__ int g_status[2];
#endif
struct StatusHooks {
    int (*read)(int* code, int* detail);
    int (*clear)();
};
void register_status_hooks(const StatusHooks& h);
// Defines this translation unit's accessors for its copy of g_status and registers them at load.
#define TB200_DEFINE_STATUS_HOOKS(tag)                                                            \
    static int status_read_##tag(int* code, int* detail) {                                       \
        int h[2] = {0, 0};                                                                        \
        cudaError_t e = cudaMemcpyFromSymbol(h, ::tb200::g_status, sizeof(h));                    \
        if (e != cudaSuccess) return ::tb200::cuda_fail(e, "cudaMemcpyFromSymbol(g_status)");     \
        *code = h[0];                                                                             \
        *detail = h[1];                                                                           \
        return TB200_OK;                                                                          \
    }                                                                                             \
    static int status_clear_##tag() {                                                             \
        int h[2] = {0, 0};                                                                        \
        cudaError_t e = cudaMemcpyToSymbol(::tb200::g_status, h, sizeof(h));                      \
        if (e != cudaSuccess) return ::tb200::cuda_fail(e, "cudaMemcpyToSymbol(g_status)");       \
        return TB200_OK;                                                                          \
    }                                                                                             \
    static const int status_registered_##tag =                                                    \
        (::tb200::register_status_hooks({status_read_##tag, status_clear_##tag}), 0);

#ifdef __CUDACC__
// ---- device side -----------------------------------------------------------------------------
__device__ __forceinline__ void record_status(int code, int detail) {
    if (atomicCAS(&g_status[0], 0, code) == 0) g_status[1] = detail;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Role cycle accounting (build variant -DTB200_ROLE_CYCLES, see tilebench_b200/profiling/role_cycles.py): statements
// wrapped in TB200_RC(...) exist only in that variant; the normal library contains none of them.
#ifdef TB200_ROLE_CYCLES
#define TB200_RC(...) __VA_ARGS__
#else
#define TB200_RC(...)
#endif

// Non-blocking probe of a phase (mbarrier.test_wait never suspends the thread): used to look at the NEXT
// stage's barriers between two instructions of the current one, so that the probe's latency is hidden and
// the blocking wait below is skipped when the answer was already "complete".
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: polls until the phase completes or kWaitCycles SM clock cycles have passed (about
// two seconds — far longer than any legitimate wait here, a whole kernel runs in milliseconds).
// The bound uses the SM-local cycle counter: reading it costs a few cycles, unlike the global
// nanosecond timer.  On expiry it records `code` and returns false; the caller unwinds and exits.
constexpr long long kWaitCycles = 1ll << 32;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int code, int detail, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (clock64() - t0 > limit_cycles) break;
    }
    record_status(code, detail);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code, int detail) {
    return mbar_wait_limit(bar, parity, code, detail, kWaitCycles);
}

// ---- TMA (tiled bulk tensor copy global -> shared, completion on an mbarrier) ----
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// All MMAs issued so far by this thread arrive on `bar` once they have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// ---- tcgen05.mma descriptors ----
// Shared-memory operand descriptor for a K-major tile stored with the 128-byte swizzle: rows of
// 128 bytes, 8-row groups 1024 bytes apart (stride byte offset), tile base 1024-byte aligned.
// Bits: [0,14) address>>4, [16,30) leading byte offset>>4 (unused for swizzled K-major, set to 1),
// [32,46) stride byte offset>>4, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor: [4,6) D format (1 = f32), [7,10) A format, [10,13) B format,
// [15] A major (0 = K), [16] B major (0 = K), [17,23) N>>3, [24,29) M>>4.
// kind::f16 formats: 0 = f16, 1 = bf16.  kind::f8f6f4 formats: 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Predicated forms for loops that the whole warp walks while one lane issues: every lane executes the
// statement, the instruction itself is guarded by `issue` (true in one lane), so the loop needs no
// divergent branch around its issue instructions.
__device__ __forceinline__ void umma_f16_ts_if(uint32_t issue, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
__device__ __forceinline__ void tc_commit_if(uint32_t issue, uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(smem_u32(bar)), "r"(issue)
        : "memory");
}

// ---- CTA pairs (cta_group::2): one MMA spans two SMs; the even CTA of the pair is the leader ----
// A shared-memory address of the executing CTA, as returned by smem_u32(), carries the CTA's rank in
// the cluster in bit 24; clearing it addresses the same offset in the even (leader) CTA of the pair.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load issued by either CTA of the pair into its own shared memory; the bytes are counted on the
// LEADER's barrier at the same offset.  Each CTA fetches its own box: nothing is broadcast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y)
        : "memory");
}
// Arrive on the leader CTA's copy of `bar` (a local arrive when executed by the leader).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerBitMask) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem, 128 rows per CTA] * B[smem, half of N per CTA]; issued by the leader only.
__device__ __forceinline__ void umma_f8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem of both CTAs] (+)= A[tmem, 128 lanes per CTA] * B[smem, half of N per CTA]; issued by the leader only.
__device__ __forceinline__ void umma_f16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// All MMAs issued so far by this thread arrive, once complete, on `bar` in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(cta_mask)
                 : "memory");
}
#endif  // __CUDACC__

// ---- host: launcher of the decode-sized W4A16 kernel (gemv_w4a16.cu), used by tb200_gemm_w4a16 -----
int launch_gemv_w4a16(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                      int64_t group, int zero_point, int64_t ldo, int64_t col_offset, cudaStream_t st);

// TMA-ring form of the same shape (gemv_w4a16_ring.cu): taken when the activations fit in shared memory.
bool gemv_ring_fits(int64_t m, int64_t k);
int launch_gemv_w4a16_ring(const void* a, const void* wp, const void* scales, void* out, int64_t m, int64_t n, int64_t k,
                           int64_t group, int zero_point, int64_t ldo, int64_t col_offset, cudaStream_t st);

// ---- host: TMA descriptor encoding through the driver entry point (no libcuda link) ----------
// 2-D row-major tensor [rows, cols] of elem_bytes-wide elements with row pitch `pitch_bytes`,
// box [box_rows, box_cols], given swizzle.  Returns TB200_OK or an error code.
int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                   uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                   CUtensorMapSwizzle swizzle);

}  // namespace tb200
