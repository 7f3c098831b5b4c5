// Exchange step of the N-partitioned GEMM, and the self-test of the bounded waits.
//
// tb200_allgather_cols: every rank holds a column slice [m, n_local] of a row-major [m, world * n_local]
// result and pushes it into the same columns of every rank's full buffer (peer-mapped memory).  One
// streaming kernel per rank: 128-bit loads from this GPU's memory, 128-bit stores to each destination, so a
// slice lands at its final strided place and no staging buffer or interleave pass is needed.  Stores only —
// nothing here loads from another GPU, and no TMA or multicast instruction is used.
//
// tb200_selftest_bounded_wait: one warp waits on an mbarrier that nothing arrives on, with a caller-chosen
// cycle limit, so a test can watch the whole expiry path (status word, clean kernel exit, host read-back,
// clear) in a few microseconds without touching the production kernels or their two-second limit.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kMaxRanks = 8;
struct GatherDst {
    int count;
    uint8_t* base[kMaxRanks];     // already offset to this rank's columns
};

}  // namespace
}  // namespace tb200

using namespace tb200;

// rows of `row_bytes` (a multiple of 16) from src (pitch src_pitch) to every dst.base[p] (pitch dst_pitch).
extern "C" __global__ void __launch_bounds__(256)
tb200_k_allgather_cols_push(const uint8_t* __restrict__ src, const GatherDst dst, int64_t rows, int64_t row_bytes,
                            int64_t src_pitch, int64_t dst_pitch) {
    const int64_t chunks_per_row = row_bytes >> 4;
    const int64_t total = rows * chunks_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + r * src_pitch + (c << 4)));
#pragma unroll 1
        for (int p = 0; p < dst.count; ++p)
            *reinterpret_cast<uint4*>(dst.base[p] + r * dst_pitch + (c << 4)) = v;
    }
    __threadfence_system();     // stores to other GPUs are visible beyond this one before the kernel retires
}

extern "C" __global__ void tb200_k_selftest_bounded_wait(long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    // parity 0 completes only after one arrival, and nobody arrives: the wait must give up at the limit
    if (threadIdx.x == 0) (void)mbar_wait_limit(&bar, 0, ST_WAIT_SELFTEST, static_cast<int>(limit_cycles & 0x7fffffff), limit_cycles);
    __syncthreads();
}

TB200_DEFINE_STATUS_HOOKS(comm)

extern "C" int tb200_allgather_cols(const void* local, int64_t ld_local, void* const* out_ptrs, int world, int rank,
                                    int64_t m, int64_t n_local, int64_t elem_bytes, int64_t ldo, void* stream) {
    clear_error();
    if (!local || !out_ptrs) return fail(TB200_ERR_ARG, "allgather_cols: null pointer");
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
        return fail(TB200_ERR_ARG, "allgather_cols: bad world=%d rank=%d (1..%d ranks)", world, rank, kMaxRanks);
    if (m <= 0 || n_local <= 0 || elem_bytes <= 0) return fail(TB200_ERR_ARG, "allgather_cols: non-positive size");
    if (ld_local < n_local || ldo < static_cast<int64_t>(world) * n_local)
        return fail(TB200_ERR_ARG, "allgather_cols: ld_local=%lld < n_local=%lld or ldo=%lld < world*n_local", (long long)ld_local,
                    (long long)n_local, (long long)ldo);
    const int64_t row_bytes = n_local * elem_bytes, src_pitch = ld_local * elem_bytes, dst_pitch = ldo * elem_bytes;
    if (row_bytes % 16 != 0 || src_pitch % 16 != 0 || dst_pitch % 16 != 0 || !aligned16(local))
        return fail(TB200_ERR_ALIGN, "allgather_cols: slices, pitches and pointers must be multiples of 16 bytes");
    GatherDst dst{};
    const uint8_t* src = static_cast<const uint8_t*>(local);
    for (int r = 0; r < world; ++r)
        if (!out_ptrs[r]) return fail(TB200_ERR_ARG, "allgather_cols: null output pointer for rank %d", r);
    // destinations in the order rank, rank + 1, ... (mod world): at any moment the ranks then store to DIFFERENT GPUs
    for (int i = 0; i < world; ++i) {
        const int r = (rank + i) % world;
        uint8_t* base = static_cast<uint8_t*>(out_ptrs[r]) + static_cast<int64_t>(rank) * row_bytes;
        if (!aligned16(base)) return fail(TB200_ERR_ALIGN, "allgather_cols: output of rank %d is not 16-byte aligned", r);
        if (r == rank && base == src) continue;            // the slice was computed in place
        dst.base[dst.count++] = base;
    }
    if (dst.count == 0) return TB200_OK;
    const int64_t total = m * (row_bytes >> 4);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(num_sms()) * 8;
    if (blocks > cap) blocks = cap;
    tb200_k_allgather_cols_push<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst, m, row_bytes,
                                                                                                           src_pitch, dst_pitch);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}

extern "C" int tb200_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
    clear_error();
    if (limit_cycles <= 0 || limit_cycles > (1ll << 28))
        return fail(TB200_ERR_ARG, "selftest_bounded_wait: limit of %lld cycles outside 1..2^28 (about 0.15 s)", (long long)limit_cycles);
    tb200_k_selftest_bounded_wait<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles);
    TB200_CUDA_TRY(cudaGetLastError());
    return TB200_OK;
}
