/*
 * tb200.h — C ABI of the B200-native `cuda` backend for TileBench's quantized-inference path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, i.e. a
 * cudaStream_t; NULL = the legacy default stream).  Unless a comment says otherwise an entry point
 *   - validates its arguments on the host and returns a nonzero TB200_ERR_* code instead of launching,
 *   - enqueues its kernels on `stream` and returns without synchronising,
 *   - allocates nothing, so it may run under CUDA-graph capture (the reference's timer executes a
 *     backend's run() under capture: tilebench/core/timer.py:120-143),
 *   - never throws.  tb200_last_error() returns the message of the calling thread's last failure.
 *
 * The reference (TileBench) has no native code: its operator boundary is the Python function
 * `run(*inputs, **kw)` of tilebench/benchmarks/operators/<op>/impl_<backend>.py, driven by
 * tilebench/core/engine.py:337-366.  Each declaration below names the reference operator whose
 * run() it stands behind, or says that the operator is new (int4 / W4A16 / block-scaled FP8 do not
 * exist in the reference; they follow its operator contract).
 */
#ifndef TB200_H_
#define TB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_ABI_VERSION 1

/* Return codes. */
#define TB200_OK              0
#define TB200_ERR_ARG         1  /* null pointer, non-positive size, unsupported divisibility     */
#define TB200_ERR_ALIGN       2  /* pointer or leading dimension breaks a stated alignment         */
#define TB200_ERR_UNSUPPORTED 3  /* dtype / shape combination the kernels do not implement         */
#define TB200_ERR_CUDA        4  /* a CUDA runtime or driver call failed (message has the text)     */
#define TB200_ERR_WORKSPACE   5  /* workspace missing or too small                                  */
#define TB200_ERR_DEVICE      6  /* device is not sm_100 (B200)                                     */
#define TB200_ERR_TIMEOUT     7  /* a bounded in-kernel wait ran out (read back by tb200_device_status) */

/* Element types of tensors that cross the ABI. */
#define TB200_DT_F32  0
#define TB200_DT_F16  1
#define TB200_DT_BF16 2
#define TB200_DT_F8E4M3 3

int         tb200_abi_version(void);
/* Message of the calling thread's most recent failing call ("" if none). */
const char* tb200_last_error(void);
/* 0 when the current device is compute capability 10.x, TB200_ERR_DEVICE otherwise. */
int         tb200_check_device(void);

/* ---------------------------------------------------------------------------------------------
 * Streaming dequantisation (HBM-bound).
 * ------------------------------------------------------------------------------------------- */

/*
 * Per-group int4 weight dequantisation (new operator `dequant_int4_group`; the nearest reference
 * operator is weight_dequant, tilebench/benchmarks/operators/weight_dequant/impl_torch.py:4-8).
 *   wp      uint8 [n, k/2]          two nibbles per byte, low nibble = even k
 *   scales  fp16  [n, k/group]
 *   out     fp16  [n, ldo] (ldo >= k, in elements)
 *   out[r,c] = fp16( (q[r,c] - zero_point) * float(scales[r, c/group]) )   — one rounding, bit-exact
 * k must be even and a multiple of group; group a multiple of 8 selects the 128-bit vector kernel.
 */
int tb200_dequant_int4_group(const void* wp, const void* scales, void* out,
                             int64_t n, int64_t k, int64_t group, int zero_point,
                             int64_t ldo, void* stream);

/*
 * Per-row int8 dequantisation.  Serves the new operator `dequant_int8_channel`
 * (out = bf16(float(w) * scale[r])) and the reference operator dequantize_rowwise
 * (tilebench/benchmarks/operators/dequantize_rowwise/impl_torch.py:4-7:
 *  out = fp16((state_x[r] * float(x)) * float(1/127)), two fp32 roundings, in that order).
 *   w      int8 [rows, cols]      scale  fp32 [rows]      out  out_dtype [rows, cols]
 *   out_dtype  TB200_DT_F16 or TB200_DT_BF16
 *   use_post   nonzero: multiply the fp32 product by `post` (a second fp32 rounding) before the cast
 */
int tb200_dequant_int8_rowwise(const void* w, const float* scale, void* out,
                               int64_t rows, int64_t cols, int out_dtype,
                               int use_post, float post, void* stream);

/*
 * Float block-scale multiply — the reference operator weight_dequant
 * (tilebench/benchmarks/operators/weight_dequant/impl_torch.py:4-8): Y[i,j] = X[i,j] * S[i/T, j/T],
 * X, S, Y of one dtype (TB200_DT_F32 / F16 / BF16), S of shape [ceil(M/T), ceil(N/T)].
 */
int tb200_weight_dequant_block(const void* x, const void* s, void* y,
                               int64_t m, int64_t n, int64_t tile, int dtype, void* stream);

/*
 * FP8 e4m3 block quantiser — the step before tb200_gemm_fp8_blockscaled (the reference only has a cast,
 * tilebench/benchmarks/operators/quantize_global/impl_torch.py:4-5).  One fp32 scale = amax / 448 per
 * [block_rows x 128] block (1 for an all-zero block), q = e4m3(x / scale) rounded to nearest even.
 *   x fp32 [rows, cols]   q e4m3 [rows, cols]   scales fp32 [rows / block_rows, cols / 128]
 * block_rows is 1 (activations) or 128 (weights); cols a multiple of 128 (rows too when block_rows is 128);
 * x 32-byte and q 8-byte aligned (TB200_ERR_ALIGN otherwise).  Bit-exact against the same formula in PyTorch
 * for finite inputs; a NaN element is ignored by the block's amax (PyTorch's amax would propagate it).
 */
int tb200_quantize_fp8_block(const float* x, void* q, float* scales, int64_t rows, int64_t cols,
                             int block_rows, void* stream);

/*
 * int4 group quantiser — the step before tb200_dequant_int4_group / tb200_gemm_w4a16 (no counterpart in the
 * reference, whose quantiser operator is a plain cast, tilebench/benchmarks/operators/quantize_global/impl_torch.py:4-5).
 *   x fp32 [n, k]  ->  wp uint8 [n, k/2] (low nibble = even k), scales fp16 [n, k/128]
 *   s = fp16(amax / 7) per group of 128 (1 where that rounds to zero), q = clamp(rint(x / s) + 8, 0, 15)
 * group must be 128 and zero_point 8; x 32-byte and wp 4-byte aligned.  Bit-exact against the same formula
 * in PyTorch for finite inputs whose group amax / 7 stays inside the fp16 range (65504); NaN elements are
 * ignored by the amax, and a larger amax makes the fp16 scale infinite (every code of the group becomes 8).
 */
int tb200_quantize_int4_group(const float* x, void* wp, void* scales, int64_t n, int64_t k, int64_t group,
                              int zero_point, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Quantised GEMMs on tcgen05 tensor cores (TMA operands, TMEM accumulators).
 * ------------------------------------------------------------------------------------------- */

/*
 * FP8 e4m3 block-scaled GEMM (new operator `gemm_fp8_blockscaled`; the nearest reference operator
 * is the unit-scale fp8 branch of tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27).
 *   a   e4m3 [m, k]   sa fp32 [m, k/128]          (one scale per 1x128 block of A)
 *   b   e4m3 [n, k]   sb fp32 [n/128, k/128]      (one scale per 128x128 block of B)
 *   out bf16 [m, ldo] = bf16( sum_kb sa[i,kb] * sb[j/128,kb] * dot(a[i,kb*128:+128], b[j,kb*128:+128]) )
 * fp32 accumulation.  Any m >= 1; n and k multiples of 128; a, b, out 16-byte aligned.
 */
int tb200_gemm_fp8_blockscaled(const void* a, const float* sa, const void* b, const float* sb,
                               void* out, int64_t m, int64_t n, int64_t k, int64_t ldo,
                               void* stream);

/*
 * int8 x packed-2-bit GEMM — the reference operator `matmul_int8`
 * (tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19; generator tilebench/data/tensors.py:439-448).
 *   a    int8  [m, k]
 *   b    uint8 [k/4, n]: bits [2i, 2i+2) of b[kb, j] hold weight B[i * k/4 + kb, j] + 1, i = 0..3
 *   out  int32 [m, ldo]:  out[r, j] = sum_k a[r, k] * B[k, j],  B in {-1, 0, 1, 2}
 * Integer arithmetic on the tensor cores (tcgen05 kind::i8, int32 accumulation): the result is exact
 * whatever the summation order.  k a multiple of 256 and n of 128 (TB200_ERR_UNSUPPORTED otherwise),
 * ldo >= n and a multiple of 4; a, b, out 16-byte aligned.
 */
int tb200_matmul_int8_packed2(const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k,
                              int64_t ldo, void* stream);

/*
 * Plain GEMM out = a . b — the reference operator `matmul_fp32_fp16_fp8`
 * (tilebench/benchmarks/operators/matmul_fp32_fp16_fp8/impl_torch.py:21-27; generator
 * tilebench/data/tensors.py:416-436).  a [m, k] and b [k, n] row-major and of one type, out [m, ldo]:
 *   TB200_DT_F16     fp16 in, fp32 accumulation, fp16 out   (TB200_DT_BF16 likewise, bf16 out)
 *   TB200_DT_F32     fp32 in, read by the tensor cores as TF32 (the reference sets allow_tf32), fp32 out
 *   TB200_DT_F8E4M3  e4m3 in, unit scales, fp32 accumulation, out e4m3 = e4m3(bf16(sum)) as the reference's
 *                    _scaled_mm(out_dtype=bfloat16) followed by a cast gives; overflow becomes NaN as in PyTorch
 * b is consumed as stored (an MN-major tensor-core operand): no transposed copy is made or cached.
 * n a multiple of 128; k a multiple of 64 (fp16, bf16), 32 (fp32) or 128 (e4m3); a, b, out and the rows of out
 * 16-byte aligned.
 */
int tb200_matmul_plain(const void* a, const void* b, void* out, int64_t m, int64_t n, int64_t k, int dtype,
                       int64_t ldo, void* stream);

/*
 * W4A16 dequant-fused GEMM (new operator `gemm_w4a16`; structural template: the packed-weight
 * GEMM tilebench/benchmarks/operators/matmul_int8/impl_torch.py:4-19).
 *   a       fp16  [m, k]
 *   wp      uint8 [n, k/2], scales fp16 [n, k/group]   as in tb200_dequant_int4_group; group a multiple of 64
 *           that divides k (128 in the benchmark configurations)
 *   out     fp16  [m, ldo]; this call writes columns [col_offset, col_offset + n) — an N-partitioned
 *           rank passes its slice of wp/scales and the offset of its slice in the full output
 *   out[i, col_offset + j] = fp16( sum_k float(a[i,k]) * float(fp16((q[j,k]-zp) * scales[j,k/group])) )
 *   workspace  fp32 scratch for the split-K variant, which is chosen for 17 <= m <= 64 when the weight has few
 *              128-row tiles (n / 128 under half the SM count); size from tb200_gemm_w4a16_workspace_bytes(),
 *              which holds for every valid group; may be NULL when that returns 0 (always the case for
 *              m <= 16 and m > 64)
 * n a multiple of 128, k a multiple of 128.
 */
size_t tb200_gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k);
int    tb200_gemm_w4a16(const void* a, const void* wp, const void* scales, void* out,
                        int64_t m, int64_t n, int64_t k, int64_t group, int zero_point,
                        int64_t ldo, int64_t col_offset,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * N-partitioned W4A16 GEMM fused with the all-gather of its column slices (config `gemm_w4a16_npart`;
 * the reference has no multi-GPU path).  Rank `rank` of `world` owns weight rows
 * [rank * n_local, (rank + 1) * n_local); out_ptrs[r] is rank r's full output [m, ldo] (fp16, ldo >= world *
 * n_local), peer-mapped into this process for r != rank (symmetric memory / CUDA IPC).  The epilogue stores
 * every finished tile into columns [rank * n_local, ...) of ALL `world` buffers by TMA stores (one tensor map per
 * rank's slice; plain bulk stores, nothing is loaded from a peer and nothing is multicast; the environment
 * knob TB200_W4_GATHER=stores makes the epilogue threads push the tile with 128-bit stores instead) — so the
 * transfer overlaps the main loop.  Needs m > 64 and
 * 16-byte aligned slices (TB200_ERR_UNSUPPORTED otherwise: gather with NCCL instead).  Callers must put a
 * cross-rank barrier between this call and any read of the gathered buffer.  out_ptrs is a HOST array.
 */
int tb200_gemm_w4a16_gather(const void* a, const void* wp_local, const void* scales_local,
                            void* const* out_ptrs, int world, int rank, int64_t m, int64_t n_local, int64_t k,
                            int64_t group, int zero_point, int64_t ldo, void* stream);

/*
 * W4A16 GEMM for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * tb200_gemm_w4a16 asks its caller for a split-K workspace when m is small (17..64 rows) and the weight is
 * narrow (fewer rows take a streaming kernel that needs none).  Some callers have
 * no way to provide one: a plugin running inside a host process that has handed all device memory to its
 * own pool, or code invoked where cudaMalloc is not permitted.  This variant computes the same result
 * with the partial sums kept in a fixed array of TB200_W4A16_STATIC_SCRATCH_BYTES that is part of the
 * library image (every GPU that loads the library holds that much memory until the process exits).  It
 * calls no cudaMalloc / cudaFree and no allocating library routine; inputs and the output are still the
 * caller's buffers.
 *   - Shapes whose split-K partials exceed the array are rejected with TB200_ERR_WORKSPACE and a message
 *     giving both sizes; shapes that need no scratch (large m) run exactly like tb200_gemm_w4a16.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that
 *     device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Every
 *     partial sum a call reads is written by that same call first, so nothing has to be cleared; but two
 *     calls that overlap on the GPU (different streams, or concurrent graphs) race on it.  Serialise them.
 */
#define TB200_W4A16_STATIC_SCRATCH_BYTES (16u << 20)
size_t tb200_gemm_w4a16_static_scratch_bytes(void);
int    tb200_gemm_w4a16_static(const void* a, const void* wp, const void* scales, void* out,
                               int64_t m, int64_t n, int64_t k, int64_t group, int zero_point,
                               int64_t ldo, int64_t col_offset, void* stream);

/*
 * Exchange step of the N-partitioned GEMM without the GEMM: pushes this rank's column slice into every rank's
 * full result (the reference has no multi-GPU path; this is the unfused counterpart of tb200_gemm_w4a16_gather).
 *   local     [m, ld_local] elements of elem_bytes: this rank's slice, columns [0, n_local)
 *   out_ptrs  HOST array of `world` device pointers: rank r's full result [m, ldo], peer-mapped into this
 *             process for r != rank; the slice lands in columns [rank * n_local, (rank + 1) * n_local) of each.
 *             When out_ptrs[rank] already holds the slice at that place (local points there) it is not copied.
 * One streaming kernel: loads from this GPU, 128-bit stores to each destination; no staging buffer, no
 * interleave pass, no loads from another GPU.  Row slices, pitches and pointers must be multiples of 16 bytes.
 * Callers put a cross-rank barrier between this call and any read of a gathered buffer.
 */
int tb200_allgather_cols(const void* local, int64_t ld_local, void* const* out_ptrs, int world, int rank,
                         int64_t m, int64_t n_local, int64_t elem_bytes, int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Device status word.  Every wait inside the GEMM kernels (mbarrier, TMEM hand-off) is bounded;
 * a wait that runs out records a code here and the kernel drains and returns instead of hanging.
 * These two calls synchronise the device and must stay outside timed regions and graph capture.
 * ------------------------------------------------------------------------------------------- */
int tb200_device_status(int* code, int* detail);   /* code 0 = clean */
int tb200_clear_device_status(void);
/*
 * Self-test of that mechanism: launches one warp that waits, with a limit of `limit_cycles` SM clock cycles
 * (1 .. 2^28), on a barrier nothing ever arrives on.  The wait runs out, the kernel records status code 6 and
 * returns normally; tb200_device_status() then reports (6, limit) until tb200_clear_device_status().  The
 * context stays usable.  No counterpart in the reference.
 */
int tb200_selftest_bounded_wait(int64_t limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TB200_H_ */
