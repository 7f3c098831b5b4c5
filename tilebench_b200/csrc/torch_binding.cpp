// PyTorch C++ extension over the tb200 C ABI.  It owns no kernels: each function checks the
// tensors (device, dtype, contiguity), unwraps data_ptr() and the current CUDA stream, and calls
// the matching extern "C" entry point of libtb200.so.  A nonzero return code becomes a Python
// exception carrying tb200_last_error(), which the benchmark engine records as `cuda_err`.
// Nothing here synchronises or allocates, so every call may run under CUDA-graph capture;
// outputs and workspaces are allocated by the Python caller with torch.empty.
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <stdexcept>
#include <string>

#include "tb200.h"

namespace {

void check_rc(int rc, const char* what) {
    if (rc == TB200_OK) return;
    std::string msg = std::string(what) + " failed (code " + std::to_string(rc) + "): " + tb200_last_error();
    if (rc == TB200_ERR_UNSUPPORTED) throw py::type_error(msg);
    if (rc == TB200_ERR_ARG || rc == TB200_ERR_ALIGN || rc == TB200_ERR_WORKSPACE) throw py::value_error(msg);
    throw std::runtime_error(msg);
}

void check_cuda(const torch::Tensor& t, const char* name, c10::ScalarType dt) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == dt, name, " has dtype ", t.scalar_type(), ", expected ", dt);
}

void* stream_of(const torch::Tensor& t) {
    return static_cast<void*>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

int dt_code(c10::ScalarType t) {
    switch (t) {
        case torch::kFloat32: return TB200_DT_F32;
        case torch::kFloat16: return TB200_DT_F16;
        case torch::kBFloat16: return TB200_DT_BF16;
        default: throw py::type_error("tb200: unsupported dtype");
    }
}

void dequant_int4_group(const torch::Tensor& wp, const torch::Tensor& scales, torch::Tensor& out, int64_t group,
                        int64_t zero_point) {
    check_cuda(wp, "wp", torch::kUInt8);
    check_cuda(scales, "scales", torch::kFloat16);
    check_cuda(out, "out", torch::kFloat16);
    TORCH_CHECK(wp.dim() == 2 && scales.dim() == 2 && out.dim() == 2, "dequant_int4_group: 2-D tensors expected");
    const int64_t n = wp.size(0), k = wp.size(1) * 2;
    TORCH_CHECK(out.size(0) == n && out.size(1) == k, "out must be [n, k]");
    TORCH_CHECK(group > 0 && scales.size(0) == n && scales.size(1) * group == k, "scales must be [n, k/group]");
    c10::cuda::CUDAGuard guard(wp.device());
    check_rc(tb200_dequant_int4_group(wp.data_ptr(), scales.data_ptr(), out.data_ptr(), n, k, group,
                                      static_cast<int>(zero_point), out.stride(0), stream_of(wp)),
             "tb200_dequant_int4_group");
}

void dequant_int8_rowwise(const torch::Tensor& w, const torch::Tensor& scale, torch::Tensor& out, bool use_post,
                          double post) {
    check_cuda(w, "w", torch::kInt8);
    check_cuda(scale, "scale", torch::kFloat32);
    TORCH_CHECK(out.is_cuda() && out.is_contiguous(), "out must be a contiguous CUDA tensor");
    TORCH_CHECK(w.dim() == 2 && scale.dim() == 1 && scale.size(0) == w.size(0), "w [rows, cols], scale [rows]");
    TORCH_CHECK(out.sizes() == w.sizes(), "out must match w's shape");
    const int dt = dt_code(out.scalar_type());
    c10::cuda::CUDAGuard guard(w.device());
    check_rc(tb200_dequant_int8_rowwise(w.data_ptr(), scale.data_ptr<float>(), out.data_ptr(), w.size(0), w.size(1), dt,
                                        use_post ? 1 : 0, static_cast<float>(post), stream_of(w)),
             "tb200_dequant_int8_rowwise");
}

void weight_dequant_block(const torch::Tensor& x, const torch::Tensor& s, torch::Tensor& y, int64_t m, int64_t n,
                          int64_t tile) {
    TORCH_CHECK(x.is_cuda() && s.is_cuda() && y.is_cuda(), "CUDA tensors expected");
    TORCH_CHECK(x.is_contiguous() && s.is_contiguous() && y.is_contiguous(), "contiguous tensors expected");
    TORCH_CHECK(x.scalar_type() == s.scalar_type() && x.scalar_type() == y.scalar_type(), "x, s, y must share a dtype");
    TORCH_CHECK(x.numel() == m * n && y.numel() == m * n, "x and y must hold m*n elements");
    TORCH_CHECK(tile > 0 && s.numel() == ((m + tile - 1) / tile) * ((n + tile - 1) / tile), "s must be [ceil(m/T), ceil(n/T)]");
    const int dt = dt_code(x.scalar_type());
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(tb200_weight_dequant_block(x.data_ptr(), s.data_ptr(), y.data_ptr(), m, n, tile, dt, stream_of(x)),
             "tb200_weight_dequant_block");
}

void gemm_fp8_blockscaled(const torch::Tensor& a, const torch::Tensor& sa, const torch::Tensor& b,
                          const torch::Tensor& sb, torch::Tensor& out) {
    check_cuda(a, "a", torch::kFloat8_e4m3fn);
    check_cuda(b, "b", torch::kFloat8_e4m3fn);
    check_cuda(sa, "sa", torch::kFloat32);
    check_cuda(sb, "sb", torch::kFloat32);
    check_cuda(out, "out", torch::kBFloat16);
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a [m,k], b [n,k]");
    const int64_t m = a.size(0), n = b.size(0), k = a.size(1);
    TORCH_CHECK(k % 128 == 0 && n % 128 == 0, "k and n must be multiples of 128");
    TORCH_CHECK(sa.dim() == 2 && sa.size(0) == m && sa.size(1) == k / 128, "sa must be [m, k/128]");
    TORCH_CHECK(sb.dim() == 2 && sb.size(0) == n / 128 && sb.size(1) == k / 128, "sb must be [n/128, k/128]");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == m && out.size(1) == n, "out must be [m, n]");
    c10::cuda::CUDAGuard guard(a.device());
    check_rc(tb200_gemm_fp8_blockscaled(a.data_ptr(), sa.data_ptr<float>(), b.data_ptr(), sb.data_ptr<float>(),
                                        out.data_ptr(), m, n, k, out.stride(0), stream_of(a)),
             "tb200_gemm_fp8_blockscaled");
}

int64_t gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    return static_cast<int64_t>(tb200_gemm_w4a16_workspace_bytes(m, n, k));
}

// out is the full [m, ldo] result; this call fills columns [col_offset, col_offset + n).
void gemm_w4a16(const torch::Tensor& a, const torch::Tensor& wp, const torch::Tensor& scales, torch::Tensor& out,
                int64_t group, int64_t zero_point, int64_t col_offset, const c10::optional<torch::Tensor>& workspace) {
    check_cuda(a, "a", torch::kFloat16);
    check_cuda(wp, "wp", torch::kUInt8);
    check_cuda(scales, "scales", torch::kFloat16);
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat16 && out.dim() == 2 && out.stride(1) == 1,
                "out must be a CUDA fp16 matrix with unit column stride");
    TORCH_CHECK(a.dim() == 2 && wp.dim() == 2 && a.size(1) == wp.size(1) * 2, "a [m,k], wp [n,k/2]");
    const int64_t m = a.size(0), k = a.size(1), n = wp.size(0);
    TORCH_CHECK(group > 0 && scales.dim() == 2 && scales.size(0) == n && scales.size(1) * group == k, "scales must be [n, k/group]");
    TORCH_CHECK(out.size(0) == m && col_offset >= 0 && out.size(1) >= col_offset + n, "out must be [m, >= col_offset + n]");
    void* ws = nullptr;
    size_t ws_bytes = 0;
    if (workspace.has_value() && workspace->defined() && workspace->numel() > 0) {
        TORCH_CHECK(workspace->is_cuda() && workspace->is_contiguous(), "workspace must be a contiguous CUDA tensor");
        ws = workspace->data_ptr();
        ws_bytes = static_cast<size_t>(workspace->numel()) * workspace->element_size();
    }
    c10::cuda::CUDAGuard guard(a.device());
    check_rc(tb200_gemm_w4a16(a.data_ptr(), wp.data_ptr(), scales.data_ptr(), out.data_ptr(), m, n, k, group,
                              static_cast<int>(zero_point), out.stride(0), col_offset, ws, ws_bytes, stream_of(a)),
             "tb200_gemm_w4a16");
}

// Fused GEMM + all-gather: out_ptrs[r] is the address of rank r's full [m, ldo] fp16 output (peer-mapped).
void gemm_w4a16_gather(const torch::Tensor& a, const torch::Tensor& wp, const torch::Tensor& scales,
                       const std::vector<int64_t>& out_ptrs, int64_t rank, int64_t ldo, int64_t group,
                       int64_t zero_point) {
    check_cuda(a, "a", torch::kFloat16);
    check_cuda(wp, "wp", torch::kUInt8);
    check_cuda(scales, "scales", torch::kFloat16);
    TORCH_CHECK(a.dim() == 2 && wp.dim() == 2 && a.size(1) == wp.size(1) * 2, "a [m,k], wp [n_local,k/2]");
    const int64_t m = a.size(0), k = a.size(1), n_local = wp.size(0);
    TORCH_CHECK(group > 0 && scales.dim() == 2 && scales.size(0) == n_local && scales.size(1) * group == k, "scales must be [n_local, k/group]");
    std::vector<void*> ptrs;
    for (int64_t p : out_ptrs) ptrs.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(p)));
    c10::cuda::CUDAGuard guard(a.device());
    check_rc(tb200_gemm_w4a16_gather(a.data_ptr(), wp.data_ptr(), scales.data_ptr(), ptrs.data(), static_cast<int>(ptrs.size()),
                                     static_cast<int>(rank), m, n_local, k, group, static_cast<int>(zero_point), ldo, stream_of(a)),
             "tb200_gemm_w4a16_gather");
}

// Pushes `local` [m, n_local] into columns [rank * n_local, ...) of every rank's full [m, ldo] buffer.
void allgather_cols(const torch::Tensor& local, const std::vector<int64_t>& out_ptrs, int64_t rank, int64_t ldo) {
    TORCH_CHECK(local.is_cuda() && local.dim() == 2 && local.stride(1) == 1, "local must be a CUDA matrix with unit column stride");
    std::vector<void*> ptrs;
    for (int64_t p : out_ptrs) ptrs.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(p)));
    c10::cuda::CUDAGuard guard(local.device());
    check_rc(tb200_allgather_cols(local.data_ptr(), local.stride(0), ptrs.data(), static_cast<int>(ptrs.size()), static_cast<int>(rank),
                                  local.size(0), local.size(1), local.element_size(), ldo, stream_of(local)),
             "tb200_allgather_cols");
}

void selftest_bounded_wait(int64_t limit_cycles) {
    check_rc(tb200_selftest_bounded_wait(limit_cycles, at::cuda::getCurrentCUDAStream().stream()), "tb200_selftest_bounded_wait");
}

void quantize_fp8_block(const torch::Tensor& x, torch::Tensor& q, torch::Tensor& scales, int64_t block_rows) {
    check_cuda(x, "x", torch::kFloat32);
    check_cuda(q, "q", torch::kFloat8_e4m3fn);
    check_cuda(scales, "scales", torch::kFloat32);
    TORCH_CHECK(x.dim() == 2 && q.sizes() == x.sizes(), "x and q must be [rows, cols]");
    TORCH_CHECK(block_rows > 0 && scales.numel() == (x.size(0) / block_rows) * (x.size(1) / 128), "scales must be [rows/block_rows, cols/128]");
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(tb200_quantize_fp8_block(x.data_ptr<float>(), q.data_ptr(), scales.data_ptr<float>(), x.size(0), x.size(1),
                                      static_cast<int>(block_rows), stream_of(x)),
             "tb200_quantize_fp8_block");
}

void matmul_int8_packed2(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out) {
    check_cuda(a, "a", torch::kInt8);
    check_cuda(b, "b", torch::kUInt8);
    check_cuda(out, "out", torch::kInt32);
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == 4 * b.size(0), "a [m,k], b [k/4,n]");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == a.size(0) && out.size(1) == b.size(1) && out.stride(1) == 1, "out must be [m,n]");
    c10::cuda::CUDAGuard guard(a.device());
    check_rc(tb200_matmul_int8_packed2(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.size(0), b.size(1), a.size(1),
                                       out.stride(0), stream_of(a)),
             "tb200_matmul_int8_packed2");
}

void matmul_plain(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "matmul_plain: tensors must be on a CUDA device");
    TORCH_CHECK(a.is_contiguous() && b.is_contiguous(), "matmul_plain: a and b must be contiguous");
    TORCH_CHECK(a.scalar_type() == b.scalar_type() && a.scalar_type() == out.scalar_type(), "matmul_plain: a, b, out must share a dtype");
    int dt = -1;
    if (a.scalar_type() == torch::kFloat32) dt = TB200_DT_F32;
    else if (a.scalar_type() == torch::kFloat16) dt = TB200_DT_F16;
    else if (a.scalar_type() == torch::kBFloat16) dt = TB200_DT_BF16;
    else if (a.scalar_type() == torch::kFloat8_e4m3fn) dt = TB200_DT_F8E4M3;
    if (dt < 0) throw py::type_error("matmul_plain: dtype must be float32, float16, bfloat16 or float8_e4m3fn");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(0), "a [m,k], b [k,n]");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == a.size(0) && out.size(1) == b.size(1) && out.stride(1) == 1, "out must be [m,n]");
    c10::cuda::CUDAGuard guard(a.device());
    check_rc(tb200_matmul_plain(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.size(0), b.size(1), a.size(1), dt,
                                out.stride(0), stream_of(a)),
             "tb200_matmul_plain");
}

void quantize_int4_group(const torch::Tensor& x, torch::Tensor& wp, torch::Tensor& scales, int64_t group, int64_t zero_point) {
    check_cuda(x, "x", torch::kFloat32);
    check_cuda(wp, "wp", torch::kUInt8);
    check_cuda(scales, "scales", torch::kFloat16);
    TORCH_CHECK(x.dim() == 2 && wp.dim() == 2 && wp.size(0) == x.size(0) && wp.size(1) * 2 == x.size(1), "x [n,k], wp [n,k/2]");
    TORCH_CHECK(group > 0 && scales.dim() == 2 && scales.size(0) == x.size(0) && scales.size(1) * group == x.size(1), "scales must be [n, k/group]");
    c10::cuda::CUDAGuard guard(x.device());
    check_rc(tb200_quantize_int4_group(x.data_ptr<float>(), wp.data_ptr(), scales.data_ptr(), x.size(0), x.size(1), group,
                                       static_cast<int>(zero_point), stream_of(x)),
             "tb200_quantize_int4_group");
}

py::tuple device_status() {
    int code = 0, detail = 0;
    check_rc(tb200_device_status(&code, &detail), "tb200_device_status");
    return py::make_tuple(code, detail);
}

void clear_device_status() { check_rc(tb200_clear_device_status(), "tb200_clear_device_status"); }
void check_device() { check_rc(tb200_check_device(), "tb200_check_device"); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "PyTorch binding of the tb200 C ABI (B200 quantized-inference kernels)";
    m.def("abi_version", &tb200_abi_version);
    m.def("check_device", &check_device);
    m.def("dequant_int4_group", &dequant_int4_group);
    m.def("dequant_int8_rowwise", &dequant_int8_rowwise);
    m.def("weight_dequant_block", &weight_dequant_block);
    m.def("gemm_fp8_blockscaled", &gemm_fp8_blockscaled);
    m.def("gemm_w4a16_workspace_bytes", &gemm_w4a16_workspace_bytes);
    m.def("gemm_w4a16", &gemm_w4a16);
    m.def("gemm_w4a16_gather", &gemm_w4a16_gather);
    m.def("allgather_cols", &allgather_cols);
    m.def("selftest_bounded_wait", &selftest_bounded_wait);
    m.def("quantize_fp8_block", &quantize_fp8_block);
    m.def("matmul_int8_packed2", &matmul_int8_packed2);
    m.def("matmul_plain", &matmul_plain);
    m.def("quantize_int4_group", &quantize_int4_group);
    m.def("device_status", &device_status);
    m.def("clear_device_status", &clear_device_status);
}
