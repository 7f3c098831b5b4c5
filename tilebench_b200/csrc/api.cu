// Host-side plumbing of the tb200 C ABI: thread-local error text, device checks, the registry of
// per-translation-unit status words, and TMA descriptor encoding through the driver entry point.
#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>
#include <string.h>
#include <vector>

namespace tb200 {

static thread_local char t_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { t_error[0] = '\0'; }
int cuda_fail(cudaError_t e, const char* what) {
    return fail(TB200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int num_sms() {
    static PerDeviceInt cached;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = cached.v[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached.v[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int current_device(int* dev) {
    TB200_CUDA_TRY(cudaGetDevice(dev));
    if (*dev < 0 || *dev >= kMaxDevices)
        return fail(TB200_ERR_UNSUPPORTED, "device index %d is outside the library's per-device tables (0..%d)", *dev, kMaxDevices - 1);
    return TB200_OK;
}

int ensure_max_smem(PerDeviceInt& done, const void* kern, int bytes) {
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != TB200_OK) return rc;
    if (done.v[dev].load(std::memory_order_acquire) == 0) {
        // setting the attribute twice from two racing threads is harmless; the flag only saves the call
        TB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        done.v[dev].store(1, std::memory_order_release);
    }
    return TB200_OK;
}

static std::vector<StatusHooks>& hooks() {
    static std::vector<StatusHooks> h;
    return h;
}
void register_status_hooks(const StatusHooks& h) { hooks().push_back(h); }

int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes, uint64_t rows,
                   uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                   CUtensorMapSwizzle swizzle) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    });
    if (!encode) return fail(TB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_bytes & 15u) != 0)
        return fail(TB200_ERR_ALIGN, "TMA operand needs a 16-byte aligned base and row pitch (base=%p pitch=%llu)", base,
                    (unsigned long long)pitch_bytes);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    (void)elem_bytes;
    if (r != CUDA_SUCCESS) return fail(TB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return TB200_OK;
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_abi_version(void) { return TB200_ABI_VERSION; }
extern "C" const char* tb200_last_error(void) { return t_error; }

extern "C" int tb200_check_device(void) {
    clear_error();
    int dev = 0, major = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    TB200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(TB200_ERR_DEVICE, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);
    return TB200_OK;
}

extern "C" int tb200_device_status(int* code, int* detail) {
    clear_error();
    if (!code || !detail) return fail(TB200_ERR_ARG, "device_status: null pointer");
    *code = 0;
    *detail = 0;
    TB200_CUDA_TRY(cudaDeviceSynchronize());
    for (const StatusHooks& h : hooks()) {
        int c = 0, d = 0;
        int rc = h.read(&c, &d);
        if (rc != TB200_OK) return rc;
        if (c != 0 && *code == 0) {
            *code = c;
            *detail = d;
        }
    }
    return TB200_OK;
}

extern "C" int tb200_clear_device_status(void) {
    clear_error();
    TB200_CUDA_TRY(cudaDeviceSynchronize());
    for (const StatusHooks& h : hooks()) {
        int rc = h.clear();
        if (rc != TB200_OK) return rc;
    }
    return TB200_OK;
}
