// C-ABI plumbing shared by all entry points: version, error strings, the
// per-thread error detail, and the fused linear chain that strings the producer
// kernel and the GEMM together over caller-provided scratch.

#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include <cuda.h>
#include <string.h>
#include "common.cuh"

namespace q8k {

static thread_local char g_error_detail[512] = "";

void set_error_detail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error_detail, sizeof(g_error_detail), fmt, ap);
    va_end(ap);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace q8k

using namespace q8k;

extern "C" int q8k_version(void) { return 100; }

extern "C" const char* q8k_error_string(int code) {
    switch (code) {
        case Q8K_OK: return "ok";
        case Q8K_ERR_INVALID_ARG: return "invalid argument";
        case Q8K_ERR_UNSUPPORTED: return "unsupported dtype or shape";
        case Q8K_ERR_WORKSPACE: return "workspace too small";
        case Q8K_ERR_CUDA: return "CUDA call failed";
        case Q8K_ERR_TOO_LARGE: return "problem exceeds a built-in capacity";
        default: return "unknown error";
    }
}

extern "C" const char* q8k_last_error_detail(void) { return g_error_detail; }

extern "C" size_t q8k_linear_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return align_up((size_t)M * (size_t)K, 256) + align_up((size_t)M * sizeof(float), 256);
}

extern "C" int q8k_linear(const void* x, int x_dtype, const void* w, int w_dtype, const float* w_scales,
                          const float* bias, void* out, int out_dtype, int M, int N, int K,
                          int use_hadamard, int fuse_gelu, void* workspace, size_t workspace_bytes,
                          int* dev_status, void* stream) {
    Q8K_REQUIRE(M >= 0 && N > 0 && K > 0, Q8K_ERR_INVALID_ARG, "linear: bad shape M=%d N=%d K=%d", M, N, K);
    if (M == 0) return Q8K_OK;
    Q8K_REQUIRE(w_dtype == Q8K_DT_I8 || w_dtype == Q8K_DT_E4M3, Q8K_ERR_UNSUPPORTED,
                "linear: weight dtype %d is not int8 or e4m3", w_dtype);
    Q8K_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0, Q8K_ERR_INVALID_ARG,
                "linear: workspace must be non-null and 256-byte aligned");
    Q8K_REQUIRE(workspace_bytes >= q8k_linear_workspace_bytes(M, K), Q8K_ERR_WORKSPACE,
                "linear: workspace of %zu bytes is smaller than the %zu needed for M=%d K=%d", workspace_bytes,
                q8k_linear_workspace_bytes(M, K), M, K);
    void* xq = workspace;
    float* x_scales = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + align_up((size_t)M * K, 256));
    int rc;
    if (use_hadamard) {
        rc = q8k_hadamard_quant(x, x_dtype, xq, w_dtype, x_scales, M, K, K, (float)(1.0 / sqrt((double)K)), stream);
    } else {
        rc = q8k_tokenwise_quant(x, x_dtype, xq, w_dtype, x_scales, M, K, K, stream);
    }
    if (rc != Q8K_OK) return rc;
    if (w_dtype == Q8K_DT_I8)
        return q8k_q8_mm(xq, w, bias, x_scales, w_scales, out, out_dtype, 1, 1, M, N, K, fuse_gelu, dev_status, stream);
    return q8k_fp8_mm(xq, w, bias, x_scales, w_scales, out, out_dtype, 1, 1, M, N, K, fuse_gelu, dev_status, stream);
}


// ------------------------------------------------------------------ q8k_linear_static
// Scratch for the allocation-free variant of q8k_linear: the quantised activations of one call
// followed by their per-row scales.  The array is part of the library image, so every GPU that
// loads the library carries it until the process exits.
namespace q8k {
constexpr size_t kStaticQuantBytes = (size_t)Q8K_LINEAR_STATIC_MAX_MK;                 // M*K bytes, 8-bit activations
constexpr size_t kStaticScaleBytes = (size_t)Q8K_LINEAR_STATIC_MAX_M * sizeof(float);  // one fp32 scale per row
static __device__ __align__(256) unsigned char g_linear_static_scratch[kStaticQuantBytes + kStaticScaleBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_ptr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

// In host code the array's name is only a handle.  The device address is looked up once per device,
// with that device current, and cached.
static int static_scratch_address(void** out) {
    int dev = -1;
    Q8K_CUDA_OK(cudaGetDevice(&dev));
    Q8K_REQUIRE(dev >= 0 && dev < kMaxDevices, Q8K_ERR_UNSUPPORTED, "linear_static: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        Q8K_CUDA_OK(cudaGetSymbolAddress(&ptr, g_linear_static_scratch));
        Q8K_REQUIRE(ptr != nullptr && (reinterpret_cast<uintptr_t>(ptr) & 255) == 0, Q8K_ERR_CUDA,
                    "linear_static: scratch symbol resolved to a null or misaligned address");
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return Q8K_OK;
}
}  // namespace q8k

extern "C" int q8k_linear_static(const void* x, int x_dtype, const void* w, int w_dtype, const float* w_scales,
                                 const float* bias, void* out, int out_dtype, int M, int N, int K,
                                 int use_hadamard, int fuse_gelu, int* dev_status, void* stream) {
    Q8K_REQUIRE(M >= 0 && N > 0 && K > 0, Q8K_ERR_INVALID_ARG, "linear_static: bad shape M=%d N=%d K=%d", M, N, K);
    if (M == 0) return Q8K_OK;
    Q8K_REQUIRE(w_dtype == Q8K_DT_I8 || w_dtype == Q8K_DT_E4M3, Q8K_ERR_UNSUPPORTED,
                "linear_static: weight dtype %d is not int8 or e4m3", w_dtype);
    Q8K_REQUIRE((size_t)M * (size_t)K <= kStaticQuantBytes && (size_t)M <= (size_t)Q8K_LINEAR_STATIC_MAX_M,
                Q8K_ERR_TOO_LARGE,
                "linear_static: M=%d K=%d exceeds the built-in scratch (M*K <= %zu and M <= %d); use q8k_linear "
                "with a caller-provided workspace", M, K, kStaticQuantBytes, Q8K_LINEAR_STATIC_MAX_M);
    void* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // Layout inside the scratch: [0, M*K) quantised rows, then the scales at a fixed offset.  Both
    // regions are fully written by the producer kernel before the GEMM reads them, so nothing has
    // to be cleared between calls.
    void* xq = scratch;
    float* x_scales = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + kStaticQuantBytes);
    int rc;
    if (use_hadamard) {
        rc = q8k_hadamard_quant(x, x_dtype, xq, w_dtype, x_scales, M, K, K, (float)(1.0 / sqrt((double)K)), stream);
    } else {
        rc = q8k_tokenwise_quant(x, x_dtype, xq, w_dtype, x_scales, M, K, K, stream);
    }
    if (rc != Q8K_OK) return rc;
    if (w_dtype == Q8K_DT_I8)
        return q8k_q8_mm(xq, w, bias, x_scales, w_scales, out, out_dtype, 1, 1, M, N, K, fuse_gelu, dev_status, stream);
    return q8k_fp8_mm(xq, w, bias, x_scales, w_scales, out, out_dtype, 1, 1, M, N, K, fuse_gelu, dev_status, stream);
}

// ------------------------------------------------------------------ peer buffers (multi-GPU set-up)
extern "C" int q8k_ipc_export(const void* ptr, unsigned char handle[Q8K_IPC_HANDLE_BYTES], int64_t* offset) {
    static_assert(sizeof(cudaIpcMemHandle_t) == Q8K_IPC_HANDLE_BYTES, "IPC handle size");
    Q8K_REQUIRE(ptr && handle && offset, Q8K_ERR_INVALID_ARG, "ipc_export: null pointer");
    // the handle names a whole allocation: find its base
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range = []() -> RangeFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<RangeFn>(p);
    }();
    Q8K_REQUIRE(range != nullptr, Q8K_ERR_CUDA, "ipc_export: cuMemGetAddressRange is not available");
    CUdeviceptr base = 0;
    size_t size = 0;
    const CUresult r = range(&base, &size, (CUdeviceptr)(uintptr_t)ptr);
    Q8K_REQUIRE(r == CUDA_SUCCESS, Q8K_ERR_CUDA, "ipc_export: cuMemGetAddressRange failed with CUresult %d", (int)r);
    cudaIpcMemHandle_t h;
    Q8K_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base)));
    memcpy(handle, &h, sizeof(h));
    *offset = (int64_t)((uintptr_t)ptr - (uintptr_t)base);
    return Q8K_OK;
}

extern "C" int q8k_ipc_open(const unsigned char handle[Q8K_IPC_HANDLE_BYTES], int64_t offset, void** ptr) {
    Q8K_REQUIRE(handle && ptr && offset >= 0, Q8K_ERR_INVALID_ARG, "ipc_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    Q8K_CUDA_OK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = reinterpret_cast<unsigned char*>(base) + offset;
    return Q8K_OK;
}

extern "C" int q8k_ipc_close(void* ptr, int64_t offset) {
    Q8K_REQUIRE(ptr && offset >= 0, Q8K_ERR_INVALID_ARG, "ipc_close: bad argument");
    Q8K_CUDA_OK(cudaIpcCloseMemHandle(reinterpret_cast<unsigned char*>(ptr) - offset));
    return Q8K_OK;
}
