// Decode GEMV for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a serving loop that has
// handed all device memory to its own arena, code running under a framework allocator that
// forbids side allocations, a plugin whose contract is "bring no memory of your own".  The
// row-major-weight GEMV needs split-K scratch, which the regular entry point takes from the
// caller as `workspace`.  This entry point takes the scratch from a fixed array that is part
// of the loaded library image instead, so the caller passes inputs and outputs only.
//
// The array is a file-scope `static __device__` object: in host code its name is only a
// stand-in for the symbol, never a device address, so the address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and that pointer is what the
// kernels receive.

#include <cuda_runtime.h>

#include <mutex>

#include "../../include/baracuda_kernels_q.h"
#include "launch.h"

namespace {

// Every GPU that loads the library holds this much device memory until the process exits.
static __device__ __align__(256) unsigned char g_gemv_static_scratch[BARACUDA_Q_GEMV_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device; looked up on the first call per device.
int32_t scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return bq::BQ_STATUS_LAUNCH_FAILURE;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_gemv_static_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return bq::BQ_STATUS_LAUNCH_FAILURE;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return bq::BQ_STATUS_OK;
}

}  // namespace

extern "C" {

size_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity(void) {
    return BARACUDA_Q_GEMV_STATIC_SCRATCH_BYTES;
}

int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha, float beta, const void* a,
    int64_t lda, int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, const void* scale_a,
    int64_t stride_scale_a, const void* scale_b, int64_t stride_scale_b, void* d, int64_t ldd, int64_t stride_d,
    void* stream) {
    // the regular entry point's checks first, in its order, so that an invalid problem reports the same status here
    const int32_t st = baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(m, n, k, batch, layout, lda, ldb, ldd, stride_a,
                                                                             stride_b, stride_d);
    if (st != bq::BQ_STATUS_OK) return st;
    if (m == 0 || n == 0 || batch == 0) return bq::BQ_STATUS_OK;
    if (!a || !b || !d || !scale_a || !scale_b) return bq::BQ_STATUS_INVALID_PROBLEM;
    // only then: the scratch this shape needs must fit the fixed array
    const size_t need = baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(m, n, k, batch, layout);
    if (need > BARACUDA_Q_GEMV_STATIC_SCRATCH_BYTES) return bq::BQ_STATUS_WORKSPACE;
    void* scratch = nullptr;
    if (need > 0) {
        const int32_t ss = scratch_for_current_device(&scratch);
        if (ss != bq::BQ_STATUS_OK) return ss;
    }
    // same kernels as the regular entry point; only the scratch differs
    return baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(m, n, k, batch, layout, alpha, beta, a, lda, stride_a, b, ldb,
                                                       stride_b, scale_a, stride_scale_a, scale_b, stride_scale_b, d, ldd,
                                                       stride_d, scratch, need, stream);
}

}  // extern "C"
