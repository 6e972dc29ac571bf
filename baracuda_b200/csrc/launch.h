// Internal launch descriptors shared by the kernels and the C-ABI file.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace bq {

// Status codes of the flat C symbols; values follow the reference's contract
// (crates/baracuda-kernels-sys/src/lib.rs:19-27).
enum : int32_t {
    BQ_STATUS_OK = 0,
    BQ_STATUS_MISALIGNED = 1,
    BQ_STATUS_INVALID_PROBLEM = 2,
    BQ_STATUS_UNSUPPORTED = 3,
    BQ_STATUS_WORKSPACE = 4,
    BQ_STATUS_LAUNCH_FAILURE = 5
};

enum : int32_t { BQ_KIND_S8 = 0, BQ_KIND_E4M3 = 1 };
enum : int32_t { BQ_LAYOUT_RRR = 0, BQ_LAYOUT_RCR = 1 };

struct GemmDesc {
    int32_t kind;     // BQ_KIND_*
    int32_t raw_out;  // 1: write the 32-bit accumulators, 0: fused dequant -> bf16
    int32_t m, n, k;
    const void* a;
    int64_t lda;
    const void* b;
    int64_t ldb;
    const float* scale_a;
    const float* scale_b;
    int32_t scale_mode;  // 0 per-tensor scalars, 1 per-row / per-column vectors
    float alpha;
    void* d;
    int64_t ldd;
    int32_t force_block_n;  // 0 = choose; else 64 / 128 / 256 (tuning and tests)
};

int32_t launch_gemm_q8(const GemmDesc& g, cudaStream_t stream);
int32_t read_and_clear_gemm_device_status();

struct GemvDesc {
    int32_t raw_out;  // 1: int32 accumulators, 0: bf16
    int32_t m, n, k, batch;
    int32_t layout;  // BQ_LAYOUT_*
    float alpha, beta;
    const int8_t* a;
    int64_t lda, stride_a;
    const int8_t* b;
    int64_t ldb, stride_b;
    const float* scale_a;
    int64_t stride_scale_a;
    const float* scale_b;
    int64_t stride_scale_b;
    void* d;
    int64_t ldd, stride_d;
    void* workspace;
    size_t workspace_bytes;
    int32_t variant;  // 0 = choose (tuning and tests)
};

int32_t launch_gemv_q8(const GemvDesc& g, cudaStream_t stream);
size_t gemv_q8_workspace_bytes(int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout);

}  // namespace bq
