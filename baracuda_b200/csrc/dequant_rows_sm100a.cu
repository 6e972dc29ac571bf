// Dequantise a matrix of raw accumulators: D[i][j] = bf16( (sa[i] * sb[j]) * acc[i][j] * alpha (+ bias[j]) ).
//
// The second half of the K-sharded ("row-parallel") linear layer: every rank's GEMM leaves its int32 / f32
// partial sums, the ranks add them (all-reduce), and this pass applies the scales exactly as the fused GEMM
// epilogue would have -- same product order, one rounding per product, no fused multiply-add -- so a sharded
// W8A8 layer returns the very bits of the unsharded one.  HBM-bound: 4 bytes in, 2 bytes out per element;
// eight columns per thread, 16-byte loads and stores, grid-stride over the rows.
//
// Follows the W8A8 dequant of the reference,
//   crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:271-274,
// and the bias placement of its RowParallelLinearPlan (after the reduction, once),
//   crates/baracuda-megatron/src/lib.rs:1010-1018, 1160-1166.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace bq {

namespace {

template <bool INT_ACC>
__device__ __forceinline__ float acc_to_float(uint32_t bits) {
    if constexpr (INT_ACC) {
        return static_cast<float>(static_cast<int32_t>(bits));
    } else {
        return __uint_as_float(bits);
    }
}

template <bool INT_ACC>
__global__ void __launch_bounds__(256)
dequant_rows_kernel(const uint32_t* __restrict__ acc, int64_t ld_acc, const float* __restrict__ sa,
                    const float* __restrict__ sb, int scale_mode, float alpha, const float* __restrict__ bias,
                    __nv_bfloat16* __restrict__ d, int64_t ldd, int m, int n, int vec) {
    const int groups = (n + 7) / 8;  // 8-column groups per row
    const int64_t total = static_cast<int64_t>(m) * groups;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(idx / groups);
        const int col0 = static_cast<int>(idx - static_cast<int64_t>(row) * groups) * 8;
        const float sa_row = scale_mode == 1 ? __ldg(sa + row) : __ldg(sa);
        const uint32_t* src = acc + static_cast<int64_t>(row) * ld_acc + col0;
        __nv_bfloat16* dst = d + static_cast<int64_t>(row) * ldd + col0;
        uint32_t r[8];
        const bool full = col0 + 8 <= n;
        if (vec && full) {
            const uint4 lo = __ldcs(reinterpret_cast<const uint4*>(src));
            const uint4 hi = __ldcs(reinterpret_cast<const uint4*>(src) + 1);
            r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
            r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = col0 + j < n ? src[j] : 0u;
        }
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = col0 + j < n ? col0 + j : n - 1;
            const float sb_col = scale_mode == 1 ? __ldg(sb + col) : __ldg(sb);
            // (sa*sb) first, then the accumulator, then alpha: the product order of the fused epilogue
            const float s = __fmul_rn(sa_row, sb_col);
            y[j] = __fmul_rn(__fmul_rn(s, acc_to_float<INT_ACC>(r[j])), alpha);
            if (bias) y[j] = __fadd_rn(y[j], __ldg(bias + col));
        }
        if (vec && full) {
            uint4 out;
            __nv_bfloat162 h;
            h = __floats2bfloat162_rn(y[0], y[1]); out.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[2], y[3]); out.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[4], y[5]); out.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[6], y[7]); out.w = *reinterpret_cast<uint32_t*>(&h);
            *reinterpret_cast<uint4*>(dst) = out;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (col0 + j < n) dst[j] = __float2bfloat16_rn(y[j]);
            }
        }
    }
}

}  // namespace

int32_t launch_dequant_rows(int32_t kind, int32_t m, int32_t n, const void* acc, int64_t ld_acc, const float* scale_a,
                            const float* scale_b, int32_t scale_mode, float alpha, const float* bias, void* d, int64_t ldd,
                            cudaStream_t stream) {
    if (m <= 0 || n <= 0) return BQ_STATUS_OK;
    const int sms = sm_count_of_current_device();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    const int64_t total = static_cast<int64_t>(m) * ((n + 7) / 8);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sms) * 16;  // a few waves of 256-thread blocks, grid-stride beyond
    if (blocks > cap) blocks = cap;
    const int vec = ((reinterpret_cast<uintptr_t>(acc) & 15u) == 0 && ((ld_acc * 4) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(d) & 15u) == 0 && ((ldd * 2) & 15) == 0)
                        ? 1
                        : 0;
    if (kind == BQ_KIND_S8) {
        dequant_rows_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<const uint32_t*>(acc), ld_acc, scale_a, scale_b, scale_mode, alpha, bias,
            static_cast<__nv_bfloat16*>(d), ldd, m, n, vec);
    } else {
        dequant_rows_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<const uint32_t*>(acc), ld_acc, scale_a, scale_b, scale_mode, alpha, bias,
            static_cast<__nv_bfloat16*>(d), ldd, m, n, vec);
    }
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

}  // namespace bq
