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

// The aligned case (16-byte aligned rows on both sides, N a multiple of 8): a CTA walks whole rows, its threads the
// 8-column groups of the row, four groups per thread at a time with all eight 16-byte loads requested before the first is
// used -- 128 bytes per thread in flight instead of 32, no 64-bit division per group, the row scale read once per row.
// (The general kernel below moved 0.60-0.64 of the copy bandwidth on 8192 x 8192; the pass is 4 bytes in, 2 out.)
template <bool INT_ACC>
__global__ void __launch_bounds__(256)
dequant_rows_fast_kernel(const uint32_t* __restrict__ acc, int64_t ld_acc, const float* __restrict__ sa,
                         const float* __restrict__ sb, int scale_mode, float alpha, const float* __restrict__ bias,
                         __nv_bfloat16* __restrict__ d, int64_t ldd, int m, int n) {
    constexpr int U = 4;
    const int groups = n >> 3;
    for (int row = blockIdx.x; row < m; row += gridDim.x) {
        const float sa_row = scale_mode == 1 ? __ldg(sa + row) : __ldg(sa);
        const uint4* src = reinterpret_cast<const uint4*>(acc + static_cast<int64_t>(row) * ld_acc);
        uint4* dst = reinterpret_cast<uint4*>(d + static_cast<int64_t>(row) * ldd);
        for (int g0 = threadIdx.x; g0 < groups; g0 += U * 256) {
            uint4 lo[U], hi[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = g0 + u * 256;
                if (g < groups) {
                    lo[u] = __ldcs(src + 2 * g);
                    hi[u] = __ldcs(src + 2 * g + 1);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = g0 + u * 256;
                if (g >= groups) break;
                const uint32_t r[8] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w};
                float sbv[8], bv[8];
                if (scale_mode == 1) {
                    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sb + 8 * g));
                    const float4 s1 = __ldg(reinterpret_cast<const float4*>(sb + 8 * g) + 1);
                    sbv[0] = s0.x; sbv[1] = s0.y; sbv[2] = s0.z; sbv[3] = s0.w;
                    sbv[4] = s1.x; sbv[5] = s1.y; sbv[6] = s1.z; sbv[7] = s1.w;
                } else {
                    const float s = __ldg(sb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) sbv[j] = s;
                }
                if (bias) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + 8 * g));
                    const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + 8 * g) + 1);
                    bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                    bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
                }
                float y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // (sa*sb) first, then the accumulator, then alpha: the product order of the fused epilogue
                    const float s = __fmul_rn(sa_row, sbv[j]);
                    y[j] = __fmul_rn(__fmul_rn(s, acc_to_float<INT_ACC>(r[j])), alpha);
                    if (bias) y[j] = __fadd_rn(y[j], bv[j]);
                }
                uint4 out;
                __nv_bfloat162 h;
                h = __floats2bfloat162_rn(y[0], y[1]); out.x = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(y[2], y[3]); out.y = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(y[4], y[5]); out.z = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(y[6], y[7]); out.w = *reinterpret_cast<uint32_t*>(&h);
                dst[g] = out;
            }
        }
    }
}

// The owner of a row block in the fused K-sharded forward: adds the `world` partial-sum slots that the ranks' GEMM
// epilogues stored into its staging buffer, applies the scales like dequant_rows_kernel, and stores the bf16 rows into
// every rank's output through peer pointers (plain stores over NVLink, peers visited from rank + 1 on so that no
// buffer is every rank's target at once).  Eight columns per thread.
struct PeerOut {
    __nv_bfloat16* y[8];
};

template <bool INT_ACC>
__global__ void __launch_bounds__(256)
reduce_dequant_broadcast_kernel(const uint32_t* __restrict__ staging, int world, int rank, int rows, int n,
                                const float* __restrict__ sa, const float* __restrict__ sb, int scale_mode, float alpha,
                                const float* __restrict__ bias, PeerOut out, int64_t ldy, int vec) {
    const int groups = (n + 7) / 8;
    const int64_t total = static_cast<int64_t>(rows) * groups;
    const int64_t slot_stride = static_cast<int64_t>(rows) * n;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(idx / groups);
        const int col0 = static_cast<int>(idx - static_cast<int64_t>(r) * groups) * 8;
        const int row = rank * rows + r;  // row of the whole [M, N] result
        const bool full = col0 + 8 <= n;
        float facc[8];
        int iacc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            facc[j] = 0.0f;
            iacc[j] = 0;
        }
        for (int s = 0; s < world; ++s) {  // slot order: the f32 sum does not depend on arrival order
            const uint32_t* src = staging + s * slot_stride + static_cast<int64_t>(r) * n + col0;
            uint32_t v[8];
            if (vec && full) {
                const uint4 lo = __ldcs(reinterpret_cast<const uint4*>(src));
                const uint4 hi = __ldcs(reinterpret_cast<const uint4*>(src) + 1);
                v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
                v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = col0 + j < n ? src[j] : 0u;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if constexpr (INT_ACC) {
                    iacc[j] += static_cast<int32_t>(v[j]);
                } else {
                    facc[j] = __fadd_rn(facc[j], __uint_as_float(v[j]));
                }
            }
        }
        const float sa_row = scale_mode == 1 ? __ldg(sa + row) : __ldg(sa);
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = col0 + j < n ? col0 + j : n - 1;
            const float sb_col = scale_mode == 1 ? __ldg(sb + col) : __ldg(sb);
            const float s = __fmul_rn(sa_row, sb_col);
            const float a = INT_ACC ? static_cast<float>(iacc[j]) : facc[j];
            y[j] = __fmul_rn(__fmul_rn(s, a), alpha);
            if (bias) y[j] = __fadd_rn(y[j], __ldg(bias + col));
        }
        uint4 packed;
        {
            __nv_bfloat162 h;
            h = __floats2bfloat162_rn(y[0], y[1]); packed.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[2], y[3]); packed.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[4], y[5]); packed.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2bfloat162_rn(y[6], y[7]); packed.w = *reinterpret_cast<uint32_t*>(&h);
        }
        for (int q = 0; q < world; ++q) {
            int dst_rank = rank + 1 + q;
            if (dst_rank >= world) dst_rank -= world;
            __nv_bfloat16* dst = out.y[dst_rank] + static_cast<int64_t>(row) * ldy + col0;
            if (vec && full) {
                *reinterpret_cast<uint4*>(dst) = packed;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (col0 + j < n) dst[j] = __float2bfloat16_rn(y[j]);
                }
            }
        }
    }
}

// Builds the interleaved gate/up operand of the gated-MLP GEMM: output row 64b + i is gate row 32b + i for i < 32 and
// up row 32b + (i - 32) otherwise.  Rows are `row_bytes` bytes (a weight row of K bytes, or 4 for a scale / bias entry).
__global__ void __launch_bounds__(256)
    interleave_gate_up_kernel(const uint8_t* __restrict__ gate, int64_t gate_pitch, const uint8_t* __restrict__ up,
                              int64_t up_pitch, uint8_t* __restrict__ out, int64_t out_pitch, int64_t f_rows,
                              int64_t row_bytes, int vec) {
    const int64_t per_row = vec ? row_bytes / 16 : row_bytes;
    const int64_t total = 2 * f_rows * per_row;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / per_row;
        const int64_t x = i - r * per_row;
        const int64_t blk = r >> 6;
        const int64_t in = r & 63;
        const uint8_t* src = in < 32 ? gate + (blk * 32 + in) * gate_pitch : up + (blk * 32 + in - 32) * up_pitch;
        if (vec) {
            reinterpret_cast<uint4*>(out + r * out_pitch)[x] = __ldg(reinterpret_cast<const uint4*>(src) + x);
        } else {
            out[r * out_pitch + x] = __ldg(src + x);
        }
    }
}

}  // namespace

int32_t launch_reduce_dequant_broadcast(int32_t kind, int32_t rank, int32_t world, int32_t rows, int32_t n,
                                        const void* staging_local, const float* scale_a, const float* scale_b,
                                        int32_t scale_mode, float alpha, const float* bias, void* const* y, int64_t ldy,
                                        cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return BQ_STATUS_OK;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !y || !staging_local) return BQ_STATUS_INVALID_PROBLEM;
    const int sms = sm_count_of_current_device();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    PeerOut out;
    int vec = ((reinterpret_cast<uintptr_t>(staging_local) & 15u) == 0 && (n % 4) == 0 && ((ldy * 2) & 15) == 0) ? 1 : 0;
    for (int q = 0; q < 8; ++q) {
        out.y[q] = q < world ? static_cast<__nv_bfloat16*>(y[q]) : nullptr;
        if (q < world && (!y[q] || (reinterpret_cast<uintptr_t>(y[q]) & 15u) != 0)) {
            if (!y[q]) return BQ_STATUS_INVALID_PROBLEM;
            vec = 0;
        }
    }
    const int64_t total = static_cast<int64_t>(rows) * ((n + 7) / 8);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    if (blocks > cap) blocks = cap;
    if (kind == BQ_KIND_S8) {
        reduce_dequant_broadcast_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<const uint32_t*>(staging_local), world, rank, rows, n, scale_a, scale_b, scale_mode, alpha, bias, out,
            ldy, vec);
    } else {
        reduce_dequant_broadcast_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<const uint32_t*>(staging_local), world, rank, rows, n, scale_a, scale_b, scale_mode, alpha, bias, out,
            ldy, vec);
    }
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

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
    // whole aligned rows of 8-column groups (and 16-byte aligned scale / bias vectors): the row-walking kernel
    const bool fast = vec && (n % 8) == 0 && (scale_mode != 1 || (reinterpret_cast<uintptr_t>(scale_b) & 15u) == 0) &&
                      (!bias || (reinterpret_cast<uintptr_t>(bias) & 15u) == 0);
    if (fast) {
        const unsigned grid = static_cast<unsigned>(m < sms * 8 ? m : sms * 8);
        if (kind == BQ_KIND_S8) {
            dequant_rows_fast_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(acc), ld_acc, scale_a, scale_b,
                                                                      scale_mode, alpha, bias, static_cast<__nv_bfloat16*>(d),
                                                                      ldd, m, n);
        } else {
            dequant_rows_fast_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(acc), ld_acc, scale_a, scale_b,
                                                                       scale_mode, alpha, bias, static_cast<__nv_bfloat16*>(d),
                                                                       ldd, m, n);
        }
        return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
    }
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

int32_t launch_interleave_gate_up(int64_t f_rows, int64_t row_bytes, const void* gate, int64_t gate_pitch, const void* up,
                                  int64_t up_pitch, void* out, int64_t out_pitch, cudaStream_t stream) {
    if (f_rows <= 0 || row_bytes <= 0) return BQ_STATUS_OK;
    const int sms = sm_count_of_current_device();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    const auto a16 = [](const void* p, int64_t pitch) {
        return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (pitch & 15) == 0;
    };
    const int vec = (row_bytes % 16 == 0 && a16(gate, gate_pitch) && a16(up, up_pitch) && a16(out, out_pitch)) ? 1 : 0;
    const int64_t total = 2 * f_rows * (vec ? row_bytes / 16 : row_bytes);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    if (blocks > cap) blocks = cap;
    interleave_gate_up_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint8_t*>(gate), gate_pitch, static_cast<const uint8_t*>(up), up_pitch,
        static_cast<uint8_t*>(out), out_pitch, f_rows, row_bytes, vec);
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

}  // namespace bq
