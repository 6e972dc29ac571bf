// Per-token (per-row) symmetric activation quantizer feeding the 8-bit GEMM / GEMV:
//   scale[r] = absmax(x[r,:]) / qmax      (1.0 for an all-zero row)
//   q[r,c]   = clamp(round_half_even(x[r,c] * (1 / scale[r])), qmin, qmax)      (s8)
//   q[r,c]   = e4m3_satfinite(x[r,c] * (1 / scale[r])),  qmax = 448             (e4m3)
// the multiply-by-reciprocal recipe of the reference's
//   dynamic_range_quantize_per_token_symmetric_kernel
//   (crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:144-201, 309-326).
// HBM-bound: one CTA per row, the row is read once (kept in registers up to 8192 columns),
// 16-byte loads, packed stores, warp-shuffle + shared-memory max reduction.  Scales are always f32,
// which is what the GEMM epilogues consume.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/baracuda_kernels_q.h"
#include "launch.h"

namespace {

constexpr int QR_THREADS = 256;
constexpr int QR_CACHE = 8;  // 4-element vectors cached per thread: 256 * 8 * 4 = 8192 columns

template <typename TIn>
__device__ __forceinline__ float4 load4(const TIn* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
    return __ldg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
template <typename TIn>
__device__ __forceinline__ float load1(const TIn* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <bool FP8>
__device__ __forceinline__ uint8_t quant1(float v, float inv, int qmin, int qmax) {
    const float t = __fmul_rn(v, inv);
    if constexpr (FP8) {
        return static_cast<uint8_t>(__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3));
    } else {
        int q = __float2int_rn(t);
        q = q < qmin ? qmin : (q > qmax ? qmax : q);
        return static_cast<uint8_t>(static_cast<int8_t>(q));
    }
}

template <typename TIn, bool FP8>
__global__ void __launch_bounds__(QR_THREADS)
quantize_rows_kernel(const TIn* __restrict__ x, int64_t ldx, float* __restrict__ scale, uint8_t* __restrict__ q,
                     int64_t ldq, int cols, int qmin, int qmax, int vec_ok) {
    const int row = blockIdx.x;
    const TIn* xr = x + static_cast<int64_t>(row) * ldx;
    uint8_t* qr = q + static_cast<int64_t>(row) * ldq;
    const int tid = threadIdx.x;
    __shared__ float s_red[QR_THREADS / 32];
    __shared__ float s_inv;

    float4 cache[QR_CACHE];
    float amax = 0.0f;
    const int nvec = vec_ok ? (cols >> 2) : 0;
    // pass 1: absolute maximum; the first QR_CACHE vectors of each thread stay in registers
#pragma unroll
    for (int i = 0; i < QR_CACHE; ++i) {
        const int v = tid + i * QR_THREADS;
        if (v < nvec) {
            cache[i] = load4<TIn>(xr + 4 * v);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(cache[i].x), fabsf(cache[i].y)), fmaxf(fabsf(cache[i].z), fabsf(cache[i].w))));
        }
    }
    for (int v = tid + QR_CACHE * QR_THREADS; v < nvec; v += QR_THREADS) {
        const float4 t = load4<TIn>(xr + 4 * v);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
    }
    for (int c = 4 * nvec + tid; c < cols; c += QR_THREADS) amax = fmaxf(amax, fabsf(load1<TIn>(xr + c)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
        float m = s_red[0];
#pragma unroll
        for (int w = 1; w < QR_THREADS / 32; ++w) m = fmaxf(m, s_red[w]);
        const float s = (m > 0.0f) ? __fdiv_rn(m, static_cast<float>(qmax)) : 1.0f;
        scale[row] = s;
        s_inv = __fdiv_rn(1.0f, s);
    }
    __syncthreads();
    const float inv = s_inv;
    // pass 2: quantize (cached vectors first, the rest is re-read — it is L2 resident by now)
#pragma unroll
    for (int i = 0; i < QR_CACHE; ++i) {
        const int v = tid + i * QR_THREADS;
        if (v < nvec) {
            uchar4 o;
            o.x = quant1<FP8>(cache[i].x, inv, qmin, qmax);
            o.y = quant1<FP8>(cache[i].y, inv, qmin, qmax);
            o.z = quant1<FP8>(cache[i].z, inv, qmin, qmax);
            o.w = quant1<FP8>(cache[i].w, inv, qmin, qmax);
            *reinterpret_cast<uchar4*>(qr + 4 * v) = o;
        }
    }
    for (int v = tid + QR_CACHE * QR_THREADS; v < nvec; v += QR_THREADS) {
        const float4 t = load4<TIn>(xr + 4 * v);
        uchar4 o;
        o.x = quant1<FP8>(t.x, inv, qmin, qmax);
        o.y = quant1<FP8>(t.y, inv, qmin, qmax);
        o.z = quant1<FP8>(t.z, inv, qmin, qmax);
        o.w = quant1<FP8>(t.w, inv, qmin, qmax);
        *reinterpret_cast<uchar4*>(qr + 4 * v) = o;
    }
    for (int c = 4 * nvec + tid; c < cols; c += QR_THREADS) qr[c] = quant1<FP8>(load1<TIn>(xr + c), inv, qmin, qmax);
}

template <typename TIn, bool FP8>
int32_t quantize_rows_run(int32_t rows, int32_t cols, int32_t qmin, int32_t qmax, const void* input, int64_t ldx,
                          void* scale, void* output, int64_t ldq, void* stream) {
    if (rows < 0 || cols < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (!FP8 && (qmin > qmax || qmax <= 0)) return bq::BQ_STATUS_INVALID_PROBLEM;
    const int64_t min_ld = cols > 0 ? cols : 1;
    if (ldx < min_ld || ldq < min_ld) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (rows == 0) return bq::BQ_STATUS_OK;
    if (!scale || (cols > 0 && (!input || !output))) return bq::BQ_STATUS_INVALID_PROBLEM;
    const uintptr_t in_align = sizeof(TIn) * 4;  // one 4-element vector
    const int vec_ok = (reinterpret_cast<uintptr_t>(input) % in_align == 0) && ((ldx * sizeof(TIn)) % in_align == 0) &&
                       (reinterpret_cast<uintptr_t>(output) % 4 == 0) && (ldq % 4 == 0);
    quantize_rows_kernel<TIn, FP8><<<rows, QR_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const TIn*>(input), ldx, static_cast<float*>(scale), static_cast<uint8_t*>(output), ldq, cols,
        FP8 ? -448 : qmin, FP8 ? 448 : qmax, vec_ok);
    return cudaPeekAtLastError() == cudaSuccess ? bq::BQ_STATUS_OK : bq::BQ_STATUS_LAUNCH_FAILURE;
}

}  // namespace

extern "C" {

int32_t baracuda_kernels_quantize_per_token_sym_f32_s8_sm100a_run(int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
                                                                  const void* input, int64_t ld_in, void* scale, void* output,
                                                                  int64_t ld_out, void* workspace, size_t workspace_bytes,
                                                                  void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return quantize_rows_run<float, false>(rows, cols, qmin, qmax, input, ld_in, scale, output, ld_out, stream);
}
int32_t baracuda_kernels_quantize_per_token_sym_bf16_s8_sm100a_run(int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
                                                                   const void* input, int64_t ld_in, void* scale,
                                                                   void* output, int64_t ld_out, void* workspace,
                                                                   size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return quantize_rows_run<__nv_bfloat16, false>(rows, cols, qmin, qmax, input, ld_in, scale, output, ld_out, stream);
}
int32_t baracuda_kernels_quantize_per_token_sym_f32_e4m3_sm100a_run(int32_t rows, int32_t cols, const void* input,
                                                                    int64_t ld_in, void* scale, void* output, int64_t ld_out,
                                                                    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return quantize_rows_run<float, true>(rows, cols, 0, 0, input, ld_in, scale, output, ld_out, stream);
}
int32_t baracuda_kernels_quantize_per_token_sym_bf16_e4m3_sm100a_run(int32_t rows, int32_t cols, const void* input,
                                                                     int64_t ld_in, void* scale, void* output, int64_t ld_out,
                                                                     void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return quantize_rows_run<__nv_bfloat16, true>(rows, cols, 0, 0, input, ld_in, scale, output, ld_out, stream);
}

}  // extern "C"
