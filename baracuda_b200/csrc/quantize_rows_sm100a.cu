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

// The fast path: every thread keeps up to QV_MAX 16-byte vectors of its row in registers as raw bits, so a row is read
// exactly once and about 256 bytes per thread are in flight while the first arrive (a 37 us launch at 8192 x 4096 bf16
// moved 2.7 TB/s with the 8-byte loads and one-row-per-256-threads shape of the general kernel below).  TPR threads share
// a row: TPR == 32 is one warp per row, eight rows per CTA and no block-wide synchronisation; larger TPR is one CTA per
// row.  Needs 16-byte aligned rows, a column count that is a whole number of vectors, and an output aligned to the
// packed store (8 bytes for bf16 input, 4 for f32).  Same arithmetic as the general kernel, bit for bit.
constexpr int QV_MAX = 16;

// Four codes packed into a word.  CLAMP = false (s8 with qmin <= -qmax, the symmetric ranges): |x * inv| cannot round
// beyond qmax <= 127, so no clamp is needed and the rounding is done by adding 1.5 * 2^23 -- the sum is x * inv rounded to
// the nearest integer, ties to even, exactly what cvt.rni gives, and its low byte is the code in two's complement; three
// byte permutes gather the four codes.  (NaN * inv stays NaN, whose low byte is 0, the value the conversion gives too.)
template <bool FP8, bool CLAMP>
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float inv, int qmin, int qmax) {
    if constexpr (FP8) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a, inv), __fmul_rn(b, inv)), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(c, inv), __fmul_rn(d, inv)), __NV_SATFINITE, __NV_E4M3);
        return lo | (hi << 16);
    } else if constexpr (CLAMP) {
        int q0 = __float2int_rn(__fmul_rn(a, inv)), q1 = __float2int_rn(__fmul_rn(b, inv));
        int q2 = __float2int_rn(__fmul_rn(c, inv)), q3 = __float2int_rn(__fmul_rn(d, inv));
        q0 = min(max(q0, qmin), qmax);
        q1 = min(max(q1, qmin), qmax);
        q2 = min(max(q2, qmin), qmax);
        q3 = min(max(q3, qmin), qmax);
        return (static_cast<uint32_t>(q0) & 0xffu) | ((static_cast<uint32_t>(q1) & 0xffu) << 8) |
               ((static_cast<uint32_t>(q2) & 0xffu) << 16) | (static_cast<uint32_t>(q3) << 24);
    } else {
        constexpr float MAGIC = 12582912.0f;  // 1.5 * 2^23
        const uint32_t y0 = __float_as_uint(__fadd_rn(__fmul_rn(a, inv), MAGIC));
        const uint32_t y1 = __float_as_uint(__fadd_rn(__fmul_rn(b, inv), MAGIC));
        const uint32_t y2 = __float_as_uint(__fadd_rn(__fmul_rn(c, inv), MAGIC));
        const uint32_t y3 = __float_as_uint(__fadd_rn(__fmul_rn(d, inv), MAGIC));
        return __byte_perm(__byte_perm(y0, y1, 0x0040), __byte_perm(y2, y3, 0x0040), 0x5410);
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <typename TIn, bool FP8, int TPR, bool CLAMP>
__global__ void __launch_bounds__(TPR == 32 ? 256 : TPR)
quantize_rows_vec_kernel(const TIn* __restrict__ x, int64_t ldx, float* __restrict__ scale, uint8_t* __restrict__ q,
                         int64_t ldq, int rows, int cols, int qmin, int qmax) {
    constexpr bool BF16 = sizeof(TIn) == 2;
    constexpr int EPV = 16 / static_cast<int>(sizeof(TIn));  // elements per 16-byte vector
    const int lane = threadIdx.x & 31;
    const int row = TPR == 32 ? blockIdx.x * 8 + (threadIdx.x >> 5) : blockIdx.x;
    const int t = TPR == 32 ? lane : threadIdx.x;
    if (row >= rows) return;  // whole warps only (TPR == 32), which never meet at a block barrier
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * ldx);
    uint8_t* qr = q + static_cast<int64_t>(row) * ldq;
    const int nvec = cols / EPV;

    uint4 raw[QV_MAX];
#pragma unroll
    for (int i = 0; i < QV_MAX; ++i) {
        const int v = t + i * TPR;
        raw[i] = v < nvec ? __ldg(xr + v) : make_uint4(0u, 0u, 0u, 0u);
    }
    // absolute maximum: bf16 values compare like their bit patterns once the sign is cleared
    float amax;
    if constexpr (BF16) {
        // packed |x| and max on bf16 pairs (exact; a NaN operand is skipped, as fmaxf skips it in the general kernel)
        __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int i = 0; i < QV_MAX; ++i) {
            const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[e])));
        }
        amax = fmaxf(__low2float(m2), __high2float(m2));
    } else {
        amax = 0.0f;
#pragma unroll
        for (int i = 0; i < QV_MAX; ++i) {
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(__uint_as_float(raw[i].x)), fabsf(__uint_as_float(raw[i].y))),
                                     fmaxf(fabsf(__uint_as_float(raw[i].z)), fabsf(__uint_as_float(raw[i].w)))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if constexpr (TPR > 32) {
        __shared__ float s_red[TPR / 32];
        if (lane == 0) s_red[threadIdx.x >> 5] = amax;
        __syncthreads();
        amax = s_red[0];
#pragma unroll
        for (int w = 1; w < TPR / 32; ++w) amax = fmaxf(amax, s_red[w]);
    }
    const float s = (amax > 0.0f) ? __fdiv_rn(amax, static_cast<float>(qmax)) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    if (t == 0) scale[row] = s;
#pragma unroll
    for (int i = 0; i < QV_MAX; ++i) {
        const int v = t + i * TPR;
        if (v < nvec) {
            if constexpr (BF16) {
                uint2 o;
                o.x = quant4<FP8, CLAMP>(bf16_lo(raw[i].x), bf16_hi(raw[i].x), bf16_lo(raw[i].y), bf16_hi(raw[i].y), inv, qmin, qmax);
                o.y = quant4<FP8, CLAMP>(bf16_lo(raw[i].z), bf16_hi(raw[i].z), bf16_lo(raw[i].w), bf16_hi(raw[i].w), inv, qmin, qmax);
                *reinterpret_cast<uint2*>(qr + 8 * v) = o;
            } else {
                *reinterpret_cast<uint32_t*>(qr + 4 * v) =
                    quant4<FP8, CLAMP>(__uint_as_float(raw[i].x), __uint_as_float(raw[i].y), __uint_as_float(raw[i].z),
                                __uint_as_float(raw[i].w), inv, qmin, qmax);
            }
        }
    }
}

template <typename TIn, bool FP8, int TPR>
void launch_vec(const TIn* x, int64_t ldx, float* scale, uint8_t* q, int64_t ldq, int rows, int cols, int qmin, int qmax,
                cudaStream_t stream) {
    const int grid = TPR == 32 ? (rows + 7) / 8 : rows;
    const int threads = TPR == 32 ? 256 : TPR;
    if (!FP8 && !(qmin <= -qmax && qmax <= 127)) {  // a range the scaled values can leave: keep the clamp
        quantize_rows_vec_kernel<TIn, FP8, TPR, true><<<grid, threads, 0, stream>>>(x, ldx, scale, q, ldq, rows, cols, qmin, qmax);
    } else {
        quantize_rows_vec_kernel<TIn, FP8, TPR, false><<<grid, threads, 0, stream>>>(x, ldx, scale, q, ldq, rows, cols, qmin, qmax);
    }
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
    // the register-resident path when rows are 16-byte aligned, a whole number of vectors long and short enough
    constexpr int EPV = 16 / static_cast<int>(sizeof(TIn));
    const uintptr_t out_align = sizeof(TIn) == 2 ? 8 : 4;
    const bool fast = cols > 0 && cols % EPV == 0 && reinterpret_cast<uintptr_t>(input) % 16 == 0 &&
                      (ldx * sizeof(TIn)) % 16 == 0 && reinterpret_cast<uintptr_t>(output) % out_align == 0 &&
                      ldq % static_cast<int64_t>(out_align) == 0 && cols / EPV <= QV_MAX * 1024;
    if (fast) {
        const TIn* xin = static_cast<const TIn*>(input);
        float* sc = static_cast<float*>(scale);
        uint8_t* out = static_cast<uint8_t*>(output);
        const int lo = FP8 ? -448 : qmin, hi = FP8 ? 448 : qmax;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const int need = (cols / EPV + QV_MAX - 1) / QV_MAX;  // threads a row needs
        if (need <= 32) launch_vec<TIn, FP8, 32>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        else if (need <= 64) launch_vec<TIn, FP8, 64>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        else if (need <= 128) launch_vec<TIn, FP8, 128>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        else if (need <= 256) launch_vec<TIn, FP8, 256>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        else if (need <= 512) launch_vec<TIn, FP8, 512>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        else launch_vec<TIn, FP8, 1024>(xin, ldx, sc, out, ldq, rows, cols, lo, hi, st);
        return cudaPeekAtLastError() == cudaSuccess ? bq::BQ_STATUS_OK : bq::BQ_STATUS_LAUNCH_FAILURE;
    }
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
