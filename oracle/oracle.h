/*
 * CPU oracle for the quantized-GEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's CPU checker for a
 * contraction (baracuda-kernelgen `oracle::eval_contraction`) and of the
 * quantizers / dequant formulas the reference's W8A8 and FP8 paths use.
 * Nothing in the shipped library calls into it: it is linked only by the test
 * suite, by the smoke check and by the benchmark's CPU-baseline leg.
 *
 * Parity status: PINNED in-tree.  The contraction, the bf16 codec and the
 * W8A8 formula are checked against the reference's own known-answer tests
 * (crates/baracuda-kernelgen/src/kiss_ref_diff.rs:1170-1345,
 *  crates/baracuda-kernelgen/src/oracle.rs:2393-2472, 2567-2668,
 *  crates/baracuda-kernels/tests/quantized_linear_smoke.rs:82-184,
 *  crates/baracuda-kernels/tests/int8_rrr_smoke.rs:159-172,
 *  crates/baracuda-kernels/tests/fp8_e4m3_rcr_smoke.rs:113-127).
 * The e4m3 codec follows the published OCP FP8 E4M3 format (the reference
 * takes it from the third-party crate float8 0.7.0 on the host and from
 * CUDA's cuda_fp8.h on the device; neither source is vendored in the
 * reference tree) and is cross-checked bit-for-bit against torch's
 * float8_e4m3fn cast in the tests.
 */
#ifndef BARACUDA_ORACLE_H
#define BARACUDA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element kinds the contraction restatement understands
 * (subset of ElementKind, crates/baracuda-kernel-vocab/src/element.rs:1014). */
enum {
    ORC_F32 = 0,
    ORC_F64 = 1,
    ORC_BF16 = 2,
    ORC_I32 = 3,
    ORC_S8 = 4,
    ORC_I64 = 5
};

/* Epilogue over the K-sum ("Reduced(0)") plus the optional [N] bias. */
enum {
    ORC_EPI_IDENTITY = 0,
    ORC_EPI_RELU = 1,
    ORC_EPI_BIAS = 2,
    ORC_EPI_BIAS_RELU = 3
};

/* Operand storage order of the B matrix, as the reference's LayoutSku names it
 * (crates/baracuda-kernel-vocab/src/layout.rs:17-34). */
enum {
    ORC_LAYOUT_RRR = 0, /* B row-major [K,N], element (k,n) at k*ldb + n */
    ORC_LAYOUT_RCR = 1  /* B col-major [K,N] == row-major [N,K], (k,n) at n*ldb + k */
};

int orc_num_threads(void);
/* Worker threads of the following calls (a launcher may have exported OMP_NUM_THREADS=1 for its ranks). */
void orc_set_num_threads(int n);

/* ---- codecs --------------------------------------------------------------*/
/* f32 -> bf16 bits, RNE, NaN quieted (oracle.rs:397-404). */
uint16_t orc_f32_to_bf16_bits(float x);
/* bf16 bits -> f32 (oracle.rs:339-341). */
float orc_bf16_bits_to_f32(uint16_t bits);
/* OCP FP8 E4M3 (finite-only, max 448, 0x7f/0xff NaN). */
float orc_e4m3_to_f32(uint8_t bits);
/* f32 -> e4m3, round-to-nearest-even, saturate-to-finite (the behaviour of
 * __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3),
 * crates/baracuda-kernels-sys/kernels/include/baracuda_dtype.cuh:44-47). */
uint8_t orc_f32_to_e4m3_satfinite(float x);

/* ---- the contraction interpreter -----------------------------------------*/
/*
 * out[b,m,n] = epi( sum_k lhs[b,m,k] * rhs[b,k,n] ), k ascending, f64
 * accumulator, operands read through their physical element strides, result
 * rounded once into `dtype` (oracle.rs:1289-1372, 980-1001, 903-945).
 * Stride triples are {batch, row, col} in ELEMENTS; bdim == 1 is the rank-2
 * case.  `bias` is the per-column [N] vector (same dtype) or NULL.
 * Returns 0, or 2 for an unsupported dtype/epilogue combination.
 */
int orc_contraction(int dtype, int64_t bdim, int64_t m, int64_t n, int64_t k,
                    const void* lhs, const int64_t lhs_strides[3],
                    const void* rhs, const int64_t rhs_strides[3],
                    const void* bias,
                    void* out, const int64_t out_strides[3],
                    int epilogue);

/* ---- fast, provably-equal cells used at the large configs ----------------*/
/*
 * int32 accumulators of an s8 x s8 contraction.  Equal, bit for bit, to
 * orc_contraction(ORC_I32) over the sign-extended operands: every product and
 * partial sum is an integer below 2^31 at the supported sizes
 * (|acc| <= 127*127*K), so the f64 K-sum of the interpreter is exact.
 * Parallel over rows (OpenMP).
 */
int orc_gemm_s8_s32(int32_t m, int32_t n, int32_t k,
                    const int8_t* a, int64_t lda,
                    const int8_t* b, int64_t ldb, int b_layout,
                    int32_t* acc, int64_t ldacc);

/* out = store( (sa[m]*sb[n]) * (float)acc ) — the W8A8 dequant of
 * baracuda_quantize_compose.cuh:271-274, product order preserved. */
void orc_dequant_s32_bf16(int32_t m, int32_t n, const int32_t* acc, int64_t ldacc,
                          const float* sa, const float* sb,
                          uint16_t* out_bf16, int64_t ldo);
void orc_dequant_s32_f32(int32_t m, int32_t n, const int32_t* acc, int64_t ldacc,
                         const float* sa, const float* sb,
                         float* out, int64_t ldo);

/*
 * f32 result of an e4m3 x e4m3 contraction: operands decoded to f32, products
 * and K-sum in f64, one rounding to f32 — i.e. orc_contraction(ORC_F32) over
 * the dequantised values.  Parallel over rows.
 */
int orc_gemm_e4m3_f32(int32_t m, int32_t n, int32_t k,
                      const uint8_t* a, int64_t lda,
                      const uint8_t* b, int64_t ldb, int b_layout,
                      float* acc, int64_t ldacc);

/* out = bf16( (sa*sb) * acc ); sa/sb are per-row/per-column vectors, or
 * scalars broadcast when the matching *_is_vector flag is 0. */
void orc_scale_f32_bf16(int32_t m, int32_t n, const float* acc, int64_t ldacc,
                        const float* sa, int sa_is_vector,
                        const float* sb, int sb_is_vector,
                        uint16_t* out_bf16, int64_t ldo);

/*
 * The reference's tensor-core int GEMM contract with an s8 result
 * (crates/baracuda-kernels/tests/int8_rrr_smoke.rs:76-131,
 *  crates/baracuda-cutlass/tests/int8_smoke.rs:85-124):
 * z = alpha*(float)acc + beta*(float)C + bias[j]; d = sat_s8(rint_even(z)).
 * c and bias may be NULL.
 */
int orc_int_gemm_s8_out(int32_t m, int32_t n, int32_t k,
                        const int8_t* a, int64_t lda,
                        const int8_t* b, int64_t ldb, int b_layout,
                        const int8_t* c, int64_t ldc,
                        const float* bias, float alpha, float beta,
                        int8_t* d, int64_t ldd);

/* ---- quantizers (input preparation for the configs) ----------------------*/
/*
 * Symmetric per-row quantizer: scale = absmax/qmax (1.0 for an all-zero row),
 * q = clamp(rint_even(x * (1/scale)), qmin, qmax)
 * (baracuda_quantize_compose.cuh:115-126, 160-200 — the multiply-by-reciprocal
 * form; the per-output-channel weight quantizer of
 * crates/baracuda-kernels/tests/quantized_linear_smoke.rs:35-61 is the same
 * routine applied to the [C_out,K] weight).
 */
void orc_quantize_rows_s8(int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
                          const float* x, int64_t ldx, float* scale, int8_t* q, int64_t ldq);
/* e4m3 twin: scale = absmax/448 (1.0 if zero), q = e4m3_satfinite(x*(1/scale)). */
void orc_quantize_rows_e4m3(int32_t rows, int32_t cols,
                            const float* x, int64_t ldx, float* scale, uint8_t* q, int64_t ldq);
/* Whole-tensor e4m3 quantizer (one scale), the delayed-scaling convention of
 * crates/baracuda-transformer-engine-sys/csrc/baracuda_te_shim.cu:300-313
 * restated as a dequant scale absmax/448. */
void orc_quantize_tensor_e4m3(int64_t count, const float* x, float* scale, uint8_t* q);

/* ---- comparator (oracle.rs:1978-2060) -------------------------------------*/
/* Returns -1 when equal, else the index of the first differing byte-element. */
int64_t orc_compare_bitexact(const void* expected, const void* actual, size_t elem_size, int64_t count);
/* Tolerant: |e-a| <= abs + rel*max(|e|,|a|); NaN==NaN; unequal infinities
 * rejected.  Returns -1 on success, else the first failing index. */
int64_t orc_compare_tolerant_f32(const float* expected, const float* actual, int64_t count,
                                 double rel, double abs_tol);

#ifdef __cplusplus
}
#endif
#endif /* BARACUDA_ORACLE_H */
