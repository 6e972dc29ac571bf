/*
 * Flat C ABI of the sm_100a quantized-GEMM hot path.
 *
 * These are the symbols a `baracuda-kernels-sys`-style binding declares as
 * `unsafe extern "C"` and the safe Plan layer calls from `run`.  They follow
 * the conventions of the reference's bespoke kernels
 * (crates/baracuda-kernels-sys/src/lib.rs:19-27 for the status codes;
 *  crates/baracuda-kernels-sys/kernels/gemm/gemm_s8_rrr_sm80.cu:28-64 and
 *  crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:235-343 for the
 *  run / can_implement / workspace_size triples):
 *
 *   - every pointer is a DEVICE pointer owned by the caller; nothing here
 *     allocates or frees; scratch is passed in as `workspace` and sized by the
 *     matching *_workspace_size;
 *   - dims are int32, leading dimensions and batch strides are int64 counted
 *     in ELEMENTS; `stream` is a cudaStream_t; launches are asynchronous and
 *     never synchronise the host;
 *   - the return value is a status: 0 ok, 1 misaligned operand, 2 invalid
 *     problem, 3 unsupported, 4 workspace missing or too small, 5 launch
 *     failure.  Empty problems (m == 0 or n == 0) return 0 without launching;
 *   - *_can_implement and *_workspace_size are pure host functions.
 *
 * Layout tags: "rcr" = A row-major [M,K], B column-major [K,N] (that is, the
 * weight stored [N,K] with K contiguous, ldb >= K), D row-major [M,N].
 * For the GEMV the `layout` argument selects 0 = RRR (B row-major [K,N],
 * ldb >= N — the only layout of the reference's gemv_dense_m1) or
 * 1 = RCR (B stored [N,K], ldb >= K).
 */
#ifndef BARACUDA_KERNELS_Q_H
#define BARACUDA_KERNELS_Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BARACUDA_Q_STATUS_OK 0
#define BARACUDA_Q_STATUS_MISALIGNED 1
#define BARACUDA_Q_STATUS_INVALID_PROBLEM 2
#define BARACUDA_Q_STATUS_UNSUPPORTED 3
#define BARACUDA_Q_STATUS_WORKSPACE 4
#define BARACUDA_Q_STATUS_LAUNCH_FAILURE 5

/* codes above 5 are free in the reference's contract (ARCHITECTURE.md:370); the sharded entry points use two */
#define BARACUDA_Q_STATUS_COMM_UNAVAILABLE 6 /* libnccl.so.2 could not be loaded */
#define BARACUDA_Q_STATUS_COMM_FAILURE 7     /* an NCCL call returned an error */

#define BARACUDA_Q_LAYOUT_RRR 0
#define BARACUDA_Q_LAYOUT_RCR 1

#define BARACUDA_Q_SCALE_PER_TENSOR 0 /* scale_a, scale_b each point at ONE float on the device */
#define BARACUDA_Q_SCALE_PER_ROW_COL 1 /* scale_a is float[M], scale_b is float[N] */

/* ---------------------------------------------------------------------------
 * W8A8 GEMM, s8 x s8 -> s32 on tcgen05, fused dequant to bf16:
 *   D[i,j] = bf16( alpha * ((scale_a[i] * scale_b[j]) * (float)acc[i,j]) )
 * The product order is the reference's W8A8 formula
 * (crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:271-274),
 * so with alpha == 1 the result equals it bit for bit.
 * Replaces the two-pass route of the reference: the s8-out tensor-core GEMM
 *   baracuda_cutlass_gemm_s8_rcr_sm80_run
 *   (crates/baracuda-cutlass-kernels-sys/kernels/gemm_s8_rcr_sm80.cu:169-183)
 * followed by a dequant pass, and the one-thread-per-cell
 *   baracuda_kernels_quantized_linear_w8a8_f32_run
 *   (crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:340-370).
 * `c` / `ldc` / `beta` keep the GEMM family's argument order: with beta != 0 the
 * epilogue adds beta * C[m, j] (C bf16 [M, ldc], 2-byte aligned, may be D itself --
 * the residual add of an output / down projection) before the bias and the
 * activation, product and sum rounded separately in f32; beta != 0 without C
 * returns 2; with beta == 0 C is not read.  The raw-accumulator SKUs take no C (3).
 * Alignment: a and b 16-byte aligned, lda and ldb multiples of 16.
 * Accumulator range: every int8 symbol of this header (GEMM, GEMV, sharded forms) returns 3 (unsupported) for
 * K > 131 071, the longest contraction whose sums cannot leave 32 bits (K * 128 * 128 < 2^31; for the K-sharded
 * forms the bound applies to the K of all ranks together).  The reference saturates instead (mma.sync
 * ".satfinite", crates/baracuda-kernels-sys/kernels/include/baracuda_int8_rrr_sm80.cuh:86-92, and the saturating
 * adds of its test oracle, crates/baracuda-kernels/tests/int8_rrr_smoke.rs:76-131); up to that K the two agree
 * bit for bit, beyond it tcgen05's behaviour is unspecified, so the call is refused rather than answered differently.
 * Small batches (the 128 x 128 output tiles cover at most half of the SMs, K >= 2048): the bf16-out and 8-bit-out GEMMs
 * (either weight layout) run as 2 or 4 K slices per tile on otherwise idle SMs -- a thread-block cluster per tile whose CTAs
 * add their partial sums through distributed shared memory before the same epilogue (and, for M > 256 against few
 * columns and K >= 7680, as two slices per 128 x 256 tile).  Nothing changes for the caller:
 * no scratch, one launch; the int8 result keeps its bits, the e4m3 result adds the slices' f32 sums in slice order
 * (inside the tolerance of the SKU).
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    const void* scale_a, const void* scale_b,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);

/* SmoothQuant inference forward, SmoothQuantLinearPlan of the reference
 * (crates/baracuda-kernels/src/quantize/smoothquant.rs:1-60, 70-140): pre-quantized s8 activation [M, K], s8 weight
 * [N, K], ONE per-tensor activation scale and per-output-channel weight scales:
 *     output[m, n] = bf16( (act_scale * weight_scale[n]) * (float)sum_k act_q[m,k] * weight_q[n,k] )
 * The reference broadcasts act_scale into a caller-owned [M] scratch with a fill launch and reuses its W8A8 kernel;
 * here the scalar travels by value in the kernel parameters, so there is no scratch and no second launch.  Same
 * product order as the reference's W8A8 formula, hence the same bits as the per-token symbol given a constant
 * scale_a vector.  Alignment and statuses as baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run. */
int32_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* act_q, int64_t lda, const void* weight_q, int64_t ldb,
    float act_scale, const void* weight_scale,
    void* output, int64_t ldd,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* act_q, int64_t lda, const void* weight_q, int64_t ldb,
    const void* output, int64_t ldd);

/* The same contraction with the int32 accumulators written as they are
 * (D is int32 [M,N]).  Exists so callers and tests can check the integer
 * result bit for bit, as the reference's CPU oracle defines it
 * (crates/baracuda-kernelgen/src/oracle.rs:1289-1372 over I32 operands).
 * alpha must be 1 and beta 0. */
int32_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);

/* ---------------------------------------------------------------------------
 * FP8 e4m3 GEMM, f32 accumulate on tcgen05, f32 scales, bf16 out:
 *   D[i,j] = bf16( alpha * ((sa * sb) * acc[i,j]) )
 * with (sa, sb) = (scale_a[0], scale_b[0]) for scale_mode 0 and
 * (scale_a[i], scale_b[j]) for scale_mode 1.
 * Replaces baracuda_kernels_gemm_fp8_e4m3_rcr_sm89_run
 *   (crates/baracuda-kernels-sys/kernels/gemm/gemm_fp8_e4m3_rcr_sm89.cu:31-50),
 * whose output is e4m3 with a scalar alpha only.
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    const void* scale_a, const void* scale_b, int32_t scale_mode,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);

/* f32 accumulators of the e4m3 contraction (D is float [M,N]); alpha 1, beta 0. */
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);

/* ---------------------------------------------------------------------------
 * The reference's own 8-bit-out GEMM contracts on tcgen05, same signatures, arch tag sm100a:
 *   s8:   D = sat_s8( rint_even( alpha*(float)acc + beta*(float)C ) )            (D, C int8)
 *         drop-in for baracuda_cutlass_gemm_s8_rcr_sm80_run / IntGemmPlan<S8> Rcr, identity epilogue
 *         (crates/baracuda-cutlass-kernels-sys/kernels/gemm_s8_rcr_sm80.cu:169-198,
 *          crates/baracuda-kernels/src/gemm/int_gemm.rs:48-637)
 *   e4m3: D = sat_e4m3( alpha*acc + beta*dequant(C) )                            (D, C e4m3)
 *         drop-in for baracuda_kernels_gemm_fp8_e4m3_rcr_sm89_run / Fp8GemmPlan Rcr, identity epilogue
 *         (crates/baracuda-kernels-sys/kernels/gemm/gemm_fp8_e4m3_rcr_sm89.cu:31-67)
 * Each product and the sum are rounded in f32, as the reference's test oracles compute them
 * (crates/baracuda-kernels/tests/int8_rrr_smoke.rs:76-131, fp8_e4m3_rcr_smoke.rs:66-93).
 * beta != 0 needs C (ldc >= n); with beta == 0, C is not read.
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_gemm_s8_rcr_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_s8_rcr_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_s8_rcr_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd,
    float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_workspace_size(int32_t m, int32_t n, int32_t k);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k,
    const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, const void* d, int64_t ldd);

/* ---------------------------------------------------------------------------
 * "rrr" twins: the weight is row-major [K,N] (ldb >= n), the layout of the reference's bespoke GEMMs
 *   baracuda_kernels_gemm_s8_rrr_sm80_run (crates/baracuda-kernels-sys/kernels/gemm/gemm_s8_rrr_sm80.cu:28-64)
 *   baracuda_kernels_gemm_fp8_e4m3_rrr_sm89_run (crates/baracuda-kernels-sys/kernels/include/baracuda_fp8_rrr_sm89.cuh).
 * Same arguments and results as the "rcr" symbols of the same name; the weight tile is fed to tcgen05 as an
 * MN-major operand.  Alignment: b 16-byte aligned, ldb a multiple of 16.
 * ------------------------------------------------------------------------- */
#define BARACUDA_Q_DECLARE_GEMM_TAIL(NAME)                                                                  \
    size_t NAME##_workspace_size(int32_t m, int32_t n, int32_t k);                                          \
    int32_t NAME##_can_implement(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, \
                                 int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd);
int32_t baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b,
    float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_GEMM_TAIL(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a)
int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode,
    float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_GEMM_TAIL(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a)
int32_t baracuda_kernels_gemm_s8_rrr_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd, float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_GEMM_TAIL(baracuda_kernels_gemm_s8_rrr_s32_sm100a)
int32_t baracuda_kernels_gemm_s8_rrr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd, float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_GEMM_TAIL(baracuda_kernels_gemm_s8_rrr_sm100a)
int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
    const void* c, int64_t ldc, void* d, int64_t ldd, float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_GEMM_TAIL(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a)

/* ---------------------------------------------------------------------------
 * Fused bias / activation epilogues: the reference's EpilogueKind chain
 * (crates/baracuda-kernel-vocab/src/layout.rs:69-96) on the 8-bit-out contracts above, computed in f32
 * registers before the one saturating store (crates/baracuda-kernels-sys/kernels/include/
 * baracuda_epilogue_int8.cuh:37-95; the bias pointer sits before alpha as in
 * baracuda_kernels_gemm_s8_rrr_sm80_bias_relu_f32_run, crates/baracuda-kernels-sys/src/lib.rs):
 *     z = alpha*acc + beta*C + bias[j]      bias: float[N] ("f32") or int32[N] ("i32", converted to float)
 *     z = relu(z) | gelu(z) = z/2*(1+erf(z/sqrt 2)) | silu(z) = z/(1+exp(-z))
 *     D = sat_s8(rint_even(z))   or   D = sat_e4m3(z)
 * Named variants replace the reference's symbol of the same suffix; the *_epilogue_run forms take the chain as
 * arguments: epilogue 0 identity (bias ignored), 1 bias, 2 bias+relu, 3 bias+gelu, 4 bias+silu;
 * bias_kind 1 float[N], 2 int32[N] (s8 only).  Status 2 when epilogue > 0 and bias is null or bias_kind is not
 * one of those.  workspace_size / can_implement are those of the identity symbol of the same family.
 * ------------------------------------------------------------------------- */
#define BARACUDA_Q_EPILOGUE_IDENTITY 0
#define BARACUDA_Q_EPILOGUE_BIAS 1
#define BARACUDA_Q_EPILOGUE_BIAS_RELU 2
#define BARACUDA_Q_EPILOGUE_BIAS_GELU 3
#define BARACUDA_Q_EPILOGUE_BIAS_SILU 4
#define BARACUDA_Q_BIAS_F32 1
#define BARACUDA_Q_BIAS_I32 2
#define BARACUDA_Q_DECLARE_EPILOGUE_RUN(NAME)                                                                        \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,            \
                 const void* c, int64_t ldc, void* d, int64_t ldd, const void* bias, int32_t bias_kind,              \
                 int32_t epilogue, float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_EPILOGUE_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_EPILOGUE_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_epilogue_run)
#define BARACUDA_Q_DECLARE_BIAS_RUN(NAME)                                                                            \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,            \
                 const void* c, int64_t ldc, void* d, int64_t ldd, const void* bias, float alpha, float beta,        \
                 void* workspace, size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_relu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_gelu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_silu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_relu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_gelu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_bias_silu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_relu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_gelu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_silu_f32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_relu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_gelu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_bias_silu_i32_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_relu_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_gelu_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_silu_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_relu_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_gelu_run)
BARACUDA_Q_DECLARE_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_silu_run)

/* The bf16-out SKUs with the same chain (no counterpart symbol in the reference; the quantized-linear forward
 * with a bias, bindings/burn/baracuda-burn/src/ops/quantize.rs, is the caller it serves):
 *     D = bf16( act( alpha * ((scale_a[i]*scale_b[j]) * acc) + beta * C[i,j] + bias[j] ) ),  bias float[N];
 * C is bf16 [M, ldc] and may be D itself; beta != 0 needs C (status 2 without it), with beta == 0 C is not read.
 * scale_mode as for the fp8 bf16 symbol; the w8a8 symbols ignore it (always per row x per column; the per-tensor
 * activation scale of SmoothQuant has its own symbol, baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run). */
#define BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(NAME)                                                                   \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,            \
                 const void* c, int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b,         \
                 int32_t scale_mode, const void* bias, int32_t epilogue, float alpha, float beta, void* workspace,   \
                 size_t workspace_bytes, void* stream);
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_epilogue_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_epilogue_run)

/* The bf16-out GEMMs as programmatic dependent launches, chosen per call: the arguments of *_bf16_sm100a_epilogue_run
 * (epilogue 0 and bias NULL for the plain GEMM).  The kernel may start while the previous kernel of `stream` is still
 * finishing -- in a layer chain, on the SMs its last, partly filled wave leaves idle -- and requests its first ring of
 * WEIGHT tiles during that overlap; activations, scales, bias, C and D are touched only after the previous kernel has
 * completed and its writes are visible.  The caller promises that the kernel launched just before on this stream does
 * not write `b` (static model weights).  Same results and statuses as the plain symbols.  No counterpart in the
 * reference. */
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_pdl_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_pdl_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_pdl_run)
BARACUDA_Q_DECLARE_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_pdl_run)

/* ---------------------------------------------------------------------------
 * Gated-MLP up-projection in one launch: D[M, F] = bf16( silu(z_gate) * z_up ),
 *   z[m, j] = alpha * (scale_a[m] * scale_b[j]) * acc[m, j] (+ bias[j]),  silu(z) = z / (1 + exp(-z)),
 * over ONE weight `b_gate_up` [n2 = 2F, K] that holds the gate and up projections interleaved in blocks of 32 rows:
 * rows 64b .. 64b+31 are gate rows 32b .. 32b+31, rows 64b+32 .. 64b+63 the matching up rows; scale_b and the
 * optional float bias are [n2] in the same order (baracuda_kernels_q_interleave_gate_up_run builds all three).
 * No counterpart in the reference: its EpilogueKind (crates/baracuda-kernel-vocab/src/layout.rs:69-96) stops at
 * BiasSilu, so a gated MLP there is two GEMMs (or one of width 2F) followed by an elementwise pass over [M, 2F];
 * here the [M, 2F] intermediate never reaches memory.
 * Status: n2 not a multiple of 64 -> 3; d not 16-byte aligned or ldd not a multiple of 8 -> 1; ldd < n2 / 2 -> 2;
 * the other rules are those of the bf16 GEMM above.  workspace_size is 0.
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run(
    int32_t m, int32_t n2, int32_t k,
    const void* a, int64_t lda, const void* b_gate_up, int64_t ldb,
    void* d, int64_t ldd,
    const void* scale_a, const void* scale_b, const void* bias /* float[n2] or NULL */,
    float alpha,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_workspace_size(int32_t m, int32_t n2, int32_t k);
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement(
    int32_t m, int32_t n2, int32_t k,
    const void* a, int64_t lda, const void* b_gate_up, int64_t ldb,
    const void* d, int64_t ldd);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_run(
    int32_t m, int32_t n2, int32_t k,
    const void* a, int64_t lda, const void* b_gate_up, int64_t ldb,
    void* d, int64_t ldd,
    const void* scale_a, const void* scale_b, int32_t scale_mode, const void* bias /* float[n2] or NULL */,
    float alpha,
    void* workspace, size_t workspace_bytes, void* stream);
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_workspace_size(int32_t m, int32_t n2, int32_t k);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_can_implement(
    int32_t m, int32_t n2, int32_t k,
    const void* a, int64_t lda, const void* b_gate_up, int64_t ldb,
    const void* d, int64_t ldd);
/* out row 64b + i = gate row 32b + i (i < 32) or up row 32b + i - 32; rows are `row_bytes` bytes (K for a weight,
 * 4 for a scale or bias vector with pitches of 4), pitches in bytes; f_rows (= F) must be a multiple of 32. */
int32_t baracuda_kernels_q_interleave_gate_up_run(
    int64_t f_rows, int64_t row_bytes,
    const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch,
    void* out, int64_t out_pitch, void* stream);

/* ---------------------------------------------------------------------------
 * Decode GEMV with int8 weights, m = 1 (and the skinny extension m <= 8):
 *   D[g,r,j] = bf16( alpha * ((scale_a[g,r] * scale_b[g,j]) * (float)acc) + beta * D[g,r,j] )
 * Argument order is that of baracuda_kernels_gemv_dense_m1_bf16_run
 *   (crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:267-281)
 * with the two scale vectors (and their batch strides) inserted before `d`.
 * stride_b == 0 broadcasts the weights over batch slots, as in the reference.
 * Misaligned or ragged operands are served by a slower byte-load kernel, so
 * status 1 is never returned by this family.
 * layout 0 (row-major weights) needs a workspace when K is split over CTAs:
 * query *_workspace_size and pass at least that much, 16-byte aligned.
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    float alpha, float beta,
    const void* a, int64_t lda, int64_t stride_a,
    const void* b, int64_t ldb, int64_t stride_b,
    const void* scale_a, int64_t stride_scale_a,
    const void* scale_b, int64_t stride_scale_b,
    void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    int64_t lda, int64_t ldb, int64_t ldd,
    int64_t stride_a, int64_t stride_b, int64_t stride_d);
size_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout);
/* The same call launched with programmatic dependent launch (per call, no process state): the kernel may start
 * while the previous kernel of `stream` is still finishing and fetches WEIGHTS during that overlap; activations,
 * scales, workspace and outputs are touched only after the previous kernel has completed and its writes are
 * visible.  The caller promises that the kernel launched just before on this stream does not write `b`
 * (true for a decode loop over static weights).  Same arguments, results and statuses as *_run; also serves
 * the s32 and the fused-quantiser forms below.  No counterpart in the reference (its GEMV predates the feature). */
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    float alpha, float beta,
    const void* a, int64_t lda, int64_t stride_a,
    const void* b, int64_t ldb, int64_t stride_b,
    const void* scale_a, int64_t stride_scale_a,
    const void* scale_b, int64_t stride_scale_b,
    void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream);

/* The same GEMV for callers that must not allocate device memory (a serving loop that has
 * given every byte to its own arena, a plugin host that forbids side allocations): the
 * split-K scratch of the row-major weight layout comes from a fixed array inside the loaded
 * library instead of a caller workspace, so only inputs and outputs are passed.
 * This entry point has no counterpart in the reference.
 *   - The array holds BARACUDA_Q_GEMV_STATIC_SCRATCH_BYTES (8 MiB) on every GPU that loads
 *     the library, until the process exits.  A shape whose *_workspace_size exceeds it is
 *     rejected with status 4; *_static_ws_capacity returns the limit.  What fits: the scratch is
 *     (160 + ceil(N / 1024)) * m * 4 KiB for row-major weights with up to 380 928 row pieces
 *     (ceil(N / 1024) * K), so every m <= 8 fits for N <= 98 304 within that bound -- e.g. all decode
 *     projections of an 8B- or 70B-class model (4096 x 14336, 14336 x 4096, 8192 x 28672 at m = 8:
 *     5.4 to 6.0 MiB); K-contiguous weights (layout 1) need no scratch at all.  Invalid problems
 *     report the same status as the regular entry point (the size limit is checked last).
 *   - Nothing is allocated or freed, here or in any routine it calls.
 *   - The first call on a device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps whatever the last call left; the part that
 *     must start at zero is cleared on the stream at the start of each call.  Two calls that
 *     can overlap on the GPU (different streams, no ordering between them) race on it: order
 *     them, or use the workspace entry point for one of them.
 * Results are identical to baracuda_kernels_gemv_q8_m1_bf16_sm100a_run. */
#define BARACUDA_Q_GEMV_STATIC_SCRATCH_BYTES (8u << 20)
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    float alpha, float beta,
    const void* a, int64_t lda, int64_t stride_a,
    const void* b, int64_t ldb, int64_t stride_b,
    const void* scale_a, int64_t stride_scale_a,
    const void* scale_b, int64_t stride_scale_b,
    void* d, int64_t ldd, int64_t stride_d,
    void* stream);
size_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity(void);

/* Decode step in one launch: the per-token quantiser of QuantizedLinearPlan's first launch
 * (dynamic_range_quantize_per_token_symmetric_kernel, crates/baracuda-kernels-sys/kernels/include/
 * baracuda_quantize_compose.cuh:144-201) runs inside the GEMV.  x is bf16 [m, ldx] (m <= 8), b the int8 weight
 * [N, K] (K contiguous), scale_b float[N]; every CTA derives scale_a[r] = absmax(x[r,:]) / qmax (1.0 for a zero row),
 * quantises the activation fragments it needs with q = clamp(rint_even(x * (1/scale_a)), qmin, qmax) and the result is
 *     D = bf16( alpha * (scale_a[r]*scale_b[j]) * sum_k q[r,k] * b[j,k] + beta * D )
 * -- the bits of quantize_per_token_sym_bf16_s8 followed by gemv_q8_m1_bf16.  scale_a_out (float[m]) receives the
 * scales when not NULL.  Served shapes: K a multiple of 512 with 16 % (K / 512) == 0 (512 ... 8192), ldx a multiple of
 * 8, ldb a multiple of 16, 16-byte aligned x and b; anything else returns status 3 from can_implement / run and the
 * caller takes the two-launch path.  No workspace. */
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run(
    int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax,
    float alpha, float beta,
    const void* x_bf16, int64_t ldx, const void* b, int64_t ldb, const void* scale_b,
    void* scale_a_out, void* d, int64_t ldd,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax,
    float alpha, float beta,
    const void* x_bf16, int64_t ldx, const void* b, int64_t ldb, const void* scale_b,
    void* scale_a_out, void* d, int64_t ldd,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(
    int32_t m, int32_t n, int32_t k, int64_t ldx, int64_t ldb, int64_t ldd);

/* The int32 sums of the same GEMV (D is int32); alpha 1, beta 0, no scales. */
int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    float alpha, float beta,
    const void* a, int64_t lda, int64_t stride_a,
    const void* b, int64_t ldb, int64_t stride_b,
    void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    float alpha, float beta,
    const void* a, int64_t lda, int64_t stride_a,
    const void* b, int64_t ldb, int64_t stride_b,
    void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout,
    int64_t lda, int64_t ldb, int64_t ldd,
    int64_t stride_a, int64_t stride_b, int64_t stride_d);
size_t baracuda_kernels_gemv_q8_m1_s32_sm100a_workspace_size(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout);

/* ---------------------------------------------------------------------------
 * Per-token (per-row) symmetric activation quantizer, the step in front of the GEMM / GEMV:
 *   scale[r] = absmax(x[r,:]) / qmax (1.0 for an all-zero row)
 *   q[r,c]   = clamp(rint_even(x[r,c] * (1/scale[r])), qmin, qmax)       (s8)
 *   q[r,c]   = e4m3_satfinite(x[r,c] * (1/scale[r])), qmax = 448         (e4m3)
 * Same recipe and argument order as
 *   baracuda_kernels_dynamic_range_quantize_per_token_sym_f32_s8_run
 *   (crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:144-201, 309-326),
 * with row pitches added (elements) and the scale always written as f32 (what the GEMM epilogues
 * read).  Input f32 or bf16 [rows, cols]; no limit on rows (the reference stops at 65 535).
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_quantize_per_token_sym_f32_s8_sm100a_run(
    int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
    const void* input, int64_t ld_in, void* scale, void* output, int64_t ld_out,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_quantize_per_token_sym_bf16_s8_sm100a_run(
    int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
    const void* input, int64_t ld_in, void* scale, void* output, int64_t ld_out,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_quantize_per_token_sym_f32_e4m3_sm100a_run(
    int32_t rows, int32_t cols,
    const void* input, int64_t ld_in, void* scale, void* output, int64_t ld_out,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_quantize_per_token_sym_bf16_e4m3_sm100a_run(
    int32_t rows, int32_t cols,
    const void* input, int64_t ld_in, void* scale, void* output, int64_t ld_out,
    void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Column-parallel (N-sharded) GEMM inside one NVLink box.  Rank r owns rows
 * [r*n_local, (r+1)*n_local) of the [N,K] weight and the matching scale_b slice;
 * activations and scale_a are replicated; every rank computes D[:, slice].
 * Follows ColumnParallelLinearPlan::forward
 *   (crates/baracuda-megatron/src/lib.rs:842-905: local GEMM, then all_gather)
 * with the reference's cuBLAS GEMM replaced by the tcgen05 kernels above.
 * `gather` selects what happens to the output:
 *   0  leave it sharded: d_local [M, n_local] only;
 *   1  ncclAllGather of d_local (contiguous, ldd == n_local) into d_full,
 *      rank-major [world, M, n_local] — the reference's layout (lib.rs:824-836);
 *   2  fused: the GEMM epilogue stores each bf16 tile into all `world` buffers
 *      peer_d[0..world) (row-major [M, ldd_full], peer-mapped device pointers,
 *      peer_d[rank] being this rank's own) at column offset rank*n_local, so the
 *      NVLink transfer overlaps the tensor-core work tile by tile and the result
 *      is a true row-major [M, N].  The caller orders the ranks afterwards
 *      (baracuda_q_nccl_stream_barrier or a host barrier) before reading.
 *   3  fused through the NVLink switch: as 2, but each tile is stored ONCE, with multimem.st, to the multicast
 *      address of the `world` buffers (peer_d[world], one entry more than for 2; the unicast pointers
 *      peer_d[0..world) are still required and serve shapes whose rows cannot take 16-byte stores).  A rank then
 *      sends M*n_local*2 bytes instead of (world-1) times that; the switch replicates.  Needs buffers bound to
 *      one multicast object (a symmetric-memory allocator that offers a multicast pointer).
 * `comm` is the ncclComm_t of this rank (may be NULL for gather 0, 2 and 3).
 * Extra statuses: 6 NCCL not loadable, 7 NCCL call failed.
 * ------------------------------------------------------------------------- */
#define BARACUDA_Q_GATHER_NONE 0
#define BARACUDA_Q_GATHER_NCCL 1
#define BARACUDA_Q_GATHER_FUSED_PEER_STORE 2
#define BARACUDA_Q_GATHER_FUSED_MULTICAST 3
#define BARACUDA_Q_MAX_PEERS 8

int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather,
    int32_t m, int32_t n_local, int32_t k,
    const void* a, int64_t lda, const void* b_local, int64_t ldb,
    void* d_local, int64_t ldd,
    const void* scale_a, const void* scale_b_local, int32_t scale_mode, float alpha,
    void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather,
    int32_t m, int32_t n_local, int32_t k,
    const void* a, int64_t lda, const void* b_local, int64_t ldb,
    void* d_local, int64_t ldd,
    const void* scale_a, const void* scale_b_local, float alpha,
    void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream);

/* The same for a row-major weight [K, N] (the "rrr" layout): rank r's shard is the column range
 * [r*n_local, (r+1)*n_local) of every weight row, so b_local points at column r*n_local of the full matrix and
 * ldb stays the full N (>= n_local); every gather mode is served. */
int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather,
    int32_t m, int32_t n_local, int32_t k,
    const void* a, int64_t lda, const void* b_local, int64_t ldb,
    void* d_local, int64_t ldd,
    const void* scale_a, const void* scale_b_local, int32_t scale_mode, float alpha,
    void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather,
    int32_t m, int32_t n_local, int32_t k,
    const void* a, int64_t lda, const void* b_local, int64_t ldb,
    void* d_local, int64_t ldd,
    const void* scale_a, const void* scale_b_local, float alpha,
    void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * K-sharded ("row-parallel") forward, the partner of the N-sharded one in an MLP block
 * (RowParallelLinearPlan::forward, crates/baracuda-megatron/src/lib.rs:1002-1200): rank r holds
 * X_local [M, K/world] and W_local [N, K/world]; Y = sum over ranks of X_local x W_local^T.
 * Each rank's tcgen05 GEMM leaves raw accumulators (int32 / f32) in `workspace` ([M, N], 4 bytes
 * each, 16-byte aligned; *_kshard_workspace_size), `reduce` = BARACUDA_Q_REDUCE_NCCL adds them with
 * ncclAllReduce(sum) on the caller's stream, and one dequant pass writes
 *     D = bf16( (scale_a[i] * scale_b[j]) * acc * alpha + bias[j] )      (bias float[N] or NULL, added once)
 * on every rank.  scale_a must be the same on all ranks (quantise the activations with a per-token scale
 * taken over the whole K); int32 sums add exactly, so the W8A8 result equals the unsharded GEMM bit for bit.
 * BARACUDA_Q_REDUCE_NONE skips the collective (world 1, or a caller that reduces the workspace itself).
 * ------------------------------------------------------------------------- */
#define BARACUDA_Q_REDUCE_NONE 0
#define BARACUDA_Q_REDUCE_NCCL 1
size_t baracuda_kernels_gemm_q8_kshard_workspace_size(int32_t m, int32_t n);
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(
    int32_t rank, int32_t world, void* comm, int32_t reduce,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* d, int64_t ldd, const void* scale_a, const void* scale_b,
    const void* bias, float alpha,
    void* workspace, size_t workspace_bytes, void* stream);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run(
    int32_t rank, int32_t world, void* comm, int32_t reduce,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode,
    const void* bias, float alpha,
    void* workspace, size_t workspace_bytes, void* stream);

/* The same forward with both exchanges fused into the kernels over peer-mapped memory (NVLink), no NCCL data path:
 *   1. the raw-accumulator GEMM's epilogue stores rows [j*M/world, (j+1)*M/world) of its partial sums into rank j's
 *      staging buffer peer_staging[j] -- [world][M/world][N] 32-bit words, slot = the storing rank -- while the
 *      tensor cores work on the next tile (GEMM + reduce-scatter in one kernel);
 *   2. each rank adds the `world` slots of its own staging buffer in slot order, applies scales / alpha / bias, and
 *      stores its M/world bf16 rows into every rank's result peer_y[q] (row pitch ldy) (reduce + all-gather in one kernel).
 * A one-float ncclAllReduce on `barrier_scratch` orders the ranks after each step, so `comm` is still needed.
 * peer_y and peer_staging are arrays of `world` device pointers valid on this rank (CUDA IPC or a symmetric-memory
 * allocator); M must divide by world, world <= BARACUDA_Q_MAX_PEERS; every rank passes the same arguments.
 * No counterpart in the reference (its RowParallelLinearPlan calls ncclAllReduce). */
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run(
    int32_t rank, int32_t world, void* comm,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    const void* bias, float alpha,
    void* const* peer_staging, void* barrier_scratch, void* stream);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run(
    int32_t rank, int32_t world, void* comm,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b, int32_t scale_mode,
    const void* bias, float alpha,
    void* const* peer_staging, void* barrier_scratch, void* stream);

/* The same fused forward with the two meeting points done by a flag barrier over peer memory instead of the one-float
 * all-reduce: no communicator, no NCCL.  peer_flags is an array of `world` device pointers valid on this rank, one
 * flag buffer per rank (baracuda_q_peer_barrier_flag_bytes() bytes each, peer-mapped like the other buffers and
 * zero-filled ONCE before first use; the barriers keep their own epoch in it).  Every rank must issue the same sequence
 * of calls on these buffers. */
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run(
    int32_t rank, int32_t world,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    const void* bias, float alpha,
    void* const* peer_staging, void* const* peer_flags, void* stream);
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run(
    int32_t rank, int32_t world,
    int32_t m, int32_t n, int32_t k_local,
    const void* a_local, int64_t lda, const void* b_local, int64_t ldb,
    void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b, int32_t scale_mode,
    const void* bias, float alpha,
    void* const* peer_staging, void* const* peer_flags, void* stream);

/* The barrier itself, a one-block kernel on `stream`: this rank stores its next epoch into its slot of every rank's
 * flag buffer and waits until every slot of its own buffer has reached it.  Whatever a rank wrote to peer memory on
 * its stream before the barrier is visible to what every rank launches after it -- the ordering the fused peer-store
 * modes need once per step (it replaces baracuda_q_nccl_stream_barrier there).  The wait is bounded: after
 * limit_cycles SM clock cycles (0 = the default of 2^31, about a second) the kernel gives up, the context stays usable
 * and baracuda_kernels_q_device_status() returns 301 once.  Ranks that share a GPU must not use it: the kernels wait
 * on one another. */
int32_t baracuda_q_peer_barrier_run(void* const* peer_flags, int32_t rank, int32_t world, int64_t limit_cycles, void* stream);
size_t baracuda_q_peer_barrier_flag_bytes(void);

/* Communicator helpers over the run-time-loaded NCCL
 * (Communicator::{new_with_id, all_gather}, crates/baracuda-nccl/src/lib.rs:243-261, 468-489).
 * unique_id writes the 128-byte ncclUniqueId; rank 0 creates it and the caller
 * distributes it.  stream_barrier is a one-float all-reduce used to order the
 * ranks on their streams after the fused peer-store mode. */
int32_t baracuda_q_nccl_version(void);
int32_t baracuda_q_nccl_unique_id(void* id_out_128_bytes);
int32_t baracuda_q_nccl_comm_init_rank(void** comm_out, int32_t world, const void* id_128_bytes, int32_t rank);
int32_t baracuda_q_nccl_comm_destroy(void* comm);
int32_t baracuda_q_nccl_stream_barrier(void* comm, void* scratch_one_float, void* stream);
/* Replicates a row-sharded operand over NVLink: every rank contributes `bytes_per_rank` contiguous bytes at `send`
 * and receives all ranks' blocks, in rank order, at `recv` (world * bytes_per_rank bytes; send may point at this
 * rank's block inside recv).  The column-parallel layer uses it so that each rank uploads only 1/world of the
 * activation rows (and of scale_a) from the host and the rest arrives from its peers
 * (Communicator::all_gather, crates/baracuda-nccl/src/lib.rs:468-489).  world == 1 is a device copy. */
int32_t baracuda_q_nccl_all_gather_bytes(void* comm, int32_t world, const void* send, void* recv, size_t bytes_per_rank,
                                         void* stream);

/* ---------------------------------------------------------------------------
 * Diagnostics and test hooks (no counterpart in the reference).
 * device_status: synchronous read-and-clear of the word a kernel sets when one
 * of its bounded barrier waits ran out (0 = none; the code names the kernel and
 * the waiting role: 101..104 1-CTA GEMM, 111..115 CTA-pair GEMM, 121..123 cluster split-K GEMM, 201..207 streaming GEMVs, 299 the self-test, 301 the peer barrier).  Call it after synchronising the stream.
 * set_tuning: forces a kernel choice for the CALLING THREAD only (thread-local; other threads' launches are not
 * affected, nothing process-wide is kept), so tests can run every kernel on the same shapes:
 *   key 0  GEMM tile: 0 automatic; 64, 128, 256 = 1-CTA kernel with that N-tile; 512 = the CTA-pair kernel;
 *   key 1  GEMV kernel: 0 automatic; 1 bulk-copy dp4a kernel; 2 register-streaming kernel; 3 tensor-core streaming
 *          kernel also for m = 1; 8 direct-load split-K kernel (row-major weights); 9 byte-load kernel;
 *   key 2  CTA-pair tile width: 0 automatic, 256, 224, 192, 128; 2 = the mixed 256 / 128 schedule;
 *   key 4  GEMM epilogue store path: 0 automatic, 1 per-thread direct stores, 2 rows staged through shared memory.
 *   key 5  CTA-pair GEMM epilogue warps: 0 automatic (eight for gelu / silu chains on at most two waves of tiles), 4, 8.
 *   key 6  split-K inside thread-block clusters (bf16-out and 8-bit-out GEMMs): 0 automatic, 1 never, 2 or 4 = that many
 *          K slices of 128 x 128 tiles, 256 = two slices of 128 x 256 tiles ([N,K] weights only), on any shape with at
 *          least that many 128-byte K blocks.
 * Any other key or value returns 2.
 * selftest_bounded_wait: launches one thread that waits, for at most limit_cycles SM clock cycles
 * (1 .. 2^28), on a barrier that nothing completes -- the time-out path of every kernel here.  After the
 * stream is synchronised device_status() returns 299 once and the context is as usable as before.
 * ------------------------------------------------------------------------- */
int32_t baracuda_kernels_q_device_status(void);
int32_t baracuda_kernels_q_selftest_bounded_wait(int64_t limit_cycles, void* stream);
int32_t baracuda_kernels_q_set_tuning(int32_t key, int32_t value);

#ifdef __cplusplus
}
#endif
#endif /* BARACUDA_KERNELS_Q_H */
