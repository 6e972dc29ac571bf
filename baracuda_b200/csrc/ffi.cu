// The flat C symbols of include/baracuda_kernels_q.h: argument validation in
// the reference's order (negative dims -> 2, empty -> 0 without a launch, null
// pointers -> 2, leading-dimension minimums -> 2, alignment -> 1), then the
// launch.  No allocation, no host synchronisation, no library state.

#include "../../include/baracuda_kernels_q.h"
#include "launch.h"

namespace {

// Test hooks of baracuda_kernels_q_set_tuning: per calling thread, so one thread forcing a kernel variant never
// changes what another thread's launches do (the boundary keeps no process-wide mutable state).
struct ThreadTuning {
    int32_t force_block_n = 0;
    int32_t gemv_variant = 0;
    int32_t force_pair_tile_n = 0;
    int32_t direct_stores = 0;
    int32_t epilogue_warps = 0;
    int32_t cluster_split_k = 0;
};
thread_local ThreadTuning t_tuning;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Longest K for which an int8 contraction cannot leave the 32-bit accumulator: K * 128 * 128 < 2^31.  The reference's
// tensor-core path saturates each mma.sync (".satfinite", baracuda_int8_rrr_sm80.cuh:86-92) and its test oracle adds
// with saturation (crates/baracuda-kernels/tests/int8_rrr_smoke.rs:76-131); what tcgen05.mma kind::i8 does on overflow
// is not specified, so beyond this K the int8 symbols answer UNSUPPORTED instead of returning sums that may differ.
constexpr int32_t kMaxInt8K = 131071;
int32_t int8_k_status(int32_t k) { return k > kMaxInt8K ? bq::BQ_STATUS_UNSUPPORTED : bq::BQ_STATUS_OK; }

// Shape / leading-dimension / alignment rules shared by run and can_implement.
// Pointer arguments may be null here (can_implement is callable before the
// buffers exist); alignment of a null pointer is not judged.
// `layout` is the weight storage: RCR = [N,K] rows of K (ldb >= k), RRR = row-major [K,N] (ldb >= n).
int32_t gemm_validate(int32_t layout, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b,
                      int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd) {
    (void)ldc;
    (void)d;
    if (m < 0 || n < 0 || k < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    const int64_t min_k = k > 0 ? k : 1;
    const int64_t min_n = n > 0 ? n : 1;
    const bool rrr = layout == bq::BQ_LAYOUT_RRR;
    if (lda < min_k || ldb < (rrr ? min_n : min_k) || ldd < min_n) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (c != nullptr) return bq::BQ_STATUS_UNSUPPORTED;
    // TMA reads both operands: 16-byte aligned bases and row pitches
    if ((a && !aligned16(a)) || (b && !aligned16(b))) return bq::BQ_STATUS_MISALIGNED;
    const int64_t b_rows = rrr ? k : n;
    if (k > 0 && ((m > 1 && (lda & 15)) || (b_rows > 1 && (ldb & 15)))) return bq::BQ_STATUS_MISALIGNED;
    return bq::BQ_STATUS_OK;
}

int32_t gemm_rcr_validate(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
                          const void* c, int64_t ldc, const void* d, int64_t ldd) {
    return gemm_validate(bq::BQ_LAYOUT_RCR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
}

// The bf16-out SKUs take C (bf16 [M, ldc], may alias D) and beta like the reference's GEMM family.
int32_t gemm_bf16_validate(int32_t layout, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b,
                           int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd) {
    const int32_t st = gemm_validate(layout, m, n, k, a, lda, b, ldb, nullptr, 0, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (c != nullptr && ldc < (n > 0 ? n : 1)) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (c != nullptr && (reinterpret_cast<uintptr_t>(c) & 1u)) return bq::BQ_STATUS_MISALIGNED;
    return bq::BQ_STATUS_OK;
}

int32_t gemm_rcr_bf16_validate(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
                               const void* c, int64_t ldc, const void* d, int64_t ldd) {
    return gemm_bf16_validate(bq::BQ_LAYOUT_RCR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
}

// Fused epilogue chain of the reference's EpilogueKind (crates/baracuda-kernel-vocab/src/layout.rs:69-96):
// 0 Identity, 1 Bias, 2 BiasRelu, 3 BiasGelu, 4 BiasSilu; bias_kind 1 = float[N], 2 = int32[N].
struct Epilogue {
    const void* bias = nullptr;
    int32_t bias_kind = 0;
    int32_t kind = 0;
};

// 0 ok; 2 when the chain and the bias pointer disagree
int32_t epilogue_validate(const Epilogue& e, bool allow_i32_bias) {
    if (e.kind < 0 || e.kind > 4) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (e.kind == 0) return bq::BQ_STATUS_OK;
    if (!e.bias) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (e.bias_kind != 1 && !(allow_i32_bias && e.bias_kind == 2)) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (reinterpret_cast<uintptr_t>(e.bias) & 3u) return bq::BQ_STATUS_MISALIGNED;
    return bq::BQ_STATUS_OK;
}

void epilogue_apply(const Epilogue& e, bq::GemmDesc& g) {
    g.bias = e.kind > 0 ? e.bias : nullptr;
    g.bias_kind = e.kind > 0 ? e.bias_kind : 0;
    g.act = e.kind >= 2 ? e.kind - 1 : 0;  // 1 relu, 2 gelu, 3 silu
}

int32_t gemm_run(int32_t layout, int32_t kind, int32_t raw, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                 const void* b, int64_t ldb, const void* c, int64_t ldc, void* d, int64_t ldd, const void* scale_a,
                 const void* scale_b, int32_t scale_mode, float alpha, float beta, void* stream,
                 const Epilogue& epi = Epilogue(), int32_t pdl = 0);

int32_t gemm_rcr_run(int32_t kind, int32_t raw, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                     const void* b, int64_t ldb, const void* c, int64_t ldc, void* d, int64_t ldd,
                     const void* scale_a, const void* scale_b, int32_t scale_mode, float alpha, float beta,
                     void* stream) {
    return gemm_run(bq::BQ_LAYOUT_RCR, kind, raw, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b, scale_mode,
                    alpha, beta, stream);
}

int32_t gemm_run(int32_t layout, int32_t kind, int32_t raw, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                 const void* b, int64_t ldb, const void* c, int64_t ldc, void* d, int64_t ldd, const void* scale_a,
                 const void* scale_b, int32_t scale_mode, float alpha, float beta, void* stream, const Epilogue& epi,
                 int32_t pdl) {
    const int32_t st = raw ? gemm_validate(layout, m, n, k, a, lda, b, ldb, c, ldc, d, ldd)
                           : gemm_bf16_validate(layout, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (const int32_t es = epilogue_validate(epi, false); es != bq::BQ_STATUS_OK) return es;
    if (kind == bq::BQ_KIND_S8 && int8_k_status(k) != bq::BQ_STATUS_OK) return bq::BQ_STATUS_UNSUPPORTED;
    if (raw && epi.kind != 0) return bq::BQ_STATUS_UNSUPPORTED;
    if (k == 0 && (epi.kind != 0 || beta != 0.0f)) return bq::BQ_STATUS_UNSUPPORTED;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if (!d || (k > 0 && (!a || !b))) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (raw && beta != 0.0f) return bq::BQ_STATUS_UNSUPPORTED;
    if (beta != 0.0f && !c) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (raw) {
        if (alpha != 1.0f) return bq::BQ_STATUS_UNSUPPORTED;
    } else {
        if (!scale_a || !scale_b) return bq::BQ_STATUS_INVALID_PROBLEM;
        if (scale_mode != BARACUDA_Q_SCALE_PER_TENSOR && scale_mode != BARACUDA_Q_SCALE_PER_ROW_COL)
            return bq::BQ_STATUS_INVALID_PROBLEM;
    }
    bq::GemmDesc g = {};
    g.b_layout = layout;
    g.kind = kind;
    g.raw_out = raw;
    g.m = m;
    g.n = n;
    g.k = k;
    g.a = a;
    g.lda = lda;
    g.b = b;
    g.ldb = ldb;
    g.scale_a = static_cast<const float*>(scale_a);
    g.scale_b = static_cast<const float*>(scale_b);
    g.scale_mode = scale_mode;
    g.alpha = alpha;
    g.d = d;
    g.ldd = ldd;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    g.direct_stores = t_tuning.direct_stores;
    g.epilogue_warps = t_tuning.epilogue_warps;
    g.n_peers = 0;
    g.peer_ld = 0;
    g.peer_col0 = 0;
    g.peer_rank = 0;
    for (auto& pd : g.peer_d) pd = nullptr;
    epilogue_apply(epi, g);
    g.q8_out = 0;
    g.c = (!raw && beta != 0.0f) ? c : nullptr;  // beta == 0: C is not read
    g.ldc = ldc;
    g.beta = beta;
    g.pdl = pdl;
    g.cluster_split_k = t_tuning.cluster_split_k;
    return bq::launch_gemm_q8(g, static_cast<cudaStream_t>(stream));
}

// Gated-MLP up-projection: weight [n2, K] with gate and up rows interleaved in blocks of 32, D = silu(z_gate) * z_up
// as bf16 [M, n2 / 2].  No counterpart in the reference (its EpilogueKind has no gated form).
int32_t gemm_swiglu_validate(int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
                             const void* d, int64_t ldd) {
    if (m < 0 || n2 < 0 || k < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    const int64_t f = n2 / 2;
    const int32_t st = gemm_validate(bq::BQ_LAYOUT_RCR, m, n2, k, a, lda, b, ldb, nullptr, 0, d,
                                       ldd < (f > 0 ? f : 1) ? 0 : INT64_MAX);  // the output has n2 / 2 columns
    if (st != bq::BQ_STATUS_OK) return st;
    if (n2 % 64 != 0) return bq::BQ_STATUS_UNSUPPORTED;
    if ((d && !aligned16(d)) || (m > 1 && (ldd & 7))) return bq::BQ_STATUS_MISALIGNED;
    return bq::BQ_STATUS_OK;
}

int32_t gemm_swiglu_run(int32_t kind, int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b,
                        int64_t ldb, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode,
                        const void* bias, float alpha, void* stream) {
    const int32_t st = gemm_swiglu_validate(m, n2, k, a, lda, b, ldb, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (bias && (reinterpret_cast<uintptr_t>(bias) & 3u)) return bq::BQ_STATUS_MISALIGNED;
    if (kind == bq::BQ_KIND_S8 && int8_k_status(k) != bq::BQ_STATUS_OK) return bq::BQ_STATUS_UNSUPPORTED;
    if (k == 0 && bias) return bq::BQ_STATUS_UNSUPPORTED;
    if (m == 0 || n2 == 0) return bq::BQ_STATUS_OK;
    if (!d || (k > 0 && (!a || !b))) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (!scale_a || !scale_b) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (scale_mode != BARACUDA_Q_SCALE_PER_TENSOR && scale_mode != BARACUDA_Q_SCALE_PER_ROW_COL)
        return bq::BQ_STATUS_INVALID_PROBLEM;
    bq::GemmDesc g = {};
    g.b_layout = bq::BQ_LAYOUT_RCR;
    g.kind = kind;
    g.m = m;
    g.n = n2;
    g.k = k;
    g.a = a;
    g.lda = lda;
    g.b = b;
    g.ldb = ldb;
    g.scale_a = static_cast<const float*>(scale_a);
    g.scale_b = static_cast<const float*>(scale_b);
    g.scale_mode = scale_mode;
    g.alpha = alpha;
    g.d = d;
    g.ldd = ldd;
    g.bias = bias;
    g.bias_kind = bias ? 1 : 0;
    g.swiglu = 1;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    if (g.force_pair_tile_n % 64 != 0 && g.force_pair_tile_n != 2) g.force_pair_tile_n = 0;
    return bq::launch_gemm_q8(g, static_cast<cudaStream_t>(stream));
}

// The reference's own contract for the 8-bit GEMMs: D has the input type, D = sat(alpha*(A x B) + beta*C).
int32_t gemm_q8_validate(int32_t layout, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b,
                         int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd) {
    const int32_t st = gemm_validate(layout, m, n, k, a, lda, b, ldb, nullptr, 0, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (c != nullptr && ldc < (n > 0 ? n : 1)) return bq::BQ_STATUS_INVALID_PROBLEM;
    return bq::BQ_STATUS_OK;
}

int32_t gemm_q8_run(int32_t layout, int32_t kind, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                    const void* b, int64_t ldb, const void* c, int64_t ldc, void* d, int64_t ldd, float alpha, float beta,
                    void* stream, const Epilogue& epi = Epilogue()) {
    const int32_t st = gemm_q8_validate(layout, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (const int32_t es = epilogue_validate(epi, kind == bq::BQ_KIND_S8); es != bq::BQ_STATUS_OK) return es;
    if (kind == bq::BQ_KIND_S8 && int8_k_status(k) != bq::BQ_STATUS_OK) return bq::BQ_STATUS_UNSUPPORTED;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if (!d || (k > 0 && (!a || !b))) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (beta != 0.0f && !c) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (k == 0) return bq::BQ_STATUS_UNSUPPORTED;
    bq::GemmDesc g = {};
    g.b_layout = layout;
    g.kind = kind;
    g.raw_out = 0;
    g.q8_out = 1;
    g.c = (beta != 0.0f) ? c : nullptr;
    g.ldc = ldc;
    g.beta = beta;
    g.m = m;
    g.n = n;
    g.k = k;
    g.a = a;
    g.lda = lda;
    g.b = b;
    g.ldb = ldb;
    g.scale_a = nullptr;
    g.scale_b = nullptr;
    g.scale_mode = 0;
    g.alpha = alpha;
    g.d = d;
    g.ldd = ldd;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    epilogue_apply(epi, g);
    g.direct_stores = 1;
    g.epilogue_warps = t_tuning.epilogue_warps;
    g.cluster_split_k = t_tuning.cluster_split_k;
    g.n_peers = 0;
    g.peer_ld = 0;
    g.peer_col0 = 0;
    g.peer_rank = 0;
    for (auto& pd : g.peer_d) pd = nullptr;
    return bq::launch_gemm_q8(g, static_cast<cudaStream_t>(stream));
}

// Mirrors gemv_validate of the reference (gemv_dense.cu:101-122), widened to
// m <= 8 and to the second weight layout.
int32_t gemv_validate(int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, int64_t lda, int64_t ldb,
                      int64_t ldd, int64_t stride_d) {
    if (m < 0 || n < 0 || k < 0 || batch < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (m > 8) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (layout != bq::BQ_LAYOUT_RRR && layout != bq::BQ_LAYOUT_RCR) return bq::BQ_STATUS_INVALID_PROBLEM;
    const int64_t min_k = k > 0 ? k : 1;
    const int64_t min_n = n > 0 ? n : 1;
    const int64_t min_ldb = (layout == bq::BQ_LAYOUT_RRR) ? min_n : min_k;
    if (lda < min_k || ldb < min_ldb || ldd < min_n) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (batch > 1 && stride_d == 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    return int8_k_status(k);  // dp4a and mma.sync (without .satfinite) wrap: refuse K that could overflow
}

int32_t gemv_run(int32_t raw, int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha,
                 float beta, const void* a, int64_t lda, int64_t stride_a, const void* b, int64_t ldb,
                 int64_t stride_b, const void* scale_a, int64_t stride_scale_a, const void* scale_b,
                 int64_t stride_scale_b, void* d, int64_t ldd, int64_t stride_d, void* workspace,
                 size_t workspace_bytes, void* stream, int32_t pdl = 0) {
    const int32_t st = gemv_validate(m, n, k, batch, layout, lda, ldb, ldd, stride_d);
    if (st != bq::BQ_STATUS_OK) return st;
    if (m == 0 || n == 0 || batch == 0) return bq::BQ_STATUS_OK;
    if (!a || !b || !d) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (raw) {
        if (alpha != 1.0f || beta != 0.0f) return bq::BQ_STATUS_UNSUPPORTED;
    } else if (!scale_a || !scale_b) {
        return bq::BQ_STATUS_INVALID_PROBLEM;
    }
    bq::GemvDesc g;
    g.raw_out = raw;
    g.m = m;
    g.n = n;
    g.k = k;
    g.batch = batch;
    g.layout = layout;
    g.alpha = alpha;
    g.beta = beta;
    g.a = static_cast<const int8_t*>(a);
    g.lda = lda;
    g.stride_a = stride_a;
    g.b = static_cast<const int8_t*>(b);
    g.ldb = ldb;
    g.stride_b = stride_b;
    g.scale_a = static_cast<const float*>(scale_a);
    g.stride_scale_a = stride_scale_a;
    g.scale_b = static_cast<const float*>(scale_b);
    g.stride_scale_b = stride_scale_b;
    g.d = d;
    g.ldd = ldd;
    g.stride_d = stride_d;
    g.workspace = workspace;
    g.workspace_bytes = workspace_bytes;
    g.variant = t_tuning.gemv_variant;
    g.pdl = pdl;
    return bq::launch_gemv_q8(g, static_cast<cudaStream_t>(stream));
}

}  // namespace

int32_t bq::launch_gemm_bf16_checked(int32_t layout, int32_t kind, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                                    const void* b, int64_t ldb, void* d, int64_t ldd, const void* scale_a,
                                    const void* scale_b, int32_t scale_mode, float alpha, void* const* peer_d,
                                    int32_t world, int32_t rank, int64_t peer_ld, cudaStream_t stream, void* mc_d) {
    if (layout != bq::BQ_LAYOUT_RCR && layout != bq::BQ_LAYOUT_RRR) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (!peer_d) {
        return gemm_run(layout, kind, 0, m, n, k, a, lda, b, ldb, nullptr, 0, d, ldd, scale_a, scale_b, scale_mode, alpha,
                        0.0f, stream);
    }
    const int32_t st = gemm_validate(layout, m, n, k, a, lda, b, ldb, nullptr, 0, d, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if (!d || (k > 0 && (!a || !b)) || !scale_a || !scale_b) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (scale_mode != BARACUDA_Q_SCALE_PER_TENSOR && scale_mode != BARACUDA_Q_SCALE_PER_ROW_COL)
        return bq::BQ_STATUS_INVALID_PROBLEM;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (k == 0 || (kind == bq::BQ_KIND_S8 && int8_k_status(k) != bq::BQ_STATUS_OK)) return bq::BQ_STATUS_UNSUPPORTED;
    bq::GemmDesc g = {};
    g.b_layout = layout;
    g.kind = kind;
    g.raw_out = 0;
    g.m = m;
    g.n = n;
    g.k = k;
    g.a = a;
    g.lda = lda;
    g.b = b;
    g.ldb = ldb;
    g.scale_a = static_cast<const float*>(scale_a);
    g.scale_b = static_cast<const float*>(scale_b);
    g.scale_mode = scale_mode;
    g.alpha = alpha;
    g.d = d;
    g.ldd = ldd;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    g.direct_stores = t_tuning.direct_stores;
    g.epilogue_warps = t_tuning.epilogue_warps;
    g.q8_out = 0;
    g.c = nullptr;
    g.ldc = 0;
    g.beta = 0.0f;
    g.n_peers = world;
    g.peer_ld = peer_ld;
    g.peer_col0 = rank * n;
    g.peer_rank = rank;
    for (int r = 0; r < 8; ++r) g.peer_d[r] = r < world ? peer_d[r] : nullptr;
    g.mc_d = mc_d;
    return bq::launch_gemm_q8(g, stream);
}

int32_t bq::launch_gemm_raw_reduce_scatter_checked(int32_t kind, int32_t m, int32_t n, int32_t k, const void* a,
                                                   int64_t lda, const void* b, int64_t ldb, void* const* staging,
                                                   int32_t world, int32_t rank, cudaStream_t stream) {
    if (!staging || world < 2 || world > BARACUDA_Q_MAX_PEERS || rank < 0 || rank >= world)
        return bq::BQ_STATUS_INVALID_PROBLEM;
    if (m <= 0 || n <= 0 || k <= 0 || m % world != 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    const int32_t st = gemm_rcr_validate(m, n, k, a, lda, b, ldb, nullptr, 0, staging[rank], n);
    if (st != bq::BQ_STATUS_OK) return st;
    if (!a || !b) return bq::BQ_STATUS_INVALID_PROBLEM;
    // every rank's K slice: the sum over ranks must stay inside 32 bits as well
    if (kind == bq::BQ_KIND_S8 && int8_k_status(k > kMaxInt8K / world ? kMaxInt8K + 1 : k) != bq::BQ_STATUS_OK)
        return bq::BQ_STATUS_UNSUPPORTED;
    for (int r = 0; r < world; ++r) {
        if (!staging[r]) return bq::BQ_STATUS_INVALID_PROBLEM;
        if (!aligned16(staging[r])) return bq::BQ_STATUS_MISALIGNED;
    }
    bq::GemmDesc g = {};
    g.b_layout = bq::BQ_LAYOUT_RCR;
    g.kind = kind;
    g.raw_out = 1;
    g.m = m;
    g.n = n;
    g.k = k;
    g.a = a;
    g.lda = lda;
    g.b = b;
    g.ldb = ldb;
    g.alpha = 1.0f;
    g.d = staging[rank];  // alignment probe only: every row is stored through peer_d
    g.ldd = n;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    g.direct_stores = 1;
    g.epilogue_warps = t_tuning.epilogue_warps;
    g.peer_rank = rank;
    g.rs_world = world;
    g.rs_rows = m / world;
    for (int r = 0; r < 8; ++r) g.peer_d[r] = r < world ? staging[r] : nullptr;
    return bq::launch_gemm_q8(g, stream);
}

extern "C" {

// ---- W8A8 -> bf16 ------------------------------------------------------------
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_rcr_run(bq::BQ_KIND_S8, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b,
                        BARACUDA_Q_SCALE_PER_ROW_COL, alpha, beta, stream);
}
size_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    const int32_t st = gemm_rcr_bf16_validate(m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
    return st != bq::BQ_STATUS_OK ? st : int8_k_status(k);
}

// ---- gated-MLP up-projection: silu(gate) * up -> bf16 ---------------------------------------
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run(
    int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b_gate_up, int64_t ldb, void* d,
    int64_t ldd, const void* scale_a, const void* scale_b, const void* bias, float alpha, void* workspace,
    size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_swiglu_run(bq::BQ_KIND_S8, m, n2, k, a, lda, b_gate_up, ldb, d, ldd, scale_a, scale_b,
                           BARACUDA_Q_SCALE_PER_ROW_COL, bias, alpha, stream);
}
size_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement(
    int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b_gate_up, int64_t ldb, const void* d,
    int64_t ldd) {
    return gemm_swiglu_validate(m, n2, k, a, lda, b_gate_up, ldb, d, ldd);
}
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_run(
    int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b_gate_up, int64_t ldb, void* d,
    int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode, const void* bias, float alpha,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_swiglu_run(bq::BQ_KIND_E4M3, m, n2, k, a, lda, b_gate_up, ldb, d, ldd, scale_a, scale_b, scale_mode, bias,
                           alpha, stream);
}
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_can_implement(
    int32_t m, int32_t n2, int32_t k, const void* a, int64_t lda, const void* b_gate_up, int64_t ldb, const void* d,
    int64_t ldd) {
    return gemm_swiglu_validate(m, n2, k, a, lda, b_gate_up, ldb, d, ldd);
}
int32_t baracuda_kernels_q_interleave_gate_up_run(int64_t f_rows, int64_t row_bytes, const void* gate, int64_t gate_pitch,
                                                  const void* up, int64_t up_pitch, void* out, int64_t out_pitch,
                                                  void* stream) {
    if (f_rows < 0 || row_bytes < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (f_rows == 0 || row_bytes == 0) return bq::BQ_STATUS_OK;
    if (!gate || !up || !out) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (f_rows % 32 != 0) return bq::BQ_STATUS_UNSUPPORTED;
    if (gate_pitch < row_bytes || up_pitch < row_bytes || out_pitch < row_bytes) return bq::BQ_STATUS_INVALID_PROBLEM;
    return bq::launch_interleave_gate_up(f_rows, row_bytes, gate, gate_pitch, up, up_pitch, out, out_pitch,
                                         static_cast<cudaStream_t>(stream));
}

// ---- W8A8 with one per-tensor activation scale passed by value (SmoothQuant inference) -------------------
int32_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_can_implement(int32_t m, int32_t n, int32_t k, const void* act_q,
                                                                           int64_t lda, const void* weight_q, int64_t ldb,
                                                                           const void* output, int64_t ldd) {
    const int32_t st = gemm_rcr_bf16_validate(m, n, k, act_q, lda, weight_q, ldb, nullptr, 0, output, ldd);
    return st != bq::BQ_STATUS_OK ? st : int8_k_status(k);
}
size_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* act_q, int64_t lda, const void* weight_q, int64_t ldb, float act_scale,
    const void* weight_scale, void* output, int64_t ldd, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    const int32_t st = gemm_rcr_bf16_validate(m, n, k, act_q, lda, weight_q, ldb, nullptr, 0, output, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (int8_k_status(k) != bq::BQ_STATUS_OK) return bq::BQ_STATUS_UNSUPPORTED;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if (!output || (k > 0 && (!act_q || !weight_q)) || !weight_scale) return bq::BQ_STATUS_INVALID_PROBLEM;
    bq::GemmDesc g = {};
    g.b_layout = bq::BQ_LAYOUT_RCR;
    g.kind = bq::BQ_KIND_S8;
    g.m = m;
    g.n = n;
    g.k = k;
    g.a = act_q;
    g.lda = lda;
    g.b = weight_q;
    g.ldb = ldb;
    g.scale_a = nullptr;
    g.sa_const = act_scale;
    g.scale_b = static_cast<const float*>(weight_scale);
    g.scale_mode = 2;
    g.alpha = 1.0f;
    g.d = output;
    g.ldd = ldd;
    g.force_block_n = t_tuning.force_block_n;
    g.force_pair_tile_n = t_tuning.force_pair_tile_n;
    g.direct_stores = t_tuning.direct_stores;
    g.epilogue_warps = t_tuning.epilogue_warps;
    g.cluster_split_k = t_tuning.cluster_split_k;
    return bq::launch_gemm_q8(g, static_cast<cudaStream_t>(stream));
}

// ---- s8 -> s32 accumulators --------------------------------------------------
int32_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_rcr_run(bq::BQ_KIND_S8, 1, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, nullptr, nullptr, 0, alpha,
                        beta, stream);
}
size_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    const int32_t st = gemm_rcr_validate(m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
    return st != bq::BQ_STATUS_OK ? st : int8_k_status(k);
}

// ---- e4m3 -> bf16 --------------------------------------------------------------
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode, float alpha,
    float beta, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_rcr_run(bq::BQ_KIND_E4M3, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b, scale_mode,
                        alpha, beta, stream);
}
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    return gemm_rcr_bf16_validate(m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
}

// ---- e4m3 -> f32 accumulators ---------------------------------------------------
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_rcr_run(bq::BQ_KIND_E4M3, 1, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, nullptr, nullptr, 0, alpha,
                        beta, stream);
}
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    return gemm_rcr_validate(m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
}

// ---- the reference's own 8-bit-out contracts ------------------------------------------------
int32_t baracuda_kernels_gemm_s8_rcr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_q8_run(bq::BQ_LAYOUT_RCR, bq::BQ_KIND_S8, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream);
}
size_t baracuda_kernels_gemm_s8_rcr_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_s8_rcr_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    const int32_t st = gemm_q8_validate(bq::BQ_LAYOUT_RCR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
    return st != bq::BQ_STATUS_OK ? st : int8_k_status(k);
}
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_q8_run(bq::BQ_LAYOUT_RCR, bq::BQ_KIND_E4M3, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream);
}
size_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_workspace_size(int32_t, int32_t, int32_t) { return 0; }
int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, const void* d, int64_t ldd) {
    return gemm_q8_validate(bq::BQ_LAYOUT_RCR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);
}

// ---- row-major weights ("rrr": B is [K,N] with ldb >= n), the layout of the reference's bespoke GEMMs ------
#define BQ_GEMM_TRIPLE_TAIL(NAME, VALIDATE)                                                                          \
    size_t NAME##_workspace_size(int32_t, int32_t, int32_t) { return 0; }                                           \
    int32_t NAME##_can_implement(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b,         \
                                 int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd) {              \
        return VALIDATE(bq::BQ_LAYOUT_RRR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);                                  \
    }

#define BQ_GEMM_TRIPLE_TAIL_S8(NAME, VALIDATE)                                                                       \
    size_t NAME##_workspace_size(int32_t, int32_t, int32_t) { return 0; }                                           \
    int32_t NAME##_can_implement(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b,         \
                                 int64_t ldb, const void* c, int64_t ldc, const void* d, int64_t ldd) {              \
        const int32_t st = VALIDATE(bq::BQ_LAYOUT_RRR, m, n, k, a, lda, b, ldb, c, ldc, d, ldd);                     \
        return st != bq::BQ_STATUS_OK ? st : int8_k_status(k);                                                       \
    }

int32_t baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, float alpha, float beta,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b,
                    BARACUDA_Q_SCALE_PER_ROW_COL, alpha, beta, stream);
}
BQ_GEMM_TRIPLE_TAIL_S8(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a, gemm_bf16_validate)

int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode, float alpha,
    float beta, void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b,
                    scale_mode, alpha, beta, stream);
}
BQ_GEMM_TRIPLE_TAIL(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a, gemm_bf16_validate)

int32_t baracuda_kernels_gemm_s8_rrr_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, 1, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, nullptr, nullptr, 0, alpha,
                    beta, stream);
}
BQ_GEMM_TRIPLE_TAIL_S8(baracuda_kernels_gemm_s8_rrr_s32_sm100a, gemm_validate)

int32_t baracuda_kernels_gemm_s8_rrr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_q8_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream);
}
BQ_GEMM_TRIPLE_TAIL_S8(baracuda_kernels_gemm_s8_rrr_sm100a, gemm_q8_validate)

int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_run(
    int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,
    int64_t ldc, void* d, int64_t ldd, float alpha, float beta, void* workspace, size_t workspace_bytes,
    void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemm_q8_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream);
}
BQ_GEMM_TRIPLE_TAIL(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a, gemm_q8_validate)

// ---- fused bias / activation epilogues -----------------------------------------------------------
#define BQ_Q8_EPILOGUE_RUN(NAME, LAYOUT, KIND)                                                                           \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,   \
                 int64_t ldc, void* d, int64_t ldd, const void* bias, int32_t bias_kind, int32_t epilogue, float alpha,    \
                 float beta, void* workspace, size_t workspace_bytes, void* stream) {                                      \
        (void)workspace;                                                                                                   \
        (void)workspace_bytes;                                                                                             \
        Epilogue e;                                                                                                        \
        e.bias = bias;                                                                                                     \
        e.bias_kind = bias_kind;                                                                                           \
        e.kind = epilogue;                                                                                                 \
        return gemm_q8_run(LAYOUT, KIND, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream, e);                 \
    }
BQ_Q8_EPILOGUE_RUN(baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_S8)
BQ_Q8_EPILOGUE_RUN(baracuda_kernels_gemm_s8_rrr_sm100a_epilogue_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8)
BQ_Q8_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_epilogue_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_E4M3)
BQ_Q8_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_epilogue_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3)

// the reference's named variants: ..._bias[_relu|_gelu|_silu]_{f32,i32}_run (s8) and ..._bias[_act]_run (e4m3)
#define BQ_Q8_NAMED_BIAS_RUN(NAME, LAYOUT, KIND, BIAS_KIND, EPI)                                                          \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,   \
                 int64_t ldc, void* d, int64_t ldd, const void* bias, float alpha, float beta, void* workspace,            \
                 size_t workspace_bytes, void* stream) {                                                                   \
        (void)workspace;                                                                                                   \
        (void)workspace_bytes;                                                                                             \
        Epilogue e;                                                                                                        \
        e.bias = bias;                                                                                                     \
        e.bias_kind = BIAS_KIND;                                                                                           \
        e.kind = EPI;                                                                                                      \
        return gemm_q8_run(LAYOUT, KIND, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta, stream, e);                 \
    }
#define BQ_S8_BIAS_FAMILY(LAY, LAYOUT)                                                                                     \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_f32_run, LAYOUT, bq::BQ_KIND_S8, 1, 1)              \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_relu_f32_run, LAYOUT, bq::BQ_KIND_S8, 1, 2)         \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_gelu_f32_run, LAYOUT, bq::BQ_KIND_S8, 1, 3)         \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_silu_f32_run, LAYOUT, bq::BQ_KIND_S8, 1, 4)         \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_i32_run, LAYOUT, bq::BQ_KIND_S8, 2, 1)              \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_relu_i32_run, LAYOUT, bq::BQ_KIND_S8, 2, 2)         \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_gelu_i32_run, LAYOUT, bq::BQ_KIND_S8, 2, 3)         \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_s8_##LAY##_sm100a_bias_silu_i32_run, LAYOUT, bq::BQ_KIND_S8, 2, 4)
BQ_S8_BIAS_FAMILY(rcr, bq::BQ_LAYOUT_RCR)
BQ_S8_BIAS_FAMILY(rrr, bq::BQ_LAYOUT_RRR)
#define BQ_FP8_BIAS_FAMILY(LAY, LAYOUT)                                                                                    \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_##LAY##_sm100a_bias_run, LAYOUT, bq::BQ_KIND_E4M3, 1, 1)          \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_##LAY##_sm100a_bias_relu_run, LAYOUT, bq::BQ_KIND_E4M3, 1, 2)     \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_##LAY##_sm100a_bias_gelu_run, LAYOUT, bq::BQ_KIND_E4M3, 1, 3)     \
    BQ_Q8_NAMED_BIAS_RUN(baracuda_kernels_gemm_fp8_e4m3_##LAY##_sm100a_bias_silu_run, LAYOUT, bq::BQ_KIND_E4M3, 1, 4)
BQ_FP8_BIAS_FAMILY(rcr, bq::BQ_LAYOUT_RCR)
BQ_FP8_BIAS_FAMILY(rrr, bq::BQ_LAYOUT_RRR)

// bf16-out SKUs with the fused chain: D = bf16( act( alpha * ((sa*sb) * acc) + bias[j] ) ), bias float[N]
#define BQ_BF16_EPILOGUE_RUN(NAME, LAYOUT, KIND, HAS_MODE)                                                                 \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,   \
                 int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode,          \
                 const void* bias, int32_t epilogue, float alpha, float beta, void* workspace, size_t workspace_bytes,     \
                 void* stream) {                                                                                           \
        (void)workspace;                                                                                                   \
        (void)workspace_bytes;                                                                                             \
        Epilogue e;                                                                                                        \
        e.bias = bias;                                                                                                     \
        e.bias_kind = 1;                                                                                                   \
        e.kind = epilogue;                                                                                                 \
        return gemm_run(LAYOUT, KIND, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b,                        \
                        HAS_MODE ? scale_mode : BARACUDA_Q_SCALE_PER_ROW_COL, alpha, beta, stream, e);                     \
    }
BQ_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_S8, false)
BQ_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_epilogue_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, false)
BQ_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_epilogue_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_E4M3, true)
BQ_BF16_EPILOGUE_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_epilogue_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3, true)

// ---- the bf16-out GEMMs as programmatic dependent launches (per call) ------------------------------------
#define BQ_BF16_PDL_RUN(NAME, LAYOUT, KIND, HAS_MODE)                                                                      \
    int32_t NAME(int32_t m, int32_t n, int32_t k, const void* a, int64_t lda, const void* b, int64_t ldb, const void* c,   \
                 int64_t ldc, void* d, int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode,          \
                 const void* bias, int32_t epilogue, float alpha, float beta, void* workspace, size_t workspace_bytes,     \
                 void* stream) {                                                                                           \
        (void)workspace;                                                                                                   \
        (void)workspace_bytes;                                                                                             \
        Epilogue e;                                                                                                        \
        e.bias = bias;                                                                                                     \
        e.bias_kind = 1;                                                                                                   \
        e.kind = epilogue;                                                                                                 \
        return gemm_run(LAYOUT, KIND, 0, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, scale_a, scale_b,                        \
                        HAS_MODE ? scale_mode : BARACUDA_Q_SCALE_PER_ROW_COL, alpha, beta, stream, e, 1);                  \
    }
BQ_BF16_PDL_RUN(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_pdl_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_S8, false)
BQ_BF16_PDL_RUN(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_pdl_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, false)
BQ_BF16_PDL_RUN(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_pdl_run, bq::BQ_LAYOUT_RCR, bq::BQ_KIND_E4M3, true)
BQ_BF16_PDL_RUN(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_pdl_run, bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3, true)

// ---- int8 GEMV ---------------------------------------------------------------------
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha, float beta, const void* a,
    int64_t lda, int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, const void* scale_a,
    int64_t stride_scale_a, const void* scale_b, int64_t stride_scale_b, void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream) {
    return gemv_run(0, m, n, k, batch, layout, alpha, beta, a, lda, stride_a, b, ldb, stride_b, scale_a,
                    stride_scale_a, scale_b, stride_scale_b, d, ldd, stride_d, workspace, workspace_bytes, stream);
}
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha, float beta, const void* a,
    int64_t lda, int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, const void* scale_a,
    int64_t stride_scale_a, const void* scale_b, int64_t stride_scale_b, void* d, int64_t ldd, int64_t stride_d,
    void* workspace, size_t workspace_bytes, void* stream) {
    return gemv_run(0, m, n, k, batch, layout, alpha, beta, a, lda, stride_a, b, ldb, stride_b, scale_a,
                    stride_scale_a, scale_b, stride_scale_b, d, ldd, stride_d, workspace, workspace_bytes, stream, 1);
}
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, int64_t lda, int64_t ldb, int64_t ldd,
    int64_t stride_a, int64_t stride_b, int64_t stride_d) {
    (void)stride_a;
    (void)stride_b;
    return gemv_validate(m, n, k, batch, layout, lda, ldb, ldd, stride_d);
}
size_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(int32_t m, int32_t n, int32_t k, int32_t batch,
                                                              int32_t layout) {
    return bq::gemv_q8_workspace_bytes(m, n, k, batch, layout);
}

int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha, float beta, const void* a,
    int64_t lda, int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, void* d, int64_t ldd,
    int64_t stride_d, void* workspace, size_t workspace_bytes, void* stream) {
    return gemv_run(1, m, n, k, batch, layout, alpha, beta, a, lda, stride_a, b, ldb, stride_b, nullptr, 0, nullptr,
                    0, d, ldd, stride_d, workspace, workspace_bytes, stream);
}
int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, float alpha, float beta, const void* a,
    int64_t lda, int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, void* d, int64_t ldd,
    int64_t stride_d, void* workspace, size_t workspace_bytes, void* stream) {
    return gemv_run(1, m, n, k, batch, layout, alpha, beta, a, lda, stride_a, b, ldb, stride_b, nullptr, 0, nullptr,
                    0, d, ldd, stride_d, workspace, workspace_bytes, stream, 1);
}
int32_t baracuda_kernels_gemv_q8_m1_s32_sm100a_can_implement(
    int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout, int64_t lda, int64_t ldb, int64_t ldd,
    int64_t stride_a, int64_t stride_b, int64_t stride_d) {
    (void)stride_a;
    (void)stride_b;
    return gemv_validate(m, n, k, batch, layout, lda, ldb, ldd, stride_d);
}
size_t baracuda_kernels_gemv_q8_m1_s32_sm100a_workspace_size(int32_t m, int32_t n, int32_t k, int32_t batch,
                                                             int32_t layout) {
    return bq::gemv_q8_workspace_bytes(m, n, k, batch, layout);
}

// ---- decode GEMV with the per-token quantiser inside --------------------------------------------
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(int32_t m, int32_t n, int32_t k, int64_t ldx,
                                                                         int64_t ldb, int64_t ldd) {
    if (m < 0 || n < 0 || k < 0) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (m > 8) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (ldx < (k > 0 ? k : 1) || ldb < (k > 0 ? k : 1) || ldd < (n > 0 ? n : 1)) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if ((ldx & 7) || (ldb & 15)) return bq::BQ_STATUS_UNSUPPORTED;  // 16-byte rows for the vector loads and bulk copies
    return bq::gemv_q8_quant_bf16_supported(m, n, k) ? bq::BQ_STATUS_OK : bq::BQ_STATUS_UNSUPPORTED;
}

namespace {
int32_t gemv_quant_bf16_run(int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax, float alpha, float beta,
                            const void* x_bf16, int64_t ldx, const void* b, int64_t ldb, const void* scale_b,
                            void* scale_a_out, void* d, int64_t ldd, int32_t pdl, void* stream) {
    const int32_t st = baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(m, n, k, ldx, ldb, ldd);
    if (st != bq::BQ_STATUS_OK) return st;
    if (m == 0 || n == 0) return bq::BQ_STATUS_OK;
    if (!x_bf16 || !b || !scale_b || !d) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (qmin > qmax || qmax <= 0 || qmin < -128 || qmax > 127) return bq::BQ_STATUS_INVALID_PROBLEM;
    if (!aligned16(x_bf16) || !aligned16(b)) return bq::BQ_STATUS_UNSUPPORTED;
    return bq::launch_gemv_q8_quant_bf16(m, n, k, qmin, qmax, alpha, beta, x_bf16, ldx, static_cast<const int8_t*>(b), ldb,
                                         static_cast<const float*>(scale_b), static_cast<float*>(scale_a_out), d, ldd, pdl,
                                         static_cast<cudaStream_t>(stream));
}
}  // namespace

int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run(
    int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax, float alpha, float beta, const void* x_bf16,
    int64_t ldx, const void* b, int64_t ldb, const void* scale_b, void* scale_a_out, void* d, int64_t ldd,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemv_quant_bf16_run(m, n, k, qmin, qmax, alpha, beta, x_bf16, ldx, b, ldb, scale_b, scale_a_out, d, ldd, 0,
                               stream);
}
int32_t baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_pdl_run(
    int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax, float alpha, float beta, const void* x_bf16,
    int64_t ldx, const void* b, int64_t ldb, const void* scale_b, void* scale_a_out, void* d, int64_t ldd,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return gemv_quant_bf16_run(m, n, k, qmin, qmax, alpha, beta, x_bf16, ldx, b, ldb, scale_b, scale_a_out, d, ldd, 1,
                               stream);
}

// ---- diagnostics / tuning -------------------------------------------------------------
int32_t baracuda_kernels_q_device_status(void) {
    int32_t gemm = bq::read_and_clear_gemm_device_status();
    const int32_t pair = bq::read_and_clear_gemm_pair_device_status();
    if (gemm == 0) gemm = pair;
    const int32_t splitk = bq::read_and_clear_gemm_splitk_device_status();
    if (gemm == 0) gemm = splitk;
    int32_t gemv = bq::read_and_clear_gemv_device_status();
    const int32_t barrier = bq::read_and_clear_peer_barrier_device_status();
    if (gemv == 0) gemv = barrier;
    return gemm != 0 ? gemm : gemv;
}

int32_t baracuda_kernels_q_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
    return bq::launch_bounded_wait_selftest(static_cast<long long>(limit_cycles), static_cast<cudaStream_t>(stream));
}

int32_t baracuda_kernels_q_set_tuning(int32_t key, int32_t value) {
    switch (key) {
        case 0:
            if (value != 0 && value != 64 && value != 128 && value != 256 && value != 512) return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.force_block_n = value;
            return bq::BQ_STATUS_OK;
        case 1:
            if (value != 0 && value != 1 && value != 2 && value != 3 && value != 8 && value != 9)
                return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.gemv_variant = value;
            return bq::BQ_STATUS_OK;
        case 4:
            if (value < 0 || value > 2) return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.direct_stores = value;
            return bq::BQ_STATUS_OK;
        case 5:
            if (value != 0 && value != 4 && value != 8) return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.epilogue_warps = value;
            return bq::BQ_STATUS_OK;
        case 6:
            if (value != 0 && value != 1 && value != 2 && value != 4 && value != 256) return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.cluster_split_k = value;
            return bq::BQ_STATUS_OK;
        case 2:
            if (value != 0 && value != 2 && value != 256 && value != 224 && value != 192 && value != 128)
                return bq::BQ_STATUS_INVALID_PROBLEM;
            t_tuning.force_pair_tile_n = value;
            return bq::BQ_STATUS_OK;
        default:
            return bq::BQ_STATUS_INVALID_PROBLEM;
    }
}

}  // extern "C"
