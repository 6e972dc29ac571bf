// Typed Plan layer over the flat C ABI, in C++17 — the compiled-language twin
// of the reference's safe Rust facade (`<Op>Descriptor` / `<Op>Args` /
// `<Op>Plan::{select, can_implement, workspace_size, run, sku,
// precision_guarantee}`; crates/baracuda-kernels/src/gemm/int_gemm.rs:48-637,
// fp8_gemm.rs:36-741, gemv_dense.rs:48-412; vocabulary from
// crates/baracuda-kernel-vocab/src/{layout,sku,plan}.rs).
//
// Header-only; link against libbaracuda_kernels_q.so.  Plans are plain data
// (descriptor + SKU), `Copy`-like, usable from any thread; `run` launches on
// the caller's stream and returns a typed error instead of throwing.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <limits>
#include <optional>

#include "baracuda_kernels_q.h"

namespace baracuda {

enum class LayoutSku : uint8_t { Rcr, Rrr };                      // layout.rs:17-34
enum class ArchSku : uint8_t { Sm80, Sm89, Sm90a, Sm100a };       // layout.rs:43-53 (+ Sm100a)
enum class EpilogueKind : uint8_t { Identity, Bias, BiasRelu, BiasGelu, BiasSilu };  // layout.rs:69-96
enum class BackendKind : uint8_t { Bespoke, Cutlass, Cublas };    // sku.rs:123-204 (subset)
enum class OpCategory : uint8_t { Gemm, Quantization };
enum class ElementKind : uint8_t { S8, Fp8E4M3, Bf16, F32, I32 };
enum class MathPrecision : uint8_t { Int8, Fp8E4M3 };
enum class ScaleMode : int32_t { PerTensor = 0, PerRowCol = 1 };

inline bool requires_bias(EpilogueKind e) { return e != EpilogueKind::Identity; }

// crates/baracuda-cutlass/src/error.rs:23-70
enum class Error : uint8_t {
    Ok,
    Unsupported,
    InvalidProblem,
    MisalignedOperand,
    WorkspaceTooSmall,
    BufferTooSmall,
    LaunchFailure,
};

// status -> Error (error.rs:83-93, int_gemm.rs:640-653)
inline Error status_to_error(int32_t st) {
    switch (st) {
        case 0: return Error::Ok;
        case 1: return Error::MisalignedOperand;
        case 2: return Error::InvalidProblem;
        case 3: return Error::Unsupported;
        case 4: return Error::WorkspaceTooSmall;
        default: return Error::LaunchFailure;
    }
}

struct PrecisionGuarantee {  // plan.rs:68-86
    MathPrecision math_precision;
    ElementKind accumulator;
    bool bit_stable_on_same_hardware;
    bool deterministic;
    bool operator==(const PrecisionGuarantee& o) const {
        return math_precision == o.math_precision && accumulator == o.accumulator &&
               bit_stable_on_same_hardware == o.bit_stable_on_same_hardware && deterministic == o.deterministic;
    }
};

struct PlanPreference {  // plan.rs:19-57
    size_t max_workspace_bytes = std::numeric_limits<size_t>::max();
    bool allow_sm90a = true;
    std::optional<BackendKind> prefer_backend = std::nullopt;
};

struct KernelSku {  // sku.rs:259-285
    OpCategory category;
    uint16_t op;
    ElementKind element;
    std::optional<ElementKind> aux_element;
    std::optional<LayoutSku> layout;
    std::optional<EpilogueKind> epilogue;
    ArchSku arch;
    BackendKind backend;
    PrecisionGuarantee precision_guarantee;
    bool operator==(const KernelSku& o) const {
        return category == o.category && op == o.op && element == o.element && aux_element == o.aux_element &&
               layout == o.layout && epilogue == o.epilogue && arch == o.arch && backend == o.backend &&
               precision_guarantee == o.precision_guarantee;
    }
    size_t hash() const {
        size_t h = static_cast<size_t>(category) * 1315423911u + op;
        h = h * 31 + static_cast<size_t>(element);
        h = h * 31 + (aux_element ? 1 + static_cast<size_t>(*aux_element) : 0);
        h = h * 31 + (layout ? 1 + static_cast<size_t>(*layout) : 0);
        h = h * 31 + (epilogue ? 1 + static_cast<size_t>(*epilogue) : 0);
        h = h * 31 + static_cast<size_t>(arch);
        return h * 31 + static_cast<size_t>(backend);
    }
};

constexpr uint16_t OP_W8A8_GEMM = 100;
constexpr uint16_t OP_FP8_SCALED_GEMM = 101;
constexpr uint16_t OP_GEMV_Q8 = 102;
constexpr uint16_t OP_GATED_MLP_UP = 103;

// A device view with its length in elements, so the typed layer can refuse a
// launch that would run off a buffer (the soundness boundary of
// gemv_dense.rs:218-268).
template <typename T>
struct DeviceSpan {
    T* ptr = nullptr;
    size_t len = 0;
};

struct Workspace {  // crates/baracuda-kernels-types/src/plan.rs:26-32
    void* ptr = nullptr;
    size_t bytes = 0;
    static Workspace none() { return {}; }
};

namespace detail {
inline size_t span_elems(int64_t rows, int64_t cols, int64_t ld) {
    return (rows == 0 || cols == 0) ? 0 : static_cast<size_t>((rows - 1) * ld + cols);
}
inline bool backend_ok(const PlanPreference& p) {
    return !p.prefer_backend || *p.prefer_backend == BackendKind::Bespoke;
}
}  // namespace detail

// ---------------------------------------------------------------------------- GEMM
struct QGemmDescriptor {  // IntGemmDescriptor, crates/baracuda-cutlass/src/types.rs:187-198
    int32_t m = 0, n = 0, k = 0;
    LayoutSku layout = LayoutSku::Rcr;
    EpilogueKind epilogue = EpilogueKind::Identity;
};

struct QGemmArgs {
    DeviceSpan<const void> a;   // [M,K] bytes, row pitch lda
    int64_t lda = 0;
    DeviceSpan<const void> b;   // weight stored [N,K] bytes, row pitch ldb
    int64_t ldb = 0;
    DeviceSpan<void> d;         // [M,N] elements of the plan's output type, row pitch ldd
    int64_t ldd = 0;
    DeviceSpan<const float> scale_a;
    DeviceSpan<const float> scale_b;
    float alpha = 1.0f;
    float beta = 0.0f;
    DeviceSpan<const float> bias;  // [N], read when the descriptor's epilogue has a bias
    DeviceSpan<const void> c;      // bf16 [M,N] with row pitch ldc, read when beta != 0 (may be d); bf16-out plans only
    int64_t ldc = 0;
};

class W8A8GemmPlan {
  public:
    // Validates once and fixes the SKU.  `raw_accumulators` selects the int32-out symbol.
    static Error select(const QGemmDescriptor& desc, const PlanPreference& pref, bool raw_accumulators,
                        W8A8GemmPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.n < 0 || desc.k < 0) return Error::InvalidProblem;
        if (raw_accumulators && desc.epilogue != EpilogueKind::Identity) return Error::Unsupported;
        out->desc_ = desc;
        out->raw_ = raw_accumulators;
        out->sku_ = KernelSku{OpCategory::Gemm, OP_W8A8_GEMM, ElementKind::S8,
                              raw_accumulators ? ElementKind::I32 : ElementKind::Bf16, desc.layout, desc.epilogue,
                              ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{MathPrecision::Int8, ElementKind::I32, true, true}};
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    const QGemmDescriptor& descriptor() const { return desc_; }
    size_t workspace_size() const {
        return raw_ ? baracuda_kernels_gemm_s8_rcr_s32_sm100a_workspace_size(desc_.m, desc_.n, desc_.k)
                    : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_workspace_size(desc_.m, desc_.n, desc_.k);
    }
    Error can_implement(const QGemmArgs& x) const {
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        auto can = rrr ? (raw_ ? baracuda_kernels_gemm_s8_rrr_s32_sm100a_can_implement
                               : baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_can_implement)
                       : (raw_ ? baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement
                               : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement);
        const int32_t st = can(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd);
        if (st != 0) return status_to_error(st);
        if (desc_.m == 0 || desc_.n == 0) return Error::Ok;  // empty problem: nothing is read or written
        if (x.a.len < detail::span_elems(desc_.m, desc_.k, x.lda)) return Error::BufferTooSmall;
        if (x.b.len < (rrr ? detail::span_elems(desc_.k, desc_.n, x.ldb) : detail::span_elems(desc_.n, desc_.k, x.ldb)))
            return Error::BufferTooSmall;
        if (x.d.len < detail::span_elems(desc_.m, desc_.n, x.ldd)) return Error::BufferTooSmall;
        if (x.c.ptr && x.c.len < detail::span_elems(desc_.m, desc_.n, x.ldc)) return Error::BufferTooSmall;
        if (!raw_) {
            if (!x.scale_a.ptr || !x.scale_b.ptr) return Error::InvalidProblem;
            if (x.scale_a.len < static_cast<size_t>(desc_.m) || x.scale_b.len < static_cast<size_t>(desc_.n))
                return Error::BufferTooSmall;
        }
        if (requires_bias(desc_.epilogue)) {
            if (!x.bias.ptr) return Error::InvalidProblem;
            if (x.bias.len < static_cast<size_t>(desc_.n)) return Error::BufferTooSmall;
        }
        return Error::Ok;
    }
    Error run(void* stream, Workspace ws, const QGemmArgs& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        int32_t st;
        if (raw_) {
            auto run = rrr ? baracuda_kernels_gemm_s8_rrr_s32_sm100a_run : baracuda_kernels_gemm_s8_rcr_s32_sm100a_run;
            st = run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, nullptr, 0, x.d.ptr, x.ldd, x.alpha, x.beta,
                     ws.ptr, ws.bytes, stream);
        } else if (desc_.epilogue != EpilogueKind::Identity) {
            auto run = rrr ? baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_epilogue_run
                           : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run;
            st = run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd, x.scale_a.ptr,
                     x.scale_b.ptr, BARACUDA_Q_SCALE_PER_ROW_COL, x.bias.ptr, static_cast<int32_t>(desc_.epilogue), x.alpha,
                     x.beta, ws.ptr, ws.bytes, stream);
        } else {
            auto run = rrr ? baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run;
            st = run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd, x.scale_a.ptr,
                     x.scale_b.ptr, x.alpha, x.beta, ws.ptr, ws.bytes, stream);
        }
        return status_to_error(st);
    }

    // The same launch as a programmatic dependent of the kernel before it on the stream (bf16-out plans): prologue
    // and the first weight tiles are issued before that kernel has finished.  The caller asserts that it does not
    // write `b`.
    Error run_dependent(void* stream, Workspace ws, const QGemmArgs& x) const {
        if (raw_) return Error::Unsupported;
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        auto run = desc_.layout == LayoutSku::Rrr ? baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_pdl_run
                                                  : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_pdl_run;
        return status_to_error(run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr,
                                   x.ldd, x.scale_a.ptr, x.scale_b.ptr, BARACUDA_Q_SCALE_PER_ROW_COL, x.bias.ptr,
                                   static_cast<int32_t>(desc_.epilogue), x.alpha, x.beta, ws.ptr, ws.bytes, stream));
    }

  private:
    QGemmDescriptor desc_{};
    KernelSku sku_{};
    bool raw_ = false;
};

class Fp8ScaledGemmPlan {
  public:
    static Error select(const QGemmDescriptor& desc, const PlanPreference& pref, ScaleMode mode, bool raw_accumulators,
                        Fp8ScaledGemmPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.n < 0 || desc.k < 0) return Error::InvalidProblem;
        if (raw_accumulators && (desc.layout != LayoutSku::Rcr || desc.epilogue != EpilogueKind::Identity))
            return Error::Unsupported;
        out->desc_ = desc;
        out->raw_ = raw_accumulators;
        out->mode_ = mode;
        out->sku_ = KernelSku{OpCategory::Gemm, OP_FP8_SCALED_GEMM, ElementKind::Fp8E4M3,
                              raw_accumulators ? ElementKind::F32 : ElementKind::Bf16, desc.layout, desc.epilogue,
                              ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{MathPrecision::Fp8E4M3, ElementKind::F32, true, true}};
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    size_t workspace_size() const {
        return baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_workspace_size(desc_.m, desc_.n, desc_.k);
    }
    Error can_implement(const QGemmArgs& x) const {
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        auto can = rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_can_implement
                       : baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement;
        const int32_t st = can(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd);
        if (st != 0) return status_to_error(st);
        if (desc_.m == 0 || desc_.n == 0) return Error::Ok;  // empty problem: nothing is read or written
        if (x.a.len < detail::span_elems(desc_.m, desc_.k, x.lda)) return Error::BufferTooSmall;
        if (x.b.len < (rrr ? detail::span_elems(desc_.k, desc_.n, x.ldb) : detail::span_elems(desc_.n, desc_.k, x.ldb)))
            return Error::BufferTooSmall;
        if (x.d.len < detail::span_elems(desc_.m, desc_.n, x.ldd)) return Error::BufferTooSmall;
        if (x.c.ptr && x.c.len < detail::span_elems(desc_.m, desc_.n, x.ldc)) return Error::BufferTooSmall;
        if (!raw_) {
            if (!x.scale_a.ptr || !x.scale_b.ptr) return Error::InvalidProblem;
            const size_t na = mode_ == ScaleMode::PerRowCol ? static_cast<size_t>(desc_.m) : 1;
            const size_t nb = mode_ == ScaleMode::PerRowCol ? static_cast<size_t>(desc_.n) : 1;
            if (x.scale_a.len < na || x.scale_b.len < nb) return Error::BufferTooSmall;
        }
        if (requires_bias(desc_.epilogue)) {
            if (!x.bias.ptr) return Error::InvalidProblem;
            if (x.bias.len < static_cast<size_t>(desc_.n)) return Error::BufferTooSmall;
        }
        return Error::Ok;
    }
    Error run(void* stream, Workspace ws, const QGemmArgs& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        int32_t st;
        if (raw_) {
            st = baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb,
                                                                   nullptr, 0, x.d.ptr, x.ldd, x.alpha, x.beta, ws.ptr,
                                                                   ws.bytes, stream);
        } else if (desc_.epilogue != EpilogueKind::Identity) {
            auto run = rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_epilogue_run
                           : baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_epilogue_run;
            st = run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd, x.scale_a.ptr,
                     x.scale_b.ptr, static_cast<int32_t>(mode_), x.bias.ptr, static_cast<int32_t>(desc_.epilogue), x.alpha,
                     x.beta, ws.ptr, ws.bytes, stream);
        } else {
            auto run = rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_run
                           : baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_run;
            st = run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd, x.scale_a.ptr,
                     x.scale_b.ptr, static_cast<int32_t>(mode_), x.alpha, x.beta, ws.ptr, ws.bytes, stream);
        }
        return status_to_error(st);
    }

    Error run_dependent(void* stream, Workspace ws, const QGemmArgs& x) const {  // as W8A8GemmPlan::run_dependent
        if (raw_) return Error::Unsupported;
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        auto run = desc_.layout == LayoutSku::Rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_pdl_run
                                                  : baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_pdl_run;
        return status_to_error(run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr,
                                   x.ldd, x.scale_a.ptr, x.scale_b.ptr, static_cast<int32_t>(mode_), x.bias.ptr,
                                   static_cast<int32_t>(desc_.epilogue), x.alpha, x.beta, ws.ptr, ws.bytes, stream));
    }

  private:
    QGemmDescriptor desc_{};
    KernelSku sku_{};
    ScaleMode mode_ = ScaleMode::PerTensor;
    bool raw_ = false;
};

// The reference's own 8-bit-out contract (IntGemmPlan<S8> / Fp8GemmPlan<Fp8E4M3>, every EpilogueKind, Rcr or Rrr):
// D = sat(act(alpha * acc + beta * C + bias)) in the input type.  `c` may be empty when beta == 0; `bias` is N
// elements of `bias_element` (BiasElement of the reference: F32, or I32 for the s8 plan).
struct Q8OutGemmArgs {
    DeviceSpan<const void> a;
    int64_t lda = 0;
    DeviceSpan<const void> b;
    int64_t ldb = 0;
    DeviceSpan<const void> c;
    int64_t ldc = 0;
    DeviceSpan<void> d;
    int64_t ldd = 0;
    float alpha = 1.0f;
    float beta = 0.0f;
    DeviceSpan<const void> bias;
    ElementKind bias_element = ElementKind::F32;
};

class IntGemmPlan {
  public:
    static Error select(const QGemmDescriptor& desc, const PlanPreference& pref, ElementKind element, IntGemmPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.n < 0 || desc.k < 0) return Error::InvalidProblem;
        if (element != ElementKind::S8 && element != ElementKind::Fp8E4M3) return Error::Unsupported;
        const bool fp8 = element == ElementKind::Fp8E4M3;
        out->desc_ = desc;
        out->fp8_ = fp8;
        out->sku_ = KernelSku{OpCategory::Gemm, fp8 ? OP_FP8_SCALED_GEMM : OP_W8A8_GEMM, element, std::nullopt, desc.layout,
                              desc.epilogue, ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{fp8 ? MathPrecision::Fp8E4M3 : MathPrecision::Int8,
                                                 fp8 ? ElementKind::F32 : ElementKind::I32, true, true}};
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    size_t workspace_size() const { return 0; }
    Error run(void* stream, Workspace ws, const Q8OutGemmArgs& x) const {
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        if (desc_.m > 0 && desc_.n > 0) {
            if (x.a.len < detail::span_elems(desc_.m, desc_.k, x.lda)) return Error::BufferTooSmall;
            if (x.b.len < (rrr ? detail::span_elems(desc_.k, desc_.n, x.ldb) : detail::span_elems(desc_.n, desc_.k, x.ldb)))
                return Error::BufferTooSmall;
            if (x.d.len < detail::span_elems(desc_.m, desc_.n, x.ldd)) return Error::BufferTooSmall;
            if (x.beta != 0.0f && x.c.len < detail::span_elems(desc_.m, desc_.n, x.ldc)) return Error::BufferTooSmall;
        }
        if (requires_bias(desc_.epilogue)) {
            const bool i32 = x.bias_element == ElementKind::I32;
            if (!x.bias.ptr || (!i32 && x.bias_element != ElementKind::F32) || (i32 && fp8_)) return Error::InvalidProblem;
            if (x.bias.len < static_cast<size_t>(desc_.n)) return Error::BufferTooSmall;
            auto run = fp8_ ? (rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_epilogue_run
                                   : baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_epilogue_run)
                            : (rrr ? baracuda_kernels_gemm_s8_rrr_sm100a_epilogue_run
                                   : baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run);
            return status_to_error(run(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr,
                                       x.ldd, x.bias.ptr, i32 ? BARACUDA_Q_BIAS_I32 : BARACUDA_Q_BIAS_F32,
                                       static_cast<int32_t>(desc_.epilogue), x.alpha, x.beta, ws.ptr, ws.bytes, stream));
        }
        auto fn = fp8_ ? (rrr ? baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_run : baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run)
                       : (rrr ? baracuda_kernels_gemm_s8_rrr_sm100a_run : baracuda_kernels_gemm_s8_rcr_sm100a_run);
        return status_to_error(fn(desc_.m, desc_.n, desc_.k, x.a.ptr, x.lda, x.b.ptr, x.ldb, x.c.ptr, x.ldc, x.d.ptr, x.ldd,
                                  x.alpha, x.beta, ws.ptr, ws.bytes, stream));
    }

  private:
    QGemmDescriptor desc_{};
    KernelSku sku_{};
    bool fp8_ = false;
};

// Gated-MLP up-projection in one launch: h[M, F] = silu(x Wg^T) * (x Wu^T) from 8-bit operands, the [M, 2F]
// intermediate staying in tensor memory.  The reference's EpilogueKind ends at BiasSilu (layout.rs:69-96); this plan
// has no counterpart there.  `b_gate_up`, `scale_b` and `bias` hold gate and up interleaved in blocks of 32 rows
// (baracuda_kernels_q_interleave_gate_up_run builds them once at weight-load time).
struct GatedMlpUpDescriptor {
    int32_t m = 0, f = 0, k = 0;
    ElementKind element = ElementKind::S8;       // S8 or Fp8E4M3
    ScaleMode scale_mode = ScaleMode::PerRowCol;  // the S8 SKU takes per-token x per-channel scales only
};

struct GatedMlpUpArgs {
    DeviceSpan<const void> a;          // [M,K] bytes, row pitch lda
    int64_t lda = 0;
    DeviceSpan<const void> b_gate_up;  // [2F,K] bytes, row pitch ldb
    int64_t ldb = 0;
    DeviceSpan<void> d;                // bf16 [M,F], row pitch ldd (a multiple of 8)
    int64_t ldd = 0;
    DeviceSpan<const float> scale_a;
    DeviceSpan<const float> scale_b;   // [2F] (or one value with ScaleMode::PerTensor)
    DeviceSpan<const float> bias;      // [2F] or empty
    float alpha = 1.0f;
};

class GatedMlpUpPlan {
  public:
    static Error select(const GatedMlpUpDescriptor& desc, const PlanPreference& pref, GatedMlpUpPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.f < 0 || desc.k < 0 || desc.f > INT32_MAX / 2) return Error::InvalidProblem;
        if (desc.element != ElementKind::S8 && desc.element != ElementKind::Fp8E4M3) return Error::Unsupported;
        if (desc.element == ElementKind::S8 && desc.scale_mode != ScaleMode::PerRowCol) return Error::InvalidProblem;
        if (desc.f % 32 != 0) return Error::Unsupported;
        const bool fp8 = desc.element == ElementKind::Fp8E4M3;
        out->desc_ = desc;
        out->sku_ = KernelSku{OpCategory::Gemm, OP_GATED_MLP_UP, desc.element, ElementKind::Bf16, LayoutSku::Rcr,
                              EpilogueKind::Identity, ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{fp8 ? MathPrecision::Fp8E4M3 : MathPrecision::Int8,
                                                 fp8 ? ElementKind::F32 : ElementKind::I32, true, true}};
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    const GatedMlpUpDescriptor& descriptor() const { return desc_; }
    size_t workspace_size() const {
        return baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_workspace_size(desc_.m, 2 * desc_.f, desc_.k);
    }
    Error can_implement(const GatedMlpUpArgs& x) const {
        const bool fp8 = desc_.element == ElementKind::Fp8E4M3;
        auto can = fp8 ? baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_can_implement
                       : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement;
        const int32_t st = can(desc_.m, 2 * desc_.f, desc_.k, x.a.ptr, x.lda, x.b_gate_up.ptr, x.ldb, x.d.ptr, x.ldd);
        if (st != 0) return status_to_error(st);
        if (desc_.m == 0 || desc_.f == 0) return Error::Ok;
        if (x.a.len < detail::span_elems(desc_.m, desc_.k, x.lda)) return Error::BufferTooSmall;
        if (x.b_gate_up.len < detail::span_elems(2 * static_cast<int64_t>(desc_.f), desc_.k, x.ldb))
            return Error::BufferTooSmall;
        if (x.d.len < detail::span_elems(desc_.m, desc_.f, x.ldd)) return Error::BufferTooSmall;
        if (!x.scale_a.ptr || !x.scale_b.ptr) return Error::InvalidProblem;
        const bool vec = desc_.scale_mode == ScaleMode::PerRowCol;
        if (x.scale_a.len < (vec ? static_cast<size_t>(desc_.m) : 1u) ||
            x.scale_b.len < (vec ? 2 * static_cast<size_t>(desc_.f) : 1u))
            return Error::BufferTooSmall;
        if (x.bias.ptr && x.bias.len < 2 * static_cast<size_t>(desc_.f)) return Error::BufferTooSmall;
        return Error::Ok;
    }
    Error run(void* stream, Workspace ws, const GatedMlpUpArgs& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        int32_t st;
        if (desc_.element == ElementKind::Fp8E4M3) {
            st = baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_run(
                desc_.m, 2 * desc_.f, desc_.k, x.a.ptr, x.lda, x.b_gate_up.ptr, x.ldb, x.d.ptr, x.ldd, x.scale_a.ptr,
                x.scale_b.ptr, static_cast<int32_t>(desc_.scale_mode), x.bias.ptr, x.alpha, ws.ptr, ws.bytes, stream);
        } else {
            st = baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run(
                desc_.m, 2 * desc_.f, desc_.k, x.a.ptr, x.lda, x.b_gate_up.ptr, x.ldb, x.d.ptr, x.ldd, x.scale_a.ptr,
                x.scale_b.ptr, x.bias.ptr, x.alpha, ws.ptr, ws.bytes, stream);
        }
        return status_to_error(st);
    }

  private:
    GatedMlpUpDescriptor desc_{};
    KernelSku sku_{};
};

// ---------------------------------------------------------------------------- GEMV
struct GemvQ8Descriptor {  // GemvDenseDescriptor, gemv_dense.rs:48-75 (m widened to 1..8)
    int32_t m = 1, n = 0, k = 0, batch = 1;
    LayoutSku layout = LayoutSku::Rrr;
};

struct GemvQ8Args {  // GemvDenseArgs, gemv_dense.rs:77-110, plus the scale vectors
    DeviceSpan<const int8_t> a;
    int64_t lda = 0, stride_a = 0;
    DeviceSpan<const int8_t> b;
    int64_t ldb = 0, stride_b = 0;
    DeviceSpan<const float> scale_a;
    int64_t stride_scale_a = 0;
    DeviceSpan<const float> scale_b;
    int64_t stride_scale_b = 0;
    DeviceSpan<void> d;  // bf16 elements (or int32 for the raw plan)
    int64_t ldd = 0, stride_d = 0;
    float alpha = 1.0f, beta = 0.0f;
};

class GemvQ8Plan {
  public:
    static Error select(const GemvQ8Descriptor& desc, const PlanPreference& pref, bool raw_accumulators,
                        GemvQ8Plan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.n < 0 || desc.k < 0 || desc.batch < 0 || desc.m > 8) return Error::InvalidProblem;
        out->desc_ = desc;
        out->raw_ = raw_accumulators;
        out->sku_ = KernelSku{OpCategory::Gemm, OP_GEMV_Q8, ElementKind::S8,
                              raw_accumulators ? ElementKind::I32 : ElementKind::Bf16, desc.layout, std::nullopt,
                              ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{MathPrecision::Int8, ElementKind::I32, true, true}};
        if (out->workspace_size() > pref.max_workspace_bytes) return Error::Unsupported;
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    int32_t layout_code() const { return desc_.layout == LayoutSku::Rrr ? 0 : 1; }
    size_t workspace_size() const {
        return baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(desc_.m, desc_.n, desc_.k, desc_.batch,
                                                                      layout_code());
    }
    Error can_implement(const GemvQ8Args& x) const {
        const int32_t st = baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(
            desc_.m, desc_.n, desc_.k, desc_.batch, layout_code(), x.lda, x.ldb, x.ldd, x.stride_a, x.stride_b,
            x.stride_d);
        if (st != 0) return status_to_error(st);
        if (x.stride_a < 0 || x.stride_b < 0 || x.stride_d < 0) return Error::InvalidProblem;
        if (desc_.batch == 0 || desc_.m == 0 || desc_.n == 0) return Error::Ok;
        const int64_t last = desc_.batch - 1;
        const bool rrr = desc_.layout == LayoutSku::Rrr;
        if (x.a.len < last * x.stride_a + detail::span_elems(desc_.m, desc_.k, x.lda)) return Error::BufferTooSmall;
        if (x.b.len < last * x.stride_b + detail::span_elems(rrr ? desc_.k : desc_.n, rrr ? desc_.n : desc_.k, x.ldb))
            return Error::BufferTooSmall;
        if (x.d.len < last * x.stride_d + detail::span_elems(desc_.m, desc_.n, x.ldd)) return Error::BufferTooSmall;
        if (!raw_) {
            if (!x.scale_a.ptr || !x.scale_b.ptr) return Error::InvalidProblem;
            if (x.scale_a.len < static_cast<size_t>(last * x.stride_scale_a + desc_.m)) return Error::BufferTooSmall;
            if (x.scale_b.len < static_cast<size_t>(last * x.stride_scale_b + desc_.n)) return Error::BufferTooSmall;
        }
        return Error::Ok;
    }
    Error run(void* stream, Workspace ws, const GemvQ8Args& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        const int32_t st =
            raw_ ? baracuda_kernels_gemv_q8_m1_s32_sm100a_run(desc_.m, desc_.n, desc_.k, desc_.batch, layout_code(),
                                                              x.alpha, x.beta, x.a.ptr, x.lda, x.stride_a, x.b.ptr, x.ldb,
                                                              x.stride_b, x.d.ptr, x.ldd, x.stride_d, ws.ptr, ws.bytes,
                                                              stream)
                 : baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(
                       desc_.m, desc_.n, desc_.k, desc_.batch, layout_code(), x.alpha, x.beta, x.a.ptr, x.lda, x.stride_a,
                       x.b.ptr, x.ldb, x.stride_b, x.scale_a.ptr, x.stride_scale_a, x.scale_b.ptr, x.stride_scale_b,
                       x.d.ptr, x.ldd, x.stride_d, ws.ptr, ws.bytes, stream);
        return status_to_error(st);
    }

    // Programmatic dependent launch, chosen per call: the weight stream starts while the kernel before this one on the
    // stream drains.  The caller asserts that that kernel does not write `b`.
    Error run_dependent(void* stream, Workspace ws, const GemvQ8Args& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        const int32_t st =
            raw_ ? baracuda_kernels_gemv_q8_m1_s32_sm100a_pdl_run(desc_.m, desc_.n, desc_.k, desc_.batch, layout_code(),
                                                                  x.alpha, x.beta, x.a.ptr, x.lda, x.stride_a, x.b.ptr,
                                                                  x.ldb, x.stride_b, x.d.ptr, x.ldd, x.stride_d, ws.ptr,
                                                                  ws.bytes, stream)
                 : baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run(
                       desc_.m, desc_.n, desc_.k, desc_.batch, layout_code(), x.alpha, x.beta, x.a.ptr, x.lda, x.stride_a,
                       x.b.ptr, x.ldb, x.stride_b, x.scale_a.ptr, x.stride_scale_a, x.scale_b.ptr, x.stride_scale_b,
                       x.d.ptr, x.ldd, x.stride_d, ws.ptr, ws.bytes, stream);
        return status_to_error(st);
    }

  private:
    GemvQ8Descriptor desc_{};
    KernelSku sku_{};
    bool raw_ = false;
};

// ---------------------------------------------------------------------------- activation quantiser and W8A8 linear
constexpr uint16_t OP_QUANTIZE_PER_TOKEN = 104;
constexpr uint16_t OP_SMOOTHQUANT_LINEAR = 105;

// QuantizePerTokenPlan (crates/baracuda-kernels/src/quantize/per_token.rs; recipe of
// dynamic_range_quantize_per_token_symmetric_kernel, baracuda_quantize_compose.cuh:144-201):
// scale[r] = absmax / qmax (1.0 for a zero row), q = clamp(rint(x * (1 / scale))).  f32 or bf16 in, s8 or e4m3 out.
struct QuantizePerTokenDescriptor {
    int32_t rows = 0, cols = 0;
    ElementKind input = ElementKind::F32;   // F32 or Bf16
    ElementKind output = ElementKind::S8;   // S8 or Fp8E4M3
    int32_t q_min = -127, q_max = 127;      // s8 only
};

class QuantizePerTokenPlan {
  public:
    static Error select(const QuantizePerTokenDescriptor& desc, const PlanPreference& pref, QuantizePerTokenPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.rows < 0 || desc.cols < 0) return Error::InvalidProblem;
        if (desc.input != ElementKind::F32 && desc.input != ElementKind::Bf16) return Error::Unsupported;
        if (desc.output != ElementKind::S8 && desc.output != ElementKind::Fp8E4M3) return Error::Unsupported;
        if (desc.output == ElementKind::S8 && (desc.q_min > desc.q_max || desc.q_max <= 0)) return Error::InvalidProblem;
        out->desc_ = desc;
        return Error::Ok;
    }
    size_t workspace_size() const { return 0; }
    // x: [rows, cols] of the input type with row pitch ld_in; q: bytes with row pitch ld_out; scale: float[rows].
    Error run(void* stream, DeviceSpan<const void> x, int64_t ld_in, DeviceSpan<float> scale, DeviceSpan<void> q,
              int64_t ld_out) const {
        const QuantizePerTokenDescriptor& d = desc_;
        if (x.len < detail::span_elems(d.rows, d.cols, ld_in) || q.len < detail::span_elems(d.rows, d.cols, ld_out))
            return Error::BufferTooSmall;
        if (scale.len < static_cast<size_t>(d.rows)) return Error::BufferTooSmall;
        int32_t st;
        if (d.output == ElementKind::S8) {
            auto run = d.input == ElementKind::F32 ? baracuda_kernels_quantize_per_token_sym_f32_s8_sm100a_run
                                                   : baracuda_kernels_quantize_per_token_sym_bf16_s8_sm100a_run;
            st = run(d.rows, d.cols, d.q_min, d.q_max, x.ptr, ld_in, scale.ptr, q.ptr, ld_out, nullptr, 0, stream);
        } else {
            auto run = d.input == ElementKind::F32 ? baracuda_kernels_quantize_per_token_sym_f32_e4m3_sm100a_run
                                                   : baracuda_kernels_quantize_per_token_sym_bf16_e4m3_sm100a_run;
            st = run(d.rows, d.cols, x.ptr, ld_in, scale.ptr, q.ptr, ld_out, nullptr, 0, stream);
        }
        return status_to_error(st);
    }

  private:
    QuantizePerTokenDescriptor desc_{};
};

// QuantizedLinearPlan (crates/baracuda-kernels/src/quantize/quantized_linear.rs:55-355): per-token quantiser, then the
// W8A8 matrix product, bf16 out.  m <= 8 takes the streaming GEMV, larger m the tcgen05 GEMM; bf16 activations with
// m <= 8 and a K the fused kernel serves run as ONE launch (quantiser inside the GEMV).
struct QuantizedLinearDescriptor {
    int32_t m = 0, c_out = 0, k = 0;
    int32_t q_min = -127, q_max = 127;
    ElementKind activation_element = ElementKind::Bf16;  // F32 or Bf16
};

struct QuantizedLinearArgs {  // quantized_linear.rs:82-120
    DeviceSpan<const void> activation;   // [M, K] f32 or bf16, packed rows
    DeviceSpan<const int8_t> weight_q;   // [C_out, K], packed rows
    DeviceSpan<const float> weight_scale;
    DeviceSpan<void> output;             // [M, C_out] bf16
    DeviceSpan<int8_t> act_q_scratch;    // [M, K]
    DeviceSpan<float> act_scale_scratch; // [M]
};

class QuantizedLinearPlan {
  public:
    static Error select(const QuantizedLinearDescriptor& desc, const PlanPreference& pref, QuantizedLinearPlan* out) {
        out->desc_ = desc;
        QuantizePerTokenDescriptor qd;
        qd.rows = desc.m;
        qd.cols = desc.k;
        qd.input = desc.activation_element;
        qd.output = ElementKind::S8;
        qd.q_min = desc.q_min;
        qd.q_max = desc.q_max;
        if (Error e = QuantizePerTokenPlan::select(qd, pref, &out->quant_); e != Error::Ok) return e;
        out->skinny_ = desc.m > 0 && desc.m <= 8;
        if (out->skinny_) {
            GemvQ8Descriptor gd;
            gd.m = desc.m;
            gd.n = desc.c_out;
            gd.k = desc.k;
            gd.batch = 1;
            gd.layout = LayoutSku::Rcr;
            return GemvQ8Plan::select(gd, pref, false, &out->gemv_);
        }
        return W8A8GemmPlan::select(QGemmDescriptor{desc.m, desc.c_out, desc.k, LayoutSku::Rcr, EpilogueKind::Identity}, pref,
                                    false, &out->gemm_);
    }
    const KernelSku& sku() const { return skinny_ ? gemv_.sku() : gemm_.sku(); }
    PrecisionGuarantee precision_guarantee() const { return sku().precision_guarantee; }
    size_t workspace_size() const { return skinny_ ? gemv_.workspace_size() : gemm_.workspace_size(); }
    // True when the whole step is one launch.
    bool fused_decode(const QuantizedLinearArgs& x) const {
        const int64_t ldk = desc_.k > 0 ? desc_.k : 1, ldn = desc_.c_out > 0 ? desc_.c_out : 1;
        return skinny_ && desc_.activation_element == ElementKind::Bf16 &&
               baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(desc_.m, desc_.c_out, desc_.k, ldk, ldk,
                                                                                  ldn) == 0 &&
               (reinterpret_cast<uintptr_t>(x.activation.ptr) & 15u) == 0 &&
               (reinterpret_cast<uintptr_t>(x.weight_q.ptr) & 15u) == 0;
    }
    // `dependent`: the matrix kernel is launched as a programmatic dependent (see GemvQ8Plan::run_dependent).
    Error run(void* stream, Workspace ws, const QuantizedLinearArgs& x, bool dependent = false) const {
        const QuantizedLinearDescriptor& d = desc_;
        const int64_t ldk = d.k > 0 ? d.k : 1, ldn = d.c_out > 0 ? d.c_out : 1;
        if (x.activation.len < detail::span_elems(d.m, d.k, ldk) || x.weight_q.len < detail::span_elems(d.c_out, d.k, ldk) ||
            x.output.len < detail::span_elems(d.m, d.c_out, ldn))
            return Error::BufferTooSmall;
        if (x.weight_scale.len < static_cast<size_t>(d.c_out) || x.act_scale_scratch.len < static_cast<size_t>(d.m))
            return Error::BufferTooSmall;
        if (fused_decode(x)) {
            auto run = dependent ? baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_pdl_run
                                 : baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run;
            return status_to_error(run(d.m, d.c_out, d.k, d.q_min, d.q_max, 1.0f, 0.0f, x.activation.ptr, ldk, x.weight_q.ptr,
                                       ldk, x.weight_scale.ptr, x.act_scale_scratch.ptr, x.output.ptr, ldn, nullptr, 0,
                                       stream));
        }
        if (x.act_q_scratch.len < detail::span_elems(d.m, d.k, ldk)) return Error::BufferTooSmall;
        if (Error e = quant_.run(stream, x.activation, ldk, x.act_scale_scratch, {x.act_q_scratch.ptr, x.act_q_scratch.len},
                                 ldk);
            e != Error::Ok)
            return e;
        const DeviceSpan<const float> sa{x.act_scale_scratch.ptr, x.act_scale_scratch.len};
        if (skinny_) {
            GemvQ8Args g;
            g.a = {x.act_q_scratch.ptr, x.act_q_scratch.len};
            g.lda = ldk;
            g.b = x.weight_q;
            g.ldb = ldk;
            g.scale_a = sa;
            g.scale_b = x.weight_scale;
            g.d = x.output;
            g.ldd = ldn;
            return dependent ? gemv_.run_dependent(stream, ws, g) : gemv_.run(stream, ws, g);
        }
        QGemmArgs g;
        g.a = {x.act_q_scratch.ptr, x.act_q_scratch.len};
        g.lda = ldk;
        g.b = {x.weight_q.ptr, x.weight_q.len};
        g.ldb = ldk;
        g.scale_a = sa;
        g.scale_b = x.weight_scale;
        g.d = x.output;
        g.ldd = ldn;
        return dependent ? gemm_.run_dependent(stream, ws, g) : gemm_.run(stream, ws, g);
    }

  private:
    QuantizedLinearDescriptor desc_{};
    QuantizePerTokenPlan quant_{};
    GemvQ8Plan gemv_{};
    W8A8GemmPlan gemm_{};
    bool skinny_ = false;
};

// SmoothQuantLinearPlan (crates/baracuda-kernels/src/quantize/smoothquant.rs:1-60, 70-330): one per-tensor activation
// scale (frozen model metadata, held by the descriptor and passed to the kernel by value) and per-channel weight
// scales.  One launch, no scratch: the reference fills an [M] scratch with the scalar and reuses its W8A8 kernel.
struct SmoothQuantLinearDescriptor {
    int32_t m = 0, n = 0, k = 0;
    float act_scale = 1.0f;
};

struct SmoothQuantLinearArgs {  // smoothquant.rs:120-150
    DeviceSpan<const int8_t> act_q;     // [M, K]
    DeviceSpan<const int8_t> weight_q;  // [N, K]
    DeviceSpan<const float> weight_scale;
    DeviceSpan<void> output;            // [M, N] bf16
};

class SmoothQuantLinearPlan {
  public:
    static Error select(const SmoothQuantLinearDescriptor& desc, const PlanPreference& pref, SmoothQuantLinearPlan* out) {
        if (!detail::backend_ok(pref)) return Error::Unsupported;
        if (desc.m < 0 || desc.n < 0 || desc.k < 0) return Error::InvalidProblem;
        if (!(desc.act_scale == desc.act_scale) || desc.act_scale - desc.act_scale != 0.0f) return Error::InvalidProblem;
        out->desc_ = desc;
        out->sku_ = KernelSku{OpCategory::Gemm, OP_SMOOTHQUANT_LINEAR, ElementKind::S8, ElementKind::Bf16, LayoutSku::Rcr,
                              EpilogueKind::Identity, ArchSku::Sm100a, BackendKind::Bespoke,
                              PrecisionGuarantee{MathPrecision::Int8, ElementKind::I32, true, true}};
        return Error::Ok;
    }
    const KernelSku& sku() const { return sku_; }
    PrecisionGuarantee precision_guarantee() const { return sku_.precision_guarantee; }
    size_t workspace_size() const {
        return baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_workspace_size(desc_.m, desc_.n, desc_.k);
    }
    Error can_implement(const SmoothQuantLinearArgs& x) const {
        const int64_t ldk = desc_.k > 0 ? desc_.k : 1, ldn = desc_.n > 0 ? desc_.n : 1;
        const int32_t st = baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_can_implement(
            desc_.m, desc_.n, desc_.k, x.act_q.ptr, ldk, x.weight_q.ptr, ldk, x.output.ptr, ldn);
        if (st != 0) return status_to_error(st);
        if (desc_.m == 0 || desc_.n == 0) return Error::Ok;
        if (x.act_q.len < detail::span_elems(desc_.m, desc_.k, ldk) || x.weight_q.len < detail::span_elems(desc_.n, desc_.k, ldk) ||
            x.output.len < detail::span_elems(desc_.m, desc_.n, ldn))
            return Error::BufferTooSmall;
        if (!x.weight_scale.ptr) return Error::InvalidProblem;
        if (x.weight_scale.len < static_cast<size_t>(desc_.n)) return Error::BufferTooSmall;
        return Error::Ok;
    }
    Error run(void* stream, Workspace ws, const SmoothQuantLinearArgs& x) const {
        if (Error e = can_implement(x); e != Error::Ok) return e;
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        const int64_t ldk = desc_.k > 0 ? desc_.k : 1, ldn = desc_.n > 0 ? desc_.n : 1;
        return status_to_error(baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run(
            desc_.m, desc_.n, desc_.k, x.act_q.ptr, ldk, x.weight_q.ptr, ldk, desc_.act_scale, x.weight_scale.ptr,
            x.output.ptr, ldn, ws.ptr, ws.bytes, stream));
    }

  private:
    SmoothQuantLinearDescriptor desc_{};
    KernelSku sku_{};
};

// ---------------------------------------------------------------------------- tensor parallel
// The reference's TensorParallelContext / ColumnParallelLinearPlan / RowParallelLinearPlan
// (crates/baracuda-megatron/src/lib.rs:153-240, 729-905, 1002-1200) for 8-bit operands.  `comm` is the handle
// made by baracuda_q_nccl_comm_init_rank (null with world 1).
struct TensorParallelContext {
    int32_t rank = 0;
    int32_t world = 1;
    void* comm = nullptr;
    bool valid() const { return world >= 1 && rank >= 0 && rank < world; }
};

// [lo, hi) of `extent` that `rank` owns; `extent` must divide evenly (lib.rs:781-785).
inline Error shard_range(int32_t extent, const TensorParallelContext& ctx, int32_t* lo, int32_t* hi) {
    if (!ctx.valid() || extent < 0 || extent % ctx.world != 0) return Error::InvalidProblem;
    const int32_t per = extent / ctx.world;
    *lo = ctx.rank * per;
    *hi = *lo + per;
    return Error::Ok;
}

// FusedMulticast: as FusedPeerStore, with the multicast address of the ranks' buffers in peer_y[world]; every tile is
// stored once and the NVLink switch replicates it.
enum class GatherMode : int32_t { None = BARACUDA_Q_GATHER_NONE, Nccl = BARACUDA_Q_GATHER_NCCL,
                                  FusedPeerStore = BARACUDA_Q_GATHER_FUSED_PEER_STORE,
                                  FusedMulticast = BARACUDA_Q_GATHER_FUSED_MULTICAST };
enum class ReduceMode : int32_t { None = BARACUDA_Q_REDUCE_NONE, Nccl = BARACUDA_Q_REDUCE_NCCL };

struct ColumnParallelArgs {
    DeviceSpan<const void> a;        // replicated activations [M, K]
    DeviceSpan<const float> scale_a; // [M] (or one float, per-tensor FP8)
    DeviceSpan<const void> w_local;  // Rcr: this rank's weight rows [N/world, K]; Rrr: its columns of the row-major
                                     // [K, N] weight (pointer at column rank * N/world, row pitch N)
    DeviceSpan<const float> scale_b_local;
    DeviceSpan<void> y_local;        // [M, N/world] bf16
    DeviceSpan<void> y_full;         // Nccl: [world, M, N/world] bf16
    void* const* peer_y = nullptr;   // FusedPeerStore / FusedMulticast: one row-major [M, N] buffer per rank (then the
                                     // multicast address, for FusedMulticast)
    int64_t ldd_full = 0;
    float alpha = 1.0f;
};

class ColumnParallelQGemmPlan {
  public:
    static Error make(const TensorParallelContext& ctx, int32_t m, int32_t out_features, int32_t k, ElementKind element,
                      ScaleMode mode, GatherMode gather, ColumnParallelQGemmPlan* out,
                      LayoutSku layout = LayoutSku::Rcr) {
        if (element != ElementKind::S8 && element != ElementKind::Fp8E4M3) return Error::Unsupported;
        out->rrr_ = layout == LayoutSku::Rrr;
        if (m < 0 || k < 0) return Error::InvalidProblem;
        int32_t lo = 0, hi = 0;
        if (Error e = shard_range(out_features, ctx, &lo, &hi); e != Error::Ok) return e;
        out->ctx_ = ctx;
        out->m_ = m;
        out->n_ = out_features;
        out->k_ = k;
        out->n_local_ = hi - lo;
        out->col0_ = lo;
        out->fp8_ = element == ElementKind::Fp8E4M3;
        out->mode_ = mode;
        out->gather_ = gather;
        return Error::Ok;
    }
    int32_t n_local() const { return n_local_; }
    int32_t first_column() const { return col0_; }
    Error forward(void* stream, const ColumnParallelArgs& x) const {
        const int64_t ldk = k_ > 0 ? k_ : 1, ldn = n_local_ > 0 ? n_local_ : 1;
        const int64_t ldb = rrr_ ? (n_ > 0 ? n_ : 1) : ldk;
        if (x.a.len < detail::span_elems(m_, k_, k_)) return Error::BufferTooSmall;
        if (x.w_local.len < (rrr_ ? detail::span_elems(k_, n_local_, ldb) : detail::span_elems(n_local_, k_, ldk)))
            return Error::BufferTooSmall;
        if (x.y_local.len < detail::span_elems(m_, n_local_, n_local_)) return Error::BufferTooSmall;
        if (gather_ == GatherMode::Nccl && x.y_full.len < static_cast<size_t>(m_) * n_) return Error::BufferTooSmall;
        const bool fused = gather_ == GatherMode::FusedPeerStore || gather_ == GatherMode::FusedMulticast;
        if (fused && !x.peer_y) return Error::InvalidProblem;
        int32_t st;
        if (fp8_) {
            auto run = rrr_ ? baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_nshard_run
                            : baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_nshard_run;
            st = run(ctx_.rank, ctx_.world, ctx_.comm, static_cast<int32_t>(gather_), m_, n_local_, k_, x.a.ptr, ldk,
                     x.w_local.ptr, ldb, x.y_local.ptr, ldn, x.scale_a.ptr, x.scale_b_local.ptr, static_cast<int32_t>(mode_),
                     x.alpha, x.y_full.ptr, x.peer_y, x.ldd_full ? x.ldd_full : n_, nullptr, 0, stream);
        } else {
            auto run = rrr_ ? baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_nshard_run
                            : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run;
            st = run(ctx_.rank, ctx_.world, ctx_.comm, static_cast<int32_t>(gather_), m_, n_local_, k_, x.a.ptr, ldk,
                     x.w_local.ptr, ldb, x.y_local.ptr, ldn, x.scale_a.ptr, x.scale_b_local.ptr, x.alpha, x.y_full.ptr,
                     x.peer_y, x.ldd_full ? x.ldd_full : n_, nullptr, 0, stream);
        }
        return status_to_error(st);
    }

  private:
    TensorParallelContext ctx_{};
    int32_t m_ = 0, n_ = 0, k_ = 0, n_local_ = 0, col0_ = 0;
    bool fp8_ = false, rrr_ = false;
    ScaleMode mode_ = ScaleMode::PerRowCol;
    GatherMode gather_ = GatherMode::None;
};

struct RowParallelArgs {
    DeviceSpan<const void> a_local;   // this rank's K slice of the activations [M, K/world]
    DeviceSpan<const float> scale_a;  // one per-token scale over the whole K, the same on every rank
    DeviceSpan<const void> w_local;   // [N, K/world]
    DeviceSpan<const float> scale_b;
    DeviceSpan<const float> bias;     // optional float[N], added once after the reduction
    DeviceSpan<void> y;               // [M, N] bf16, written on every rank
    float alpha = 1.0f;
};

class RowParallelQGemmPlan {
  public:
    static Error make(const TensorParallelContext& ctx, int32_t m, int32_t out_features, int32_t in_features,
                      ElementKind element, ScaleMode mode, ReduceMode reduce, RowParallelQGemmPlan* out) {
        if (element != ElementKind::S8 && element != ElementKind::Fp8E4M3) return Error::Unsupported;
        if (m < 0 || out_features < 0) return Error::InvalidProblem;
        int32_t lo = 0, hi = 0;
        if (Error e = shard_range(in_features, ctx, &lo, &hi); e != Error::Ok) return e;
        out->ctx_ = ctx;
        out->m_ = m;
        out->n_ = out_features;
        out->k_local_ = hi - lo;
        out->k0_ = lo;
        out->fp8_ = element == ElementKind::Fp8E4M3;
        out->mode_ = mode;
        out->reduce_ = reduce;
        return Error::Ok;
    }
    int32_t k_local() const { return k_local_; }
    int32_t first_k() const { return k0_; }
    size_t workspace_size() const { return baracuda_kernels_gemm_q8_kshard_workspace_size(m_, n_); }
    Error forward(void* stream, Workspace ws, const RowParallelArgs& x) const {
        if (ws.bytes < workspace_size()) return Error::WorkspaceTooSmall;
        if (x.a_local.len < detail::span_elems(m_, k_local_, k_local_) ||
            x.w_local.len < detail::span_elems(n_, k_local_, k_local_))
            return Error::BufferTooSmall;
        if (x.y.len < detail::span_elems(m_, n_, n_)) return Error::BufferTooSmall;
        if (x.bias.ptr && x.bias.len < static_cast<size_t>(n_)) return Error::BufferTooSmall;
        const int64_t ldk = k_local_ > 0 ? k_local_ : 1, ldn = n_ > 0 ? n_ : 1;
        const int32_t st =
            fp8_ ? baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run(
                       ctx_.rank, ctx_.world, ctx_.comm, static_cast<int32_t>(reduce_), m_, n_, k_local_, x.a_local.ptr, ldk,
                       x.w_local.ptr, ldk, x.y.ptr, ldn, x.scale_a.ptr, x.scale_b.ptr, static_cast<int32_t>(mode_),
                       x.bias.ptr, x.alpha, ws.ptr, ws.bytes, stream)
                 : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(
                       ctx_.rank, ctx_.world, ctx_.comm, static_cast<int32_t>(reduce_), m_, n_, k_local_, x.a_local.ptr, ldk,
                       x.w_local.ptr, ldk, x.y.ptr, ldn, x.scale_a.ptr, x.scale_b.ptr, x.bias.ptr, x.alpha, ws.ptr, ws.bytes,
                       stream);
        return status_to_error(st);
    }

    // Both exchanges inside the kernels over peer-mapped memory (no all-reduce of the sums): `peer_y` and `peer_staging`
    // hold `world` device pointers valid on this rank ([M, N] bf16 results, [world][M / world][N] 32-bit staging).  The
    // ranks meet twice per call: through the flag barrier when `peer_flags` is given (`world` flag buffers of
    // baracuda_q_peer_barrier_flag_bytes() bytes, zeroed once; no communicator needed), else through a one-float
    // all-reduce on `barrier_scratch`.
    Error forward_fused(void* stream, const RowParallelArgs& x, void* const* peer_y, void* const* peer_staging,
                        void* const* peer_flags, float* barrier_scratch = nullptr) const {
        if (!peer_y || !peer_staging || (!peer_flags && !barrier_scratch)) return Error::InvalidProblem;
        if (ctx_.world < 2 || m_ % ctx_.world != 0) return Error::InvalidProblem;
        if (x.a_local.len < detail::span_elems(m_, k_local_, k_local_) ||
            x.w_local.len < detail::span_elems(n_, k_local_, k_local_))
            return Error::BufferTooSmall;
        if (x.bias.ptr && x.bias.len < static_cast<size_t>(n_)) return Error::BufferTooSmall;
        const int64_t ldk = k_local_ > 0 ? k_local_ : 1, ldn = n_ > 0 ? n_ : 1;
        int32_t st;
        if (peer_flags) {
            st = fp8_ ? baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run(
                            ctx_.rank, ctx_.world, m_, n_, k_local_, x.a_local.ptr, ldk, x.w_local.ptr, ldk, peer_y, ldn,
                            x.scale_a.ptr, x.scale_b.ptr, static_cast<int32_t>(mode_), x.bias.ptr, x.alpha, peer_staging,
                            peer_flags, stream)
                      : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run(
                            ctx_.rank, ctx_.world, m_, n_, k_local_, x.a_local.ptr, ldk, x.w_local.ptr, ldk, peer_y, ldn,
                            x.scale_a.ptr, x.scale_b.ptr, x.bias.ptr, x.alpha, peer_staging, peer_flags, stream);
        } else {
            st = fp8_ ? baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run(
                            ctx_.rank, ctx_.world, ctx_.comm, m_, n_, k_local_, x.a_local.ptr, ldk, x.w_local.ptr, ldk, peer_y,
                            ldn, x.scale_a.ptr, x.scale_b.ptr, static_cast<int32_t>(mode_), x.bias.ptr, x.alpha, peer_staging,
                            barrier_scratch, stream)
                      : baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run(
                            ctx_.rank, ctx_.world, ctx_.comm, m_, n_, k_local_, x.a_local.ptr, ldk, x.w_local.ptr, ldk, peer_y,
                            ldn, x.scale_a.ptr, x.scale_b.ptr, x.bias.ptr, x.alpha, peer_staging, barrier_scratch, stream);
        }
        return status_to_error(st);
    }

  private:
    TensorParallelContext ctx_{};
    int32_t m_ = 0, n_ = 0, k_local_ = 0, k0_ = 0;
    bool fp8_ = false;
    ScaleMode mode_ = ScaleMode::PerRowCol;
    ReduceMode reduce_ = ReduceMode::Nccl;
};

}  // namespace baracuda

namespace std {
template <>
struct hash<baracuda::KernelSku> {
    size_t operator()(const baracuda::KernelSku& s) const noexcept { return s.hash(); }
};
}  // namespace std
