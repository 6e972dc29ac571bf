//! Flat C symbols of the sm_100a quantized-GEMM library (`libbaracuda_kernels_q.so`).
//!
//! Same conventions as every bespoke family in this crate: device pointers owned by the
//! caller, `i32` dims, `i64` leading dimensions and strides in elements, a `cudaStream_t`
//! as `*mut c_void`, an `i32` status (0 ok, 1 misaligned, 2 invalid problem, 3 unsupported,
//! 4 workspace, 5 launch failure; 6 / 7 only from the sharded entry points: NCCL not
//! loadable / NCCL call failed).  `*_can_implement` and `*_workspace_size` are pure host
//! functions.  Not compiled in the environment this file was written in.

use core::ffi::c_void;

/// `scale_a` / `scale_b` each point at one `f32`.
pub const BARACUDA_Q_SCALE_PER_TENSOR: i32 = 0;
/// `scale_a` is `f32[M]`, `scale_b` is `f32[N]`.
pub const BARACUDA_Q_SCALE_PER_ROW_COL: i32 = 1;
/// GEMV weight layout: row-major `[K, N]` (the reference GEMV's only layout).
pub const BARACUDA_Q_LAYOUT_RRR: i32 = 0;
/// GEMV weight layout: `[N, K]`, K contiguous.
pub const BARACUDA_Q_LAYOUT_RCR: i32 = 1;
/// Longest K the int8 symbols accept (the sums cannot leave 32 bits up to here).
pub const BARACUDA_Q_MAX_INT8_K: i32 = 131_071;

macro_rules! gemm_bf16_family {
    ($run:ident, $can:ident, $ws:ident $(, $mode:ident : $mode_ty:ty)?) => {
        extern "C" {
            /// `D = bf16(alpha * ((sa * sb) * acc) + beta * C)`; see the header for the scale modes.
            pub fn $run(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *mut c_void, ldd: i64,
                scale_a: *const c_void, scale_b: *const c_void, $($mode: $mode_ty,)?
                alpha: f32, beta: f32,
                workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
            ) -> i32;
            /// Host-only validity check (pointers may be null).
            pub fn $can(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *const c_void, ldd: i64,
            ) -> i32;
            /// Always 0.
            pub fn $ws(m: i32, n: i32, k: i32) -> usize;
        }
    };
}

gemm_bf16_family!(
    baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run,
    baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement,
    baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_workspace_size
);
gemm_bf16_family!(
    baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run,
    baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_can_implement,
    baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_workspace_size
);
gemm_bf16_family!(
    baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_run,
    baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement,
    baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_workspace_size,
    scale_mode: i32
);
gemm_bf16_family!(
    baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_run,
    baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_can_implement,
    baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_workspace_size,
    scale_mode: i32
);

macro_rules! gemm_bf16_epilogue_run {
    ($name:ident) => {
        extern "C" {
            /// The bf16 SKU with the `EpilogueKind` chain: `epilogue` 0 identity .. 4 bias+silu, `bias` is `f32[N]`.
            pub fn $name(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *mut c_void, ldd: i64,
                scale_a: *const c_void, scale_b: *const c_void, scale_mode: i32,
                bias: *const c_void, epilogue: i32, alpha: f32, beta: f32,
                workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
            ) -> i32;
        }
    };
}
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_epilogue_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_epilogue_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_epilogue_run);
// The same arguments, launched as programmatic dependents of the kernel before them on the stream (a per-call choice:
// the caller promises that kernel does not write `b`).
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_pdl_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_pdl_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_pdl_run);
gemm_bf16_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_pdl_run);

macro_rules! gemm_same_type_family {
    ($run:ident, $can:ident, $ws:ident) => {
        extern "C" {
            /// The reference's own 8-bit-out contract (`IntGemmPlan` / `Fp8GemmPlan`) or the raw accumulators.
            pub fn $run(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *mut c_void, ldd: i64,
                alpha: f32, beta: f32,
                workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
            ) -> i32;
            pub fn $can(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *const c_void, ldd: i64,
            ) -> i32;
            pub fn $ws(m: i32, n: i32, k: i32) -> usize;
        }
    };
}
gemm_same_type_family!(baracuda_kernels_gemm_s8_rcr_sm100a_run, baracuda_kernels_gemm_s8_rcr_sm100a_can_implement, baracuda_kernels_gemm_s8_rcr_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_s8_rrr_sm100a_run, baracuda_kernels_gemm_s8_rrr_sm100a_can_implement, baracuda_kernels_gemm_s8_rrr_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run, baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_can_implement, baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_run, baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_can_implement, baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_s8_rcr_s32_sm100a_run, baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement, baracuda_kernels_gemm_s8_rcr_s32_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_s8_rrr_s32_sm100a_run, baracuda_kernels_gemm_s8_rrr_s32_sm100a_can_implement, baracuda_kernels_gemm_s8_rrr_s32_sm100a_workspace_size);
gemm_same_type_family!(baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run, baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_can_implement, baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_workspace_size);

macro_rules! gemm_same_type_epilogue_run {
    ($name:ident) => {
        extern "C" {
            /// `bias_kind` 1 = `f32[N]`, 2 = `i32[N]` (s8 only); `epilogue` as in `EpilogueKind`.
            pub fn $name(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *mut c_void, ldd: i64,
                bias: *const c_void, bias_kind: i32, epilogue: i32, alpha: f32, beta: f32,
                workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
            ) -> i32;
        }
    };
}
gemm_same_type_epilogue_run!(baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run);
gemm_same_type_epilogue_run!(baracuda_kernels_gemm_s8_rrr_sm100a_epilogue_run);
gemm_same_type_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_epilogue_run);
gemm_same_type_epilogue_run!(baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_epilogue_run);

macro_rules! gemm_same_type_bias_run {
    ($($name:ident),+ $(,)?) => {
        extern "C" {
            $(
            /// Signature of the reference's `baracuda_kernels_gemm_s8_rrr_sm80_bias…_run` /
            /// `baracuda_kernels_gemm_fp8_e4m3_{rcr,rrr}_sm89_bias…_run` (`bias` before `alpha`); the suffix names the
            /// activation and, for s8, the bias element (`f32` or `i32`).
            pub fn $name(
                m: i32, n: i32, k: i32,
                a: *const c_void, lda: i64, b: *const c_void, ldb: i64,
                c: *const c_void, ldc: i64, d: *mut c_void, ldd: i64,
                bias: *const c_void, alpha: f32, beta: f32,
                workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
            ) -> i32;
            )+
        }
    };
}
gemm_same_type_bias_run!(
    baracuda_kernels_gemm_s8_rcr_sm100a_bias_f32_run, baracuda_kernels_gemm_s8_rcr_sm100a_bias_relu_f32_run,
    baracuda_kernels_gemm_s8_rcr_sm100a_bias_gelu_f32_run, baracuda_kernels_gemm_s8_rcr_sm100a_bias_silu_f32_run,
    baracuda_kernels_gemm_s8_rcr_sm100a_bias_i32_run, baracuda_kernels_gemm_s8_rcr_sm100a_bias_relu_i32_run,
    baracuda_kernels_gemm_s8_rcr_sm100a_bias_gelu_i32_run, baracuda_kernels_gemm_s8_rcr_sm100a_bias_silu_i32_run,
    baracuda_kernels_gemm_s8_rrr_sm100a_bias_f32_run, baracuda_kernels_gemm_s8_rrr_sm100a_bias_relu_f32_run,
    baracuda_kernels_gemm_s8_rrr_sm100a_bias_gelu_f32_run, baracuda_kernels_gemm_s8_rrr_sm100a_bias_silu_f32_run,
    baracuda_kernels_gemm_s8_rrr_sm100a_bias_i32_run, baracuda_kernels_gemm_s8_rrr_sm100a_bias_relu_i32_run,
    baracuda_kernels_gemm_s8_rrr_sm100a_bias_gelu_i32_run, baracuda_kernels_gemm_s8_rrr_sm100a_bias_silu_i32_run,
    baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_run, baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_relu_run,
    baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_gelu_run, baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_bias_silu_run,
    baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_run, baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_relu_run,
    baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_gelu_run, baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_bias_silu_run,
);

extern "C" {
    /// SmoothQuant inference forward: one per-tensor activation scale by value, per-channel weight scales.
    pub fn baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run(
        m: i32, n: i32, k: i32,
        act_q: *const c_void, lda: i64, weight_q: *const c_void, ldb: i64,
        act_scale: f32, weight_scale: *const c_void,
        output: *mut c_void, ldd: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_can_implement(
        m: i32, n: i32, k: i32,
        act_q: *const c_void, lda: i64, weight_q: *const c_void, ldb: i64,
        output: *const c_void, ldd: i64,
    ) -> i32;
    pub fn baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_workspace_size(m: i32, n: i32, k: i32) -> usize;

    /// Int8 decode GEMV, bf16 out.  Argument order of `baracuda_kernels_gemv_dense_m1_bf16_run`
    /// with the two scale vectors (and their batch strides) inserted before `d`.
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        alpha: f32, beta: f32,
        a: *const c_void, lda: i64, stride_a: i64,
        b: *const c_void, ldb: i64, stride_b: i64,
        scale_a: *const c_void, stride_scale_a: i64,
        scale_b: *const c_void, stride_scale_b: i64,
        d: *mut c_void, ldd: i64, stride_d: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    /// The same call under programmatic dependent launch: the caller promises that the kernel launched just
    /// before on `stream` does not write the weights `b`.
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        alpha: f32, beta: f32,
        a: *const c_void, lda: i64, stride_a: i64,
        b: *const c_void, ldb: i64, stride_b: i64,
        scale_a: *const c_void, stride_scale_a: i64,
        scale_b: *const c_void, stride_scale_b: i64,
        d: *mut c_void, ldd: i64, stride_d: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        lda: i64, ldb: i64, ldd: i64,
        stride_a: i64, stride_b: i64, stride_d: i64,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(m: i32, n: i32, k: i32, batch: i32, layout: i32) -> usize;
    /// Same GEMV with its scratch inside the library image (callers that may not allocate); 8 MiB limit.
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        alpha: f32, beta: f32,
        a: *const c_void, lda: i64, stride_a: i64,
        b: *const c_void, ldb: i64, stride_b: i64,
        scale_a: *const c_void, stride_scale_a: i64,
        scale_b: *const c_void, stride_scale_b: i64,
        d: *mut c_void, ldd: i64, stride_d: i64,
        stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity() -> usize;
    /// The int32 sums of the same GEMV.
    pub fn baracuda_kernels_gemv_q8_m1_s32_sm100a_run(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        alpha: f32, beta: f32,
        a: *const c_void, lda: i64, stride_a: i64,
        b: *const c_void, ldb: i64, stride_b: i64,
        d: *mut c_void, ldd: i64, stride_d: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_s32_sm100a_pdl_run(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        alpha: f32, beta: f32,
        a: *const c_void, lda: i64, stride_a: i64,
        b: *const c_void, ldb: i64, stride_b: i64,
        d: *mut c_void, ldd: i64, stride_d: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_s32_sm100a_can_implement(
        m: i32, n: i32, k: i32, batch: i32, layout: i32,
        lda: i64, ldb: i64, ldd: i64,
        stride_a: i64, stride_b: i64, stride_d: i64,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_s32_sm100a_workspace_size(m: i32, n: i32, k: i32, batch: i32, layout: i32) -> usize;
    /// Decode step in one launch: per-token quantiser inside the GEMV (bf16 activations in).
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run(
        m: i32, n: i32, k: i32, qmin: i32, qmax: i32,
        alpha: f32, beta: f32,
        x_bf16: *const c_void, ldx: i64, b: *const c_void, ldb: i64, scale_b: *const c_void,
        scale_a_out: *mut c_void, d: *mut c_void, ldd: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_pdl_run(
        m: i32, n: i32, k: i32, qmin: i32, qmax: i32,
        alpha: f32, beta: f32,
        x_bf16: *const c_void, ldx: i64, b: *const c_void, ldb: i64, scale_b: *const c_void,
        scale_a_out: *mut c_void, d: *mut c_void, ldd: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(
        m: i32, n: i32, k: i32, ldx: i64, ldb: i64, ldd: i64,
    ) -> i32;

    /// Per-token symmetric quantizers (`dynamic_range_quantize_per_token_sym_*` with row pitches).
    pub fn baracuda_kernels_quantize_per_token_sym_f32_s8_sm100a_run(
        rows: i32, cols: i32, qmin: i32, qmax: i32,
        input: *const c_void, ld_in: i64, scale: *mut c_void, output: *mut c_void, ld_out: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_quantize_per_token_sym_bf16_s8_sm100a_run(
        rows: i32, cols: i32, qmin: i32, qmax: i32,
        input: *const c_void, ld_in: i64, scale: *mut c_void, output: *mut c_void, ld_out: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_quantize_per_token_sym_f32_e4m3_sm100a_run(
        rows: i32, cols: i32,
        input: *const c_void, ld_in: i64, scale: *mut c_void, output: *mut c_void, ld_out: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_quantize_per_token_sym_bf16_e4m3_sm100a_run(
        rows: i32, cols: i32,
        input: *const c_void, ld_in: i64, scale: *mut c_void, output: *mut c_void, ld_out: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;

    /// Column-parallel forward; `gather` 0 sharded, 1 ncclAllGather (rank-major), 2 fused peer stores,
    /// 3 fused multicast stores (`peer_d` then has `world + 1` entries, the last the multicast address).
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_nshard_run(
        rank: i32, world: i32, comm: *mut c_void, gather: i32,
        m: i32, n_local: i32, k: i32,
        a: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d_local: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b_local: *const c_void, scale_mode: i32, alpha: f32,
        d_full: *mut c_void, peer_d: *const *mut c_void, ldd_full: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run(
        rank: i32, world: i32, comm: *mut c_void, gather: i32,
        m: i32, n_local: i32, k: i32,
        a: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d_local: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b_local: *const c_void, alpha: f32,
        d_full: *mut c_void, peer_d: *const *mut c_void, ldd_full: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;

    /// The same for a row-major `[K, N]` weight: `b_local` points at column `rank * n_local`, `ldb` stays the full N.
    pub fn baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_nshard_run(
        rank: i32, world: i32, comm: *mut c_void, gather: i32,
        m: i32, n_local: i32, k: i32,
        a: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d_local: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b_local: *const c_void, scale_mode: i32, alpha: f32,
        d_full: *mut c_void, peer_d: *const *mut c_void, ldd_full: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_nshard_run(
        rank: i32, world: i32, comm: *mut c_void, gather: i32,
        m: i32, n_local: i32, k: i32,
        a: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d_local: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b_local: *const c_void, alpha: f32,
        d_full: *mut c_void, peer_d: *const *mut c_void, ldd_full: i64,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;

    /// Row-parallel (K-sharded) forward: raw accumulators in `workspace` (`[M, N]` 32-bit words), `reduce` 0 none,
    /// 1 `ncclAllReduce(sum)`, then one pass that applies scales, alpha and the optional `f32[N]` bias.
    pub fn baracuda_kernels_gemm_q8_kshard_workspace_size(m: i32, n: i32) -> usize;
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(
        rank: i32, world: i32, comm: *mut c_void, reduce: i32,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d: *mut c_void, ldd: i64, scale_a: *const c_void, scale_b: *const c_void,
        bias: *const c_void, alpha: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run(
        rank: i32, world: i32, comm: *mut c_void, reduce: i32,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        d: *mut c_void, ldd: i64, scale_a: *const c_void, scale_b: *const c_void, scale_mode: i32,
        bias: *const c_void, alpha: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    /// Both exchanges inside the kernels over peer-mapped memory: `peer_y` and `peer_staging` hold `world` device
    /// pointers valid on this rank (`[M, N]` bf16 results, `[world][M / world][N]` 32-bit staging).
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run(
        rank: i32, world: i32, comm: *mut c_void,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        peer_y: *const *mut c_void, ldy: i64, scale_a: *const c_void, scale_b: *const c_void,
        bias: *const c_void, alpha: f32,
        peer_staging: *const *mut c_void, barrier_scratch: *mut c_void, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run(
        rank: i32, world: i32, comm: *mut c_void,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        peer_y: *const *mut c_void, ldy: i64, scale_a: *const c_void, scale_b: *const c_void, scale_mode: i32,
        bias: *const c_void, alpha: f32,
        peer_staging: *const *mut c_void, barrier_scratch: *mut c_void, stream: *mut c_void,
    ) -> i32;

    /// The fused forward with the ranks meeting through a flag barrier over peer memory (no communicator):
    /// `peer_flags` holds `world` pointers to flag buffers of `baracuda_q_peer_barrier_flag_bytes()` bytes, zeroed once.
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run(
        rank: i32, world: i32,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        peer_y: *const *mut c_void, ldy: i64, scale_a: *const c_void, scale_b: *const c_void,
        bias: *const c_void, alpha: f32,
        peer_staging: *const *mut c_void, peer_flags: *const *mut c_void, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run(
        rank: i32, world: i32,
        m: i32, n: i32, k_local: i32,
        a_local: *const c_void, lda: i64, b_local: *const c_void, ldb: i64,
        peer_y: *const *mut c_void, ldy: i64, scale_a: *const c_void, scale_b: *const c_void, scale_mode: i32,
        bias: *const c_void, alpha: f32,
        peer_staging: *const *mut c_void, peer_flags: *const *mut c_void, stream: *mut c_void,
    ) -> i32;
    /// The barrier itself (one-block kernel on `stream`; bounded wait, `limit_cycles` 0 = about a second; status 301).
    pub fn baracuda_q_peer_barrier_run(
        peer_flags: *const *mut c_void, rank: i32, world: i32, limit_cycles: i64, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_q_peer_barrier_flag_bytes() -> usize;

    /// Gated-MLP up-projection over an interleaved gate/up weight `[n2, K]`: `D = silu(z_gate) * z_up`, bf16 `[M, n2 / 2]`.
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run(
        m: i32, n2: i32, k: i32,
        a: *const c_void, lda: i64, b_gate_up: *const c_void, ldb: i64,
        d: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b: *const c_void, bias: *const c_void,
        alpha: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_workspace_size(m: i32, n2: i32, k: i32) -> usize;
    pub fn baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement(
        m: i32, n2: i32, k: i32,
        a: *const c_void, lda: i64, b_gate_up: *const c_void, ldb: i64,
        d: *const c_void, ldd: i64,
    ) -> i32;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_run(
        m: i32, n2: i32, k: i32,
        a: *const c_void, lda: i64, b_gate_up: *const c_void, ldb: i64,
        d: *mut c_void, ldd: i64,
        scale_a: *const c_void, scale_b: *const c_void, scale_mode: i32, bias: *const c_void,
        alpha: f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_workspace_size(m: i32, n2: i32, k: i32) -> usize;
    pub fn baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_can_implement(
        m: i32, n2: i32, k: i32,
        a: *const c_void, lda: i64, b_gate_up: *const c_void, ldb: i64,
        d: *const c_void, ldd: i64,
    ) -> i32;
    /// Builds the interleaved operand (and, with 4-byte rows, the interleaved scale / bias vectors): out row
    /// `64 b + i` = gate row `32 b + i` for `i < 32`, else up row `32 b + i - 32`; pitches in bytes.
    pub fn baracuda_kernels_q_interleave_gate_up_run(
        f_rows: i64, row_bytes: i64,
        gate: *const c_void, gate_pitch: i64, up: *const c_void, up_pitch: i64,
        out: *mut c_void, out_pitch: i64, stream: *mut c_void,
    ) -> i32;

    /// Communicator helpers over the run-time-loaded NCCL (`Communicator::{new_with_id, all_gather}` of baracuda-nccl).
    pub fn baracuda_q_nccl_version() -> i32;
    pub fn baracuda_q_nccl_unique_id(id_out_128_bytes: *mut c_void) -> i32;
    pub fn baracuda_q_nccl_comm_init_rank(comm_out: *mut *mut c_void, world: i32, id_128_bytes: *const c_void, rank: i32) -> i32;
    pub fn baracuda_q_nccl_comm_destroy(comm: *mut c_void) -> i32;
    pub fn baracuda_q_nccl_stream_barrier(comm: *mut c_void, scratch_one_float: *mut c_void, stream: *mut c_void) -> i32;
    pub fn baracuda_q_nccl_all_gather_bytes(
        comm: *mut c_void, world: i32, send: *const c_void, recv: *mut c_void, bytes_per_rank: usize, stream: *mut c_void,
    ) -> i32;

    /// Test hooks: a kernel choice for the calling thread only (see the header for keys and values), and a launch
    /// whose only thread waits `limit_cycles` on a barrier nothing completes (status 299 afterwards).
    pub fn baracuda_kernels_q_set_tuning(key: i32, value: i32) -> i32;
    pub fn baracuda_kernels_q_selftest_bounded_wait(limit_cycles: i64, stream: *mut c_void) -> i32;

    /// Read-and-clear of the word a kernel sets when one of its bounded waits ran out (0 = none).
    pub fn baracuda_kernels_q_device_status() -> i32;
}
