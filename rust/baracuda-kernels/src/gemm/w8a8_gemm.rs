//! `W8A8GemmPlan` — s8 x s8 -> s32 on `tcgen05.mma` with the per-token x per-channel dequant fused
//! into a bf16 store (sm_100a).
//!
//! One launch where `QuantizedLinearPlan` needs its one-thread-per-cell kernel
//! (`quantize/quantized_linear.rs:262-355`) or the s8-out `IntGemmPlan` needs a dequant pass:
//!
//! ```text
//! D[m, n] = bf16( act( alpha * ((scale_a[m] * scale_b[n]) * (float)acc[m, n]) + beta * C[m, n] + bias[n] ) )
//! ```
//!
//! with the reference's product order (`baracuda_quantize_compose.cuh:271-274`), so with `alpha == 1`
//! and no C / bias the result equals `quantized_linear_w8a8` bit for bit, rounded once to bf16.
//! Both weight layouts (`LayoutSku::Rcr`: `[N, K]` rows; `LayoutSku::Rrr`: row-major `[K, N]`).
//! Not compiled in the environment this file was written in.

use core::ffi::c_void;

use baracuda_cutlass::{Error, Result};
use baracuda_driver::Stream;
use baracuda_kernels_sys as sys;
use baracuda_kernels_types::{
    ArchSku, BackendKind, ElementKind, EpilogueKind, KernelSku, LayoutSku, MathPrecision, MatrixMut, MatrixRef,
    OpCategory, PlanPreference, PrecisionGuarantee, VectorRef, Workspace, S8,
};
use half::bf16;

/// Category-local op discriminant of this family inside `OpCategory::Gemm`.
pub const OP_W8A8_GEMM: u16 = 0x0801;

/// Shape, weight layout and epilogue chain.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub struct W8A8GemmDescriptor {
    /// Rows of the activation and of the output (tokens).
    pub m: i32,
    /// Output channels.
    pub n: i32,
    /// Reduction depth; at most 131 071 (the int32 accumulator cannot overflow up to there).
    pub k: i32,
    /// Weight storage: `Rcr` = `[N, K]`, `Rrr` = `[K, N]`.
    pub layout: LayoutSku,
    /// `Identity` or one of the `Bias*` chains (bias is `f32[N]`).
    pub epilogue: EpilogueKind,
}

/// Device views of one launch.
#[derive(Debug)]
pub struct W8A8GemmArgs<'a> {
    /// Quantized activations, row-major `[M, K]`.
    pub a: MatrixRef<'a, S8>,
    /// Quantized weights in the descriptor's layout.
    pub b: MatrixRef<'a, S8>,
    /// Optional residual, row-major `[M, N]` bf16; may alias `d`'s storage. Read only when `beta != 0`.
    pub c: Option<MatrixRef<'a, bf16>>,
    /// Output, row-major `[M, N]`.
    pub d: MatrixMut<'a, bf16>,
    /// Per-token scales, `f32[M]`.
    pub scale_a: VectorRef<'a, f32>,
    /// Per-output-channel scales, `f32[N]`.
    pub scale_b: VectorRef<'a, f32>,
    /// Required by the `Bias*` epilogues, `f32[N]`.
    pub bias: Option<VectorRef<'a, f32>>,
    /// Multiplier on the dequantised accumulator.
    pub alpha: f32,
    /// Multiplier on `c`.
    pub beta: f32,
}

/// The plan: a validated descriptor and the SKU fixed at `select`.
#[derive(Debug)]
pub struct W8A8GemmPlan {
    desc: W8A8GemmDescriptor,
    sku: KernelSku,
}

fn epilogue_code(e: EpilogueKind) -> i32 {
    match e {
        EpilogueKind::Identity => 0,
        EpilogueKind::Bias => 1,
        EpilogueKind::BiasRelu => 2,
        EpilogueKind::BiasGelu => 3,
        EpilogueKind::BiasSilu => 4,
    }
}

pub(crate) fn map_status(code: i32, what: &'static str) -> Result<()> {
    match code {
        0 => Ok(()),
        1 => Err(Error::MisalignedOperand(what)),
        2 => Err(Error::InvalidProblem(what)),
        3 => Err(Error::Unsupported(what)),
        4 => Err(Error::WorkspaceTooSmall { needed: 0, got: 0 }),
        n => Err(Error::CutlassInternal(n)),
    }
}

impl W8A8GemmPlan {
    /// Validates the descriptor once and fixes the SKU. Bespoke-only: `pref.prefer_backend` may be
    /// `None` or `Some(BackendKind::Bespoke)`.
    pub fn select(_stream: &Stream, desc: &W8A8GemmDescriptor, pref: PlanPreference) -> Result<Self> {
        if desc.m < 0 || desc.n < 0 || desc.k < 0 {
            return Err(Error::InvalidProblem("W8A8GemmPlan: M, N, K must be non-negative"));
        }
        if desc.k > sys::BARACUDA_Q_MAX_INT8_K {
            return Err(Error::Unsupported("W8A8GemmPlan: K beyond 131071 could overflow the int32 accumulator"));
        }
        match pref.prefer_backend {
            None | Some(BackendKind::Bespoke) => {}
            Some(_) => return Err(Error::Unsupported("W8A8GemmPlan: bespoke-kernel-backed only")),
        }
        let sku = KernelSku {
            category: OpCategory::Gemm,
            op: OP_W8A8_GEMM,
            element: ElementKind::S8,
            aux_element: Some(ElementKind::Bf16),
            layout: Some(desc.layout),
            epilogue: Some(desc.epilogue),
            arch: ArchSku::Sm100a,
            backend: BackendKind::Bespoke,
            precision_guarantee: PrecisionGuarantee {
                math_precision: MathPrecision::Int8,
                accumulator: ElementKind::I32,
                deterministic: true,
                bit_stable_on_same_hardware: true,
            },
        };
        Ok(Self { desc: *desc, sku })
    }

    /// Selection identity: `Copy + Eq + Hash`, usable as an autotuner cache key.
    pub fn sku(&self) -> KernelSku {
        self.sku
    }

    /// Integer accumulation: exact and bit-stable.
    pub fn precision_guarantee(&self) -> PrecisionGuarantee {
        self.sku.precision_guarantee
    }

    /// No scratch.
    pub fn workspace_size(&self) -> usize {
        0
    }

    /// Shape, leading-dimension, alignment and buffer-length checks; the typed layer is the soundness
    /// boundary for lengths, the C side re-checks everything else.
    pub fn can_implement(&self, args: &W8A8GemmArgs<'_>) -> Result<()> {
        let d = &self.desc;
        let (b_rows, b_cols) = match d.layout {
            LayoutSku::Rcr => (d.n, d.k),
            LayoutSku::Rrr => (d.k, d.n),
        };
        if (args.a.rows, args.a.cols) != (d.m, d.k) || (args.b.rows, args.b.cols) != (b_rows, b_cols)
            || (args.d.rows, args.d.cols) != (d.m, d.n)
        {
            return Err(Error::InvalidProblem("W8A8GemmPlan: operand shape does not match the descriptor"));
        }
        if d.epilogue.requires_bias() != args.bias.is_some() {
            return Err(Error::InvalidProblem("W8A8GemmPlan: bias must be given exactly for the Bias* epilogues"));
        }
        if args.beta != 0.0 && args.c.is_none() {
            return Err(Error::InvalidProblem("W8A8GemmPlan: beta != 0 needs C"));
        }
        let span = |rows: i32, cols: i32, ld: i64| -> i64 {
            if rows == 0 || cols == 0 { 0 } else { (rows as i64 - 1) * ld + cols as i64 }
        };
        let need = |have: usize, want: i64| -> Result<()> {
            if (have as i64) < want {
                Err(Error::BufferTooSmall { needed: want as usize, got: have })
            } else {
                Ok(())
            }
        };
        need(args.a.data.len(), span(d.m, d.k, args.a.ld))?;
        need(args.b.data.len(), span(b_rows, b_cols, args.b.ld))?;
        need(args.d.data.len(), span(d.m, d.n, args.d.ld))?;
        need(args.scale_a.data.len(), d.m as i64)?;
        need(args.scale_b.data.len(), d.n as i64)?;
        if let Some(bias) = &args.bias {
            need(bias.data.len(), d.n as i64)?;
        }
        if let Some(c) = &args.c {
            need(c.data.len(), span(d.m, d.n, c.ld))?;
        }
        let (c_ptr, ldc) = match &args.c {
            Some(c) => (c.data.as_raw().0 as *const c_void, c.ld),
            None => (core::ptr::null(), 0),
        };
        let code = unsafe {
            match d.layout {
                LayoutSku::Rcr => sys::baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement(
                    d.m, d.n, d.k, args.a.data.as_raw().0 as *const c_void, args.a.ld,
                    args.b.data.as_raw().0 as *const c_void, args.b.ld, c_ptr, ldc,
                    args.d.data.as_raw().0 as *const c_void, args.d.ld),
                LayoutSku::Rrr => sys::baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_can_implement(
                    d.m, d.n, d.k, args.a.data.as_raw().0 as *const c_void, args.a.ld,
                    args.b.data.as_raw().0 as *const c_void, args.b.ld, c_ptr, ldc,
                    args.d.data.as_raw().0 as *const c_void, args.d.ld),
            }
        };
        map_status(code, "W8A8GemmPlan::can_implement")
    }

    /// Asynchronous launch on `stream`; no allocation, no host synchronisation (graph-capture safe).
    pub fn run(&self, stream: &Stream, _workspace: Workspace<'_>, args: W8A8GemmArgs<'_>) -> Result<()> {
        self.can_implement(&args)?;
        let d = &self.desc;
        let a = args.a.data.as_raw().0 as *const c_void;
        let b = args.b.data.as_raw().0 as *const c_void;
        let out = args.d.data.as_raw().0 as *mut c_void;
        let sa = args.scale_a.data.as_raw().0 as *const c_void;
        let sb = args.scale_b.data.as_raw().0 as *const c_void;
        let (c_ptr, ldc) = match &args.c {
            Some(c) => (c.data.as_raw().0 as *const c_void, c.ld),
            None => (core::ptr::null(), 0),
        };
        let bias = args.bias.as_ref().map_or(core::ptr::null(), |v| v.data.as_raw().0 as *const c_void);
        let s = stream.as_raw() as *mut c_void;
        let code = unsafe {
            match (d.layout, d.epilogue) {
                (LayoutSku::Rcr, EpilogueKind::Identity) => sys::baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run(
                    d.m, d.n, d.k, a, args.a.ld, b, args.b.ld, c_ptr, ldc, out, args.d.ld, sa, sb,
                    args.alpha, args.beta, core::ptr::null_mut(), 0, s),
                (LayoutSku::Rrr, EpilogueKind::Identity) => sys::baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run(
                    d.m, d.n, d.k, a, args.a.ld, b, args.b.ld, c_ptr, ldc, out, args.d.ld, sa, sb,
                    args.alpha, args.beta, core::ptr::null_mut(), 0, s),
                (LayoutSku::Rcr, e) => sys::baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run(
                    d.m, d.n, d.k, a, args.a.ld, b, args.b.ld, c_ptr, ldc, out, args.d.ld, sa, sb,
                    sys::BARACUDA_Q_SCALE_PER_ROW_COL, bias, epilogue_code(e), args.alpha, args.beta,
                    core::ptr::null_mut(), 0, s),
                (LayoutSku::Rrr, e) => sys::baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_epilogue_run(
                    d.m, d.n, d.k, a, args.a.ld, b, args.b.ld, c_ptr, ldc, out, args.d.ld, sa, sb,
                    sys::BARACUDA_Q_SCALE_PER_ROW_COL, bias, epilogue_code(e), args.alpha, args.beta,
                    core::ptr::null_mut(), 0, s),
            }
        };
        map_status(code, "W8A8GemmPlan::run")
    }

    /// The same launch as a programmatic dependent of the kernel before it on `stream`: prologue and the first
    /// weight tiles are issued while that kernel finishes.  The caller asserts that it does not write `args.b`.
    pub fn run_dependent(&self, stream: &Stream, _workspace: Workspace<'_>, args: W8A8GemmArgs<'_>) -> Result<()> {
        self.can_implement(&args)?;
        let d = &self.desc;
        let (c_ptr, ldc) = match &args.c {
            Some(c) => (c.data.as_raw().0 as *const c_void, c.ld),
            None => (core::ptr::null(), 0),
        };
        let bias = args.bias.as_ref().map_or(core::ptr::null(), |v| v.data.as_raw().0 as *const c_void);
        let f = match d.layout {
            LayoutSku::Rcr => sys::baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_pdl_run,
            LayoutSku::Rrr => sys::baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_pdl_run,
        };
        let code = unsafe {
            f(d.m, d.n, d.k, args.a.data.as_raw().0 as *const c_void, args.a.ld, args.b.data.as_raw().0 as *const c_void,
              args.b.ld, c_ptr, ldc, args.d.data.as_raw().0 as *mut c_void, args.d.ld,
              args.scale_a.data.as_raw().0 as *const c_void, args.scale_b.data.as_raw().0 as *const c_void,
              sys::BARACUDA_Q_SCALE_PER_ROW_COL, bias, epilogue_code(d.epilogue), args.alpha, args.beta,
              core::ptr::null_mut(), 0, stream.as_raw() as *mut c_void)
        };
        map_status(code, "W8A8GemmPlan::run_dependent")
    }
}
