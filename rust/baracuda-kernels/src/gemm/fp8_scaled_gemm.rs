//! `Fp8ScaledGemmPlan` — e4m3 x e4m3 -> f32 on `tcgen05.mma kind::f8f6f4` with f32 scales fused into
//! a bf16 store (sm_100a).
//!
//! The reference's `Fp8GemmPlan` (`gemm/fp8_gemm.rs:36-741`) stores e4m3 with a scalar alpha; serving
//! FP8 linear layers needs the dequantised result, so this plan carries the scales:
//!
//! ```text
//! D[m, n] = bf16( act( alpha * ((sa * sb) * acc[m, n]) + beta * C[m, n] + bias[n] ) )
//! (sa, sb) = (scale_a[0], scale_b[0])   for ScaleMode::PerTensor
//!          = (scale_a[m], scale_b[n])   for ScaleMode::PerRowCol
//! ```
//!
//! Not compiled in the environment this file was written in.

use core::ffi::c_void;

use baracuda_cutlass::{Error, Result};
use baracuda_driver::Stream;
use baracuda_kernels_sys as sys;
use baracuda_kernels_types::{
    ArchSku, BackendKind, ElementKind, EpilogueKind, Fp8E4M3, KernelSku, LayoutSku, MathPrecision, MatrixMut,
    MatrixRef, OpCategory, PlanPreference, PrecisionGuarantee, VectorRef, Workspace,
};
use half::bf16;

use super::w8a8_gemm::map_status;

/// Category-local op discriminant of this family inside `OpCategory::Gemm`.
pub const OP_FP8_SCALED_GEMM: u16 = 0x0802;

/// Which scales the launch reads.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub enum ScaleMode {
    /// One f32 each (the per-tensor recipe: scale = absmax / 448).
    PerTensor,
    /// `f32[M]` per token and `f32[N]` per output channel.
    PerRowCol,
}

/// Shape, weight layout, epilogue chain and scale mode.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub struct Fp8ScaledGemmDescriptor {
    /// Rows of the activation and of the output.
    pub m: i32,
    /// Output channels.
    pub n: i32,
    /// Reduction depth.
    pub k: i32,
    /// Weight storage: `Rcr` = `[N, K]`, `Rrr` = `[K, N]`.
    pub layout: LayoutSku,
    /// `Identity` or one of the `Bias*` chains.
    pub epilogue: EpilogueKind,
    /// Per tensor, or per row and per column.
    pub scale_mode: ScaleMode,
}

/// Device views of one launch.
#[derive(Debug)]
pub struct Fp8ScaledGemmArgs<'a> {
    /// e4m3 activations, row-major `[M, K]`.
    pub a: MatrixRef<'a, Fp8E4M3>,
    /// e4m3 weights in the descriptor's layout.
    pub b: MatrixRef<'a, Fp8E4M3>,
    /// Optional residual (bf16, may alias `d`), read when `beta != 0`.
    pub c: Option<MatrixRef<'a, bf16>>,
    /// Output, row-major `[M, N]`.
    pub d: MatrixMut<'a, bf16>,
    /// 1 or M floats.
    pub scale_a: VectorRef<'a, f32>,
    /// 1 or N floats.
    pub scale_b: VectorRef<'a, f32>,
    /// `f32[N]` for the `Bias*` epilogues.
    pub bias: Option<VectorRef<'a, f32>>,
    /// Multiplier on the scaled accumulator.
    pub alpha: f32,
    /// Multiplier on `c`.
    pub beta: f32,
}

/// The plan.
#[derive(Debug)]
pub struct Fp8ScaledGemmPlan {
    desc: Fp8ScaledGemmDescriptor,
    sku: KernelSku,
}

impl Fp8ScaledGemmPlan {
    /// Validates the descriptor once and fixes the SKU.
    pub fn select(_stream: &Stream, desc: &Fp8ScaledGemmDescriptor, pref: PlanPreference) -> Result<Self> {
        if desc.m < 0 || desc.n < 0 || desc.k < 0 {
            return Err(Error::InvalidProblem("Fp8ScaledGemmPlan: M, N, K must be non-negative"));
        }
        match pref.prefer_backend {
            None | Some(BackendKind::Bespoke) => {}
            Some(_) => return Err(Error::Unsupported("Fp8ScaledGemmPlan: bespoke-kernel-backed only")),
        }
        let sku = KernelSku {
            category: OpCategory::Gemm,
            op: OP_FP8_SCALED_GEMM,
            element: ElementKind::Fp8E4M3,
            aux_element: Some(ElementKind::Bf16),
            layout: Some(desc.layout),
            epilogue: Some(desc.epilogue),
            arch: ArchSku::Sm100a,
            backend: BackendKind::Bespoke,
            // one CTA pair owns one output tile and accumulates its K blocks in a fixed order
            precision_guarantee: PrecisionGuarantee {
                math_precision: MathPrecision::Fp8E4M3,
                accumulator: ElementKind::F32,
                deterministic: true,
                bit_stable_on_same_hardware: true,
            },
        };
        Ok(Self { desc: *desc, sku })
    }

    /// Selection identity.
    pub fn sku(&self) -> KernelSku {
        self.sku
    }

    /// f32 accumulation in a fixed order per tile.
    pub fn precision_guarantee(&self) -> PrecisionGuarantee {
        self.sku.precision_guarantee
    }

    /// No scratch.
    pub fn workspace_size(&self) -> usize {
        0
    }

    /// Shape and buffer-length checks, then the C side's `can_implement`.
    pub fn can_implement(&self, args: &Fp8ScaledGemmArgs<'_>) -> Result<()> {
        let d = &self.desc;
        let (b_rows, b_cols) = match d.layout {
            LayoutSku::Rcr => (d.n, d.k),
            LayoutSku::Rrr => (d.k, d.n),
        };
        if (args.a.rows, args.a.cols) != (d.m, d.k) || (args.b.rows, args.b.cols) != (b_rows, b_cols)
            || (args.d.rows, args.d.cols) != (d.m, d.n)
        {
            return Err(Error::InvalidProblem("Fp8ScaledGemmPlan: operand shape does not match the descriptor"));
        }
        if d.epilogue.requires_bias() != args.bias.is_some() {
            return Err(Error::InvalidProblem("Fp8ScaledGemmPlan: bias must be given exactly for the Bias* epilogues"));
        }
        if args.beta != 0.0 && args.c.is_none() {
            return Err(Error::InvalidProblem("Fp8ScaledGemmPlan: beta != 0 needs C"));
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
        let (na, nb) = match d.scale_mode {
            ScaleMode::PerTensor => (1, 1),
            ScaleMode::PerRowCol => (d.m as i64, d.n as i64),
        };
        need(args.a.data.len(), span(d.m, d.k, args.a.ld))?;
        need(args.b.data.len(), span(b_rows, b_cols, args.b.ld))?;
        need(args.d.data.len(), span(d.m, d.n, args.d.ld))?;
        need(args.scale_a.data.len(), na)?;
        need(args.scale_b.data.len(), nb)?;
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
                LayoutSku::Rcr => sys::baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement(
                    d.m, d.n, d.k, args.a.data.as_raw().0 as *const c_void, args.a.ld,
                    args.b.data.as_raw().0 as *const c_void, args.b.ld, c_ptr, ldc,
                    args.d.data.as_raw().0 as *const c_void, args.d.ld),
                LayoutSku::Rrr => sys::baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_can_implement(
                    d.m, d.n, d.k, args.a.data.as_raw().0 as *const c_void, args.a.ld,
                    args.b.data.as_raw().0 as *const c_void, args.b.ld, c_ptr, ldc,
                    args.d.data.as_raw().0 as *const c_void, args.d.ld),
            }
        };
        map_status(code, "Fp8ScaledGemmPlan::can_implement")
    }

    /// Asynchronous launch on `stream`; graph-capture safe.
    pub fn run(&self, stream: &Stream, workspace: Workspace<'_>, args: Fp8ScaledGemmArgs<'_>) -> Result<()> {
        self.launch(stream, workspace, args, false)
    }

    /// The same launch as a programmatic dependent of the kernel before it on `stream`: prologue and the first
    /// weight tiles are issued while that kernel finishes.  The caller asserts that it does not write `args.b`.
    pub fn run_dependent(&self, stream: &Stream, workspace: Workspace<'_>, args: Fp8ScaledGemmArgs<'_>) -> Result<()> {
        self.launch(stream, workspace, args, true)
    }

    fn launch(&self, stream: &Stream, _workspace: Workspace<'_>, args: Fp8ScaledGemmArgs<'_>, dependent: bool) -> Result<()> {
        self.can_implement(&args)?;
        let d = &self.desc;
        let mode = match d.scale_mode {
            ScaleMode::PerTensor => sys::BARACUDA_Q_SCALE_PER_TENSOR,
            ScaleMode::PerRowCol => sys::BARACUDA_Q_SCALE_PER_ROW_COL,
        };
        let epi = match d.epilogue {
            EpilogueKind::Identity => 0,
            EpilogueKind::Bias => 1,
            EpilogueKind::BiasRelu => 2,
            EpilogueKind::BiasGelu => 3,
            EpilogueKind::BiasSilu => 4,
        };
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
        // the four symbols share one signature
        let f = match (d.layout, dependent) {
            (LayoutSku::Rcr, false) => sys::baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_epilogue_run,
            (LayoutSku::Rrr, false) => sys::baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_epilogue_run,
            (LayoutSku::Rcr, true) => sys::baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_pdl_run,
            (LayoutSku::Rrr, true) => sys::baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_pdl_run,
        };
        let code = unsafe {
            f(d.m, d.n, d.k, a, args.a.ld, b, args.b.ld, c_ptr, ldc, out, args.d.ld, sa, sb, mode, bias, epi,
              args.alpha, args.beta, core::ptr::null_mut(), 0, s)
        };
        map_status(code, if dependent { "Fp8ScaledGemmPlan::run_dependent" } else { "Fp8ScaledGemmPlan::run" })
    }
}
