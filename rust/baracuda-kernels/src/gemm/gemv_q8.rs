//! `GemvQ8Plan` — the capture-safe decode GEMV of `GemvDensePlan` (`gemm/gemv_dense.rs:48-412`) for int8
//! weights with the W8A8 dequant fused, m = 1 (and the skinny extension m <= 8), sm_100a.
//!
//! ```text
//! D[g, r, j] = bf16( alpha * ((scale_a[g, r] * scale_b[g, j]) * (float)sum_k A[g, r, k] * B[g, k, j]) + beta * D[g, r, j] )
//! ```
//!
//! Weight layouts: `LayoutSku::Rrr` (row-major `[K, N]`, the reference GEMV's only layout; needs the
//! caller's scratch, see `workspace_size`) and `LayoutSku::Rcr` (`[N, K]`, K contiguous: the weight of a
//! `QuantizedLinearPlan`, no scratch).  `stride_b == 0` broadcasts the weights over batch slots.
//! `run_dependent` selects the `*_pdl_run` symbol.  Not compiled in the environment this file was written in.

use core::ffi::c_void;

use baracuda_cutlass::{Error, Result};
use baracuda_driver::Stream;
use baracuda_kernels_sys as sys;
use baracuda_kernels_types::{
    ArchSku, BackendKind, ElementKind, KernelSku, LayoutSku, MathPrecision, MatrixMut, MatrixRef, OpCategory,
    PlanPreference, PrecisionGuarantee, VectorRef, Workspace, S8,
};
use half::bf16;

use super::w8a8_gemm::map_status;

/// Category-local op discriminant of this family inside `OpCategory::Gemm`.
pub const OP_GEMV_Q8: u16 = 0x0803;

/// `GemvDenseDescriptor` with the weight layout added; `m` may be 1..=8.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub struct GemvQ8Descriptor {
    /// Activation rows (decode batch folded into M), 1..=8.
    pub m: i32,
    /// Output columns.
    pub n: i32,
    /// Reduction depth; at most 131 071.
    pub k: i32,
    /// Batch slots (strided).
    pub batch: i32,
    /// `Rrr`: `[K, N]`; `Rcr`: `[N, K]`.
    pub layout: LayoutSku,
}

/// `GemvDenseArgs` plus the two scale vectors.
#[derive(Debug)]
pub struct GemvQ8Args<'a> {
    /// `[m, K]` int8 activations of slot 0.
    pub a: MatrixRef<'a, S8>,
    /// Elements between consecutive slots of `a`.
    pub stride_a: i64,
    /// Weights of slot 0 in the descriptor's layout.
    pub b: MatrixRef<'a, S8>,
    /// Elements between consecutive slots of `b`; 0 broadcasts one weight matrix.
    pub stride_b: i64,
    /// Per-token scales `f32[m]` of slot 0.
    pub scale_a: VectorRef<'a, f32>,
    /// Elements between consecutive slots of `scale_a`.
    pub stride_scale_a: i64,
    /// Per-channel scales `f32[N]` of slot 0.
    pub scale_b: VectorRef<'a, f32>,
    /// Elements between consecutive slots of `scale_b`.
    pub stride_scale_b: i64,
    /// `[m, N]` bf16 output of slot 0.
    pub d: MatrixMut<'a, bf16>,
    /// Elements between consecutive slots of `d`; non-zero when `batch > 1`.
    pub stride_d: i64,
    /// Multiplier on the dequantised sum.
    pub alpha: f32,
    /// Multiplier on the existing contents of `d`.
    pub beta: f32,
}

/// The plan.
#[derive(Debug)]
pub struct GemvQ8Plan {
    desc: GemvQ8Descriptor,
    sku: KernelSku,
}

fn layout_code(l: LayoutSku) -> i32 {
    match l {
        LayoutSku::Rrr => sys::BARACUDA_Q_LAYOUT_RRR,
        LayoutSku::Rcr => sys::BARACUDA_Q_LAYOUT_RCR,
    }
}

impl GemvQ8Plan {
    /// Validates the descriptor and the workspace budget; bespoke-only.
    pub fn select(_stream: &Stream, desc: &GemvQ8Descriptor, pref: PlanPreference) -> Result<Self> {
        if desc.m < 0 || desc.n < 0 || desc.k < 0 || desc.batch < 0 {
            return Err(Error::InvalidProblem("GemvQ8Plan: M, N, K, batch must be non-negative"));
        }
        if desc.m > 8 {
            return Err(Error::InvalidProblem("GemvQ8Plan: m <= 8; larger m belongs on W8A8GemmPlan"));
        }
        match pref.prefer_backend {
            None | Some(BackendKind::Bespoke) => {}
            Some(_) => return Err(Error::Unsupported("GemvQ8Plan: bespoke-kernel-backed only")),
        }
        let plan = Self {
            desc: *desc,
            sku: KernelSku {
                category: OpCategory::Gemm,
                op: OP_GEMV_Q8,
                element: ElementKind::S8,
                aux_element: Some(ElementKind::Bf16),
                layout: Some(desc.layout),
                epilogue: None,
                arch: ArchSku::Sm100a,
                backend: BackendKind::Bespoke,
                precision_guarantee: PrecisionGuarantee {
                    math_precision: MathPrecision::Int8,
                    accumulator: ElementKind::I32,
                    deterministic: true,
                    bit_stable_on_same_hardware: true,
                },
            },
        };
        if plan.workspace_size() > pref.max_workspace_bytes {
            return Err(Error::Unsupported("GemvQ8Plan: workspace budget too small for this shape"));
        }
        Ok(plan)
    }

    /// Selection identity.
    pub fn sku(&self) -> KernelSku {
        self.sku
    }

    /// Integer accumulation: exact.
    pub fn precision_guarantee(&self) -> PrecisionGuarantee {
        self.sku.precision_guarantee
    }

    /// Scratch for the row-major weight layout (partial rows of the K split); 0 for `Rcr`.
    pub fn workspace_size(&self) -> usize {
        let d = &self.desc;
        unsafe { sys::baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(d.m, d.n, d.k, d.batch, layout_code(d.layout)) }
    }

    /// The rejection table of `gemv_validate` (`gemv_dense.cu:101-122`) widened to m <= 8 and the second
    /// layout, plus the buffer-length checks this typed layer owns.
    pub fn can_implement(&self, args: &GemvQ8Args<'_>) -> Result<()> {
        let d = &self.desc;
        let code = unsafe {
            sys::baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement(
                d.m, d.n, d.k, d.batch, layout_code(d.layout), args.a.ld, args.b.ld, args.d.ld,
                args.stride_a, args.stride_b, args.stride_d)
        };
        map_status(code, "GemvQ8Plan::can_implement")?;
        if args.stride_a < 0 || args.stride_b < 0 || args.stride_d < 0 || args.stride_scale_a < 0 || args.stride_scale_b < 0 {
            return Err(Error::InvalidProblem("GemvQ8Plan: negative batch strides walk before the buffer base"));
        }
        if d.m == 0 || d.n == 0 || d.batch == 0 {
            return Ok(());
        }
        let last = (d.batch as i64 - 1).max(0);
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
        let (b_rows, b_cols) = match d.layout {
            LayoutSku::Rrr => (d.k, d.n),
            LayoutSku::Rcr => (d.n, d.k),
        };
        need(args.a.data.len(), last * args.stride_a + span(d.m, d.k, args.a.ld))?;
        need(args.b.data.len(), last * args.stride_b + span(b_rows, b_cols, args.b.ld))?;
        need(args.d.data.len(), last * args.stride_d + span(d.m, d.n, args.d.ld))?;
        need(args.scale_a.data.len(), last * args.stride_scale_a + d.m as i64)?;
        need(args.scale_b.data.len(), last * args.stride_scale_b + d.n as i64)
    }

    /// Plain launch.
    pub fn run(&self, stream: &Stream, workspace: Workspace<'_>, args: GemvQ8Args<'_>) -> Result<()> {
        self.launch(stream, workspace, args, false)
    }

    /// Launch under programmatic dependent launch: the kernel prefetches weights while the previous kernel
    /// of `stream` drains. The caller promises that kernel does not write `b`.
    pub fn run_dependent(&self, stream: &Stream, workspace: Workspace<'_>, args: GemvQ8Args<'_>) -> Result<()> {
        self.launch(stream, workspace, args, true)
    }

    fn launch(&self, stream: &Stream, workspace: Workspace<'_>, args: GemvQ8Args<'_>, dependent: bool) -> Result<()> {
        self.can_implement(&args)?;
        let d = &self.desc;
        let need = self.workspace_size();
        let (ws_ptr, ws_bytes) = match workspace {
            Workspace::None => (core::ptr::null_mut(), 0usize),
            Workspace::Borrowed(s) => (s.as_raw().0 as *mut c_void, s.len()),
        };
        if ws_bytes < need {
            return Err(Error::WorkspaceTooSmall { needed: need, got: ws_bytes });
        }
        let f = if dependent {
            sys::baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run
        } else {
            sys::baracuda_kernels_gemv_q8_m1_bf16_sm100a_run
        };
        let code = unsafe {
            f(d.m, d.n, d.k, d.batch, layout_code(d.layout), args.alpha, args.beta,
              args.a.data.as_raw().0 as *const c_void, args.a.ld, args.stride_a,
              args.b.data.as_raw().0 as *const c_void, args.b.ld, args.stride_b,
              args.scale_a.data.as_raw().0 as *const c_void, args.stride_scale_a,
              args.scale_b.data.as_raw().0 as *const c_void, args.stride_scale_b,
              args.d.data.as_raw().0 as *mut c_void, args.d.ld, args.stride_d,
              ws_ptr, ws_bytes, stream.as_raw() as *mut c_void)
        };
        map_status(code, "GemvQ8Plan::run")
    }
}
