//! Dispatch table of the sm_100a quantized contractions: `ContractionKey` cell -> plan family and the
//! flat C symbols a table-driven caller (Fuel binds symbols from a table, see the note in
//! `kernels/gemm/gemv_dense.cu:32-36`) resolves for it.
//!
//! A row matches a key when the precision coordinates (`wdt / acc / out / mp`) and the weight order
//! agree and the M class is in the row's regime; the first matching row wins.  Not compiled in the
//! environment this file was written in.

use baracuda_kernel_vocab::contraction_cells_sm100a::WeightOrder;
use baracuda_kernel_vocab::element::ElementKind;
use baracuda_kernel_vocab::layout::{ArchSku, LayoutSku};
use baracuda_kernel_vocab::structure_key::{ContractionKey, LayoutOrder, MpCode, SizeClass};

/// Plan family that serves a row.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub enum Sm100aPlanFamily {
    /// `GemvQ8Plan` (M <= 8).
    GemvQ8,
    /// `W8A8GemmPlan`.
    W8A8Gemm,
    /// `Fp8ScaledGemmPlan`.
    Fp8ScaledGemm,
}

/// One table row.
#[derive(Copy, Clone, Debug)]
pub struct Sm100aDispatchEntry {
    /// Weight dtype coordinate.
    pub wdt: ElementKind,
    /// Accumulator coordinate.
    pub acc: ElementKind,
    /// Output dtype coordinate.
    pub out: ElementKind,
    /// Math-precision coordinate.
    pub mp: MpCode,
    /// Weight storage order.
    pub weight: WeightOrder,
    /// `true`: only the skinny regime (`SizeClass::Tiny`).
    pub decode_only: bool,
    /// Plan family.
    pub family: Sm100aPlanFamily,
    /// Layout the plan's descriptor takes.
    pub layout: LayoutSku,
    /// Architecture tag of the SKU.
    pub arch: ArchSku,
    /// `*_run` symbol.
    pub run: &'static str,
    /// `*_can_implement` symbol.
    pub can_implement: &'static str,
    /// `*_workspace_size` symbol.
    pub workspace_size: &'static str,
}

macro_rules! entry {
    ($wdt:ident, $acc:ident, $weight:ident, $decode:expr, $family:ident, $layout:ident, $base:literal) => {
        Sm100aDispatchEntry {
            wdt: ElementKind::$wdt,
            acc: ElementKind::$acc,
            out: ElementKind::Bf16,
            mp: MpCode::St,
            weight: WeightOrder::$weight,
            decode_only: $decode,
            family: Sm100aPlanFamily::$family,
            layout: LayoutSku::$layout,
            arch: ArchSku::Sm100a,
            run: concat!($base, "_run"),
            can_implement: concat!($base, "_can_implement"),
            workspace_size: concat!($base, "_workspace_size"),
        }
    };
}

/// The table. Decode rows come first so that M <= 8 never lands on a 128-row tensor-core tile.
pub static SM100A_Q_DISPATCH: &[Sm100aDispatchEntry] = &[
    entry!(S8, I32, KContiguous, true, GemvQ8, Rcr, "baracuda_kernels_gemv_q8_m1_bf16_sm100a"),
    entry!(S8, I32, NContiguous, true, GemvQ8, Rrr, "baracuda_kernels_gemv_q8_m1_bf16_sm100a"),
    entry!(S8, I32, KContiguous, false, W8A8Gemm, Rcr, "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a"),
    entry!(S8, I32, NContiguous, false, W8A8Gemm, Rrr, "baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a"),
    entry!(Fp8E4M3, F32, KContiguous, false, Fp8ScaledGemm, Rcr, "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a"),
    entry!(Fp8E4M3, F32, NContiguous, false, Fp8ScaledGemm, Rrr, "baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a"),
];

fn weight_order_of(rhs: &LayoutOrder) -> Option<WeightOrder> {
    match rhs.perm() {
        [0, 1] => Some(WeightOrder::NContiguous),
        [1, 0] => Some(WeightOrder::KContiguous),
        _ => None,
    }
}

/// The row that serves `key`, or `None` (batched lhs permutations, other dtypes, other outputs).
pub fn lookup(key: &ContractionKey) -> Option<&'static Sm100aDispatchEntry> {
    if !key.lhs_order.is_identity() {
        return None;
    }
    let weight = weight_order_of(&key.rhs_order)?;
    let decode = matches!(key.m, SizeClass::Tiny);
    SM100A_Q_DISPATCH.iter().find(|e| {
        e.wdt == key.wdt && e.acc == key.acc && e.out == key.out && e.mp == key.mp && e.weight == weight
            && (!e.decode_only || decode)
            && (e.family != Sm100aPlanFamily::GemvQ8 || key.batch.is_none() || decode)
    })
}

#[cfg(test)]
mod tests {
    use super::*;
    use baracuda_kernel_vocab::contraction_cells_sm100a::{fp8_e4m3_bf16_cell, w8a8_bf16_cell};

    #[test]
    fn decode_and_prefill_cells_reach_different_families() {
        let dec = lookup(&w8a8_bf16_cell(1, 14336, 4096, WeightOrder::NContiguous, None)).unwrap();
        assert_eq!(dec.family, Sm100aPlanFamily::GemvQ8);
        assert_eq!(dec.layout, LayoutSku::Rrr);
        let pre = lookup(&w8a8_bf16_cell(8192, 28672, 4096, WeightOrder::KContiguous, None)).unwrap();
        assert_eq!(pre.family, Sm100aPlanFamily::W8A8Gemm);
        assert_eq!(pre.run, "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run");
        let fp8 = lookup(&fp8_e4m3_bf16_cell(8192, 28672, 8192, WeightOrder::KContiguous, None)).unwrap();
        assert_eq!(fp8.family, Sm100aPlanFamily::Fp8ScaledGemm);
    }
}
