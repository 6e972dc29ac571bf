//! `ContractionKey` cells of the mixed-dtype contractions the sm_100a quantized kernels serve.
//!
//! The canonical accumulator lattice already maps `S8` to `I32` and everything else to `F32`
//! (`contraction_acc`, `structure_key.rs:647-657`), and `contraction_mp` gives `St` for both
//! (`structure_key.rs:666-671`): no operand is rounded on its way into the multiply.  What is
//! new is the OUTPUT coordinate: these cells store `Bf16` although lhs and rhs are 8-bit, which
//! the sk3 key (`wdt / acc / out / mp`) can express and the pre-sk3 key could not.
//!
//! Token forms (the trailing precision group of `StructureKey::to_token`, `structure_key.rs:2371-2388`):
//!   W8A8 -> bf16 :  `.../s8/i32/bf16/st`
//!   FP8  -> bf16 :  `.../e4m3/f32/bf16/st`
//! Not compiled in the environment this file was written in.

use crate::element::ElementKind;
use crate::structure_key::{ContractionKey, DivBucket, LayoutOrder, MpCode, SizeClass};

/// Storage order of the weight operand: `[N, K]` rows (the transposed-rhs class `derive_contraction`
/// reports for strides `[1, k]`, `structure_key.rs:694-732`) or canonical row-major `[K, N]`.
#[derive(Copy, Clone, Debug, Eq, PartialEq, Hash)]
pub enum WeightOrder {
    /// `[N, K]`, K contiguous — `LayoutSku::Rcr`.
    KContiguous,
    /// `[K, N]`, N contiguous — `LayoutSku::Rrr`.
    NContiguous,
}

fn rhs_order(w: WeightOrder) -> LayoutOrder {
    match w {
        WeightOrder::KContiguous => LayoutOrder::from_perm(&[1, 0]),
        WeightOrder::NContiguous => LayoutOrder::from_perm(&[0, 1]),
    }
}

fn k_div(k: i64) -> DivBucket {
    if k % 16 == 0 {
        DivBucket::Div16
    } else if k % 8 == 0 {
        DivBucket::Div8
    } else if k % 4 == 0 {
        DivBucket::Div4
    } else if k % 2 == 0 {
        DivBucket::Div2
    } else {
        DivBucket::Any
    }
}

/// s8 x s8 -> i32 accumulate -> bf16 store (per-token x per-channel dequant fused in the epilogue).
pub fn w8a8_bf16_cell(m: i64, n: i64, k: i64, weight: WeightOrder, batch: Option<i64>) -> ContractionKey {
    ContractionKey {
        m: SizeClass::of(m),
        n: SizeClass::of(n),
        k: SizeClass::of(k),
        k_div: k_div(k),
        batch: batch.map(SizeClass::of),
        lhs_order: LayoutOrder::from_perm(&[0, 1]),
        rhs_order: rhs_order(weight),
        wdt: ElementKind::S8,
        acc: ElementKind::I32,
        out: ElementKind::Bf16,
        mp: MpCode::St,
    }
}

/// e4m3 x e4m3 -> f32 accumulate -> bf16 store (f32 scales fused in the epilogue).
pub fn fp8_e4m3_bf16_cell(m: i64, n: i64, k: i64, weight: WeightOrder, batch: Option<i64>) -> ContractionKey {
    ContractionKey {
        m: SizeClass::of(m),
        n: SizeClass::of(n),
        k: SizeClass::of(k),
        k_div: k_div(k),
        batch: batch.map(SizeClass::of),
        lhs_order: LayoutOrder::from_perm(&[0, 1]),
        rhs_order: rhs_order(weight),
        wdt: ElementKind::Fp8E4M3,
        acc: ElementKind::F32,
        out: ElementKind::Bf16,
        mp: MpCode::St,
    }
}

/// `true` for the cells the decode GEMV serves: the skinny regime (`SizeClass::Tiny`, M <= 8).
pub fn is_decode_cell(key: &ContractionKey) -> bool {
    matches!(key.m, SizeClass::Tiny) && key.wdt == ElementKind::S8 && key.out == ElementKind::Bf16
}

#[cfg(test)]
mod tests {
    use super::*;

    #[test]
    fn mixed_cells_differ_from_the_homogeneous_ones_only_in_out() {
        let c = w8a8_bf16_cell(8192, 28672, 4096, WeightOrder::KContiguous, None);
        assert_eq!((c.wdt, c.acc, c.out, c.mp), (ElementKind::S8, ElementKind::I32, ElementKind::Bf16, MpCode::St));
        let f = fp8_e4m3_bf16_cell(8192, 28672, 8192, WeightOrder::KContiguous, None);
        assert_eq!((f.wdt, f.acc, f.out, f.mp), (ElementKind::Fp8E4M3, ElementKind::F32, ElementKind::Bf16, MpCode::St));
        assert_ne!(c, f);
    }

    #[test]
    fn decode_shapes_land_in_the_tiny_m_class() {
        assert!(is_decode_cell(&w8a8_bf16_cell(1, 14336, 4096, WeightOrder::NContiguous, None)));
        assert!(is_decode_cell(&w8a8_bf16_cell(8, 14336, 4096, WeightOrder::KContiguous, None)));
        assert!(!is_decode_cell(&w8a8_bf16_cell(512, 14336, 4096, WeightOrder::KContiguous, None)));
    }
}
