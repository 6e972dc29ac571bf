"""Regenerates the committed fixtures of tests/golden/.

reference_known_answers.json — inputs and expected values transcribed from the
  reference's own tests (file:line beside each), used to pin the CPU oracle.
w8a8_fp8_cases.npz — small seeded W8A8 / FP8 problems in the benchmark's value
  distributions, with the oracle's outputs frozen: the GPU parity tests compare
  against these bytes, and a CPU test re-derives them to catch oracle drift.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import pyoracle as orc  # noqa: E402


def known_answers() -> dict:
    return {
        "matmul_identity": {  # crates/baracuda-kernelgen/src/kiss_ref_diff.rs:1170-1192
            "lhs": [1, 2, 3, 4, 5, 6], "rhs": [7, 8, 9, 10, 11, 12], "shape_mkn": [2, 3, 2],
            "expect": [58, 64, 139, 154]},
        "matmul_relu": {  # kiss_ref_diff.rs:1195-1216
            "lhs": [1, -3], "rhs": [2, 5, 4, 1], "shape_mkn": [1, 2, 2], "expect": [0, 2]},
        "matmul_bias_relu": {  # kiss_ref_diff.rs:1298-1320
            "lhs": [1, 2], "rhs": [3, 4, 5, 6], "bias": [-100, 1], "shape_mkn": [1, 2, 2], "expect": [0, 17]},
        "batched_matmul": {  # kiss_ref_diff.rs:1323-1345
            "lhs": [1, 2, 3, 4], "rhs": [1, 2, 3, 4, 5, 6, 7, 8], "shape_bmkn": [2, 1, 2, 2],
            "expect": [7, 10, 43, 50]},
        "quantized_linear_w8a8_f32_basic": {  # crates/baracuda-kernels/tests/quantized_linear_smoke.rs:82-101
            "m": 2, "c_out": 3, "k": 8,
            "activation": [0.5, -0.3, 0.8, 1.2, -0.4, 0.6, 0.9, -0.7,
                           4.0, -2.5, 1.8, -3.2, 2.1, -1.4, 0.9, 3.6],
            "weight": [0.1, -0.2, 0.15, 0.05, -0.1, 0.08, -0.12, 0.18,
                       0.4, 0.3, -0.5, 0.6, -0.45, 0.55, -0.35, 0.4,
                       1.2, -0.8, 1.0, 0.9, -1.1, 0.7, 1.3, -0.95],
            "tolerance_rel_vs_full_precision": 0.03},
        "int8_pattern": {  # crates/baracuda-kernels/tests/int8_rrr_smoke.rs:159-172, 442-500
            "a": "((7*i) % 15) - 7", "b": "((11*i) % 13) - 6", "alpha": 0.125,
            "shapes_mnk": [[64, 64, 32], [128, 128, 128], [256, 128, 64], [100, 70, 50]]},
        "fp8_pattern": {  # crates/baracuda-kernels/tests/fp8_e4m3_rcr_smoke.rs:113-127, 225-247
            "a": "(((5*i) % 13) - 6) * 0.125", "b": "(((7*i) % 11) - 5) * 0.125", "alpha": 0.25,
            "shapes_mnk": [[64, 64, 32], [128, 128, 128], [256, 128, 64], [100, 70, 50]]},
    }


def seeded_cases() -> dict:
    out = {}
    rng = np.random.default_rng(1234)
    for tag, (m, k, n) in {"c0s": (64, 256, 96), "ragged": (37, 80, 53)}.items():
        a = rng.standard_normal((m, k)).astype(np.float32)          # activations N(0,1)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)  # weights N(0,0.02), stored [N,K]
        aq, sa = orc.quantize_rows_s8(a)
        wq, sb = orc.quantize_rows_s8(w)
        acc = orc.gemm_s8_s32(aq, wq, orc.RCR, m, n, k)
        out[f"{tag}_a_f32"], out[f"{tag}_b_f32"] = a, w
        out[f"{tag}_a_q"], out[f"{tag}_b_q"], out[f"{tag}_sa"], out[f"{tag}_sb"] = aq, wq, sa, sb
        out[f"{tag}_acc"] = acc
        out[f"{tag}_out_bf16"] = orc.dequant_s32_bf16(acc, sa, sb)
    m, k, n = 64, 128, 72
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    aq, sa = orc.quantize_rows_e4m3(a)
    wq, sb = orc.quantize_rows_e4m3(w)
    acc = orc.gemm_e4m3_f32(aq, wq, orc.RCR, m, n, k)
    out["fp8_a_f32"], out["fp8_b_f32"] = a, w
    out["fp8_a_q"], out["fp8_b_q"], out["fp8_sa"], out["fp8_sb"] = aq, wq, sa, sb
    out["fp8_acc"] = acc
    out["fp8_out_bf16"] = orc.scale_f32_bf16(acc, sa, sb)
    return out


if __name__ == "__main__":
    (HERE / "reference_known_answers.json").write_text(json.dumps(known_answers(), indent=1) + "\n")
    np.savez_compressed(HERE / "w8a8_fp8_cases.npz", **seeded_cases())
    print("wrote", sorted(p.name for p in HERE.iterdir()))
