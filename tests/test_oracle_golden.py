"""Pins the CPU oracle against the reference's own known-answer tests.

Every case below restates a test (inputs and expected outputs) that lives in
the reference tree; the file:line of each is in the docstring.  If these pass,
the oracle's contraction, codecs, quantizers and W8A8 formula compute what the
reference's CPU code computes on the same inputs.
"""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_matmul_identity(oracle):
    """crates/baracuda-kernelgen/src/kiss_ref_diff.rs:1170-1192."""
    out = oracle.contraction(oracle.F32, [1, 2, 3, 4, 5, 6], (0, 3, 1), [7, 8, 9, 10, 11, 12], (0, 2, 1), (1, 2, 2, 3))
    assert out.tolist() == [58.0, 64.0, 139.0, 154.0]


def test_matmul_relu_epilogue(oracle):
    """kiss_ref_diff.rs:1195-1216: raw [-10, 2] -> relu -> [0, 2]."""
    out = oracle.contraction(oracle.F32, [1, -3], (0, 2, 1), [2, 5, 4, 1], (0, 2, 1), (1, 1, 2, 2),
                             epilogue=oracle.EPI_RELU)
    assert out.tolist() == [0.0, 2.0]


def test_matmul_bias_relu(oracle):
    """kiss_ref_diff.rs:1298-1320: [-87, 17] -> relu -> [0, 17]."""
    out = oracle.contraction(oracle.F32, [1, 2], (0, 2, 1), [3, 4, 5, 6], (0, 2, 1), (1, 1, 2, 2),
                             bias=[-100.0, 1.0], epilogue=oracle.EPI_BIAS_RELU)
    assert out.tolist() == [0.0, 17.0]


def test_batched_matmul(oracle):
    """kiss_ref_diff.rs:1323-1345: [2,1,2]·[2,2,2] -> [7,10,43,50]."""
    out = oracle.contraction(oracle.F32, [1, 2, 3, 4], (2, 2, 1), [1, 2, 3, 4, 5, 6, 7, 8], (4, 2, 1), (2, 1, 2, 2))
    assert out.tolist() == [7.0, 10.0, 43.0, 50.0]


def test_transposed_rhs_by_physical_strides(oracle):
    """crates/baracuda-kernelgen/src/oracle.rs:2433-2472: rhs stored [N,K], strides [1,k]."""
    m, k, n = 2, 3, 2
    lhs = [1., 2., 3., 4., 5., 6.]
    rhs_phys = [10., 12., 14., 11., 13., 15.]
    out = oracle.contraction(oracle.F32, lhs, (0, k, 1), rhs_phys, (0, 1, k), (1, m, n, k))
    lhs_l = np.array(lhs, dtype=np.float32).reshape(m, k)
    rhs_l = np.array([[10., 11.], [12., 13.], [14., 15.]], dtype=np.float32)
    assert out.tolist() == (lhs_l @ rhs_l).ravel().tolist()


@pytest.mark.parametrize("batched", [False, True])
@pytest.mark.parametrize("lhs_t", [False, True])
@pytest.mark.parametrize("rhs_t", [False, True])
def test_layout_batch_matrix(oracle, batched, lhs_t, rhs_t):
    """oracle.rs:2567-2668: {batched} x {lhs^T} x {rhs^T}, data b*100+idx+1."""
    m, k, n = 2, 3, 2
    bdim = 2 if batched else 1
    lhs_log = [np.array([bi * 100 + i + 1 for i in range(m * k)], dtype=np.float32).reshape(m, k) for bi in range(bdim)]
    rhs_log = [np.array([bi * 100 + i + 1 for i in range(k * n)], dtype=np.float32).reshape(k, n) for bi in range(bdim)]

    def phys(mats, rows, cols, transposed):
        if transposed:
            return np.concatenate([x.T.ravel() for x in mats]), (rows * cols, 1, rows)
        return np.concatenate([x.ravel() for x in mats]), (rows * cols, cols, 1)

    lp, ls = phys(lhs_log, m, k, lhs_t)
    rp, rs = phys(rhs_log, k, n, rhs_t)
    out = oracle.contraction(oracle.F32, lp, ls, rp, rs, (bdim, m, n, k))
    want = np.concatenate([(lhs_log[b] @ rhs_log[b]).ravel() for b in range(bdim)])
    assert out.tolist() == want.tolist()


def test_bf16_codec(oracle):
    """oracle.rs:2393-2410 plus the RNE rule of oracle.rs:397-404, against torch's bf16 cast."""
    assert oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(np.array([1.0])))[0] == 1.0
    assert np.isnan(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(np.array([np.nan])))[0])
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 4000),
                        np.array([0.0, -0.0, 1.0, -2.5, 65504.0, 3.3895314e38, np.inf, -np.inf], dtype=np.float32)])
    # exact ties: a bf16 value plus half an ulp
    base = (rng.integers(0x3000, 0x4800, 512).astype(np.uint32) << 16) | 0x8000
    x = np.concatenate([x, base.view(np.float32)]).astype(np.float32)
    got = oracle.f32_to_bf16_bits(x)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)


def test_e4m3_codec_against_torch(oracle):
    """The published E4M3 format: decode of all 256 codes and RNE/saturating encode, vs torch float8_e4m3fn."""
    table = oracle.e4m3_decode_table()
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    finite = ~np.isnan(want)
    assert np.array_equal(table[finite], want[finite])
    assert np.isnan(table[0x7F]) and np.isnan(table[0xFF])
    assert table[0x7E] == 448.0 and table[0x08] == 2.0 ** -6 and table[0x01] == 2.0 ** -9
    rng = np.random.default_rng(11)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-4, 3, 20000),
        np.array([0.0, -0.0, 448.0, -448.0, 447.9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 0.0175, 17.0, 18.0, 19.0],
                 dtype=np.float32),
        # every midpoint between adjacent finite codes (ties must go to the even mantissa)
        ((table[1:0x7F] + table[0:0x7E]) / 2).astype(np.float32),
    ])
    x = np.clip(x, -448.0, 448.0).astype(np.float32)
    got = oracle.f32_to_e4m3(x)
    want_bits = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, want_bits)
    # saturate-to-finite beyond the largest value, NaN stays NaN
    assert oracle.f32_to_e4m3(np.array([1e9, -1e9, np.inf], dtype=np.float32)).tolist() == [0x7E, 0xFE, 0x7E]
    assert oracle.f32_to_e4m3(np.array([np.nan], dtype=np.float32))[0] & 0x7F == 0x7F


def _int8_patterns(m, n, k):
    """crates/baracuda-kernels/tests/int8_rrr_smoke.rs:159-172."""
    a = np.array([((i * 7) % 15) - 7 for i in range(m * k)], dtype=np.int8)
    b = np.array([((i * 11) % 13) - 6 for i in range(k * n)], dtype=np.int8)
    return a, b


@pytest.mark.parametrize("shape", [(64, 64, 32), (128, 128, 128), (256, 128, 64), (100, 70, 50)])
def test_int8_smoke_shapes_fast_cell_equals_interpreter(oracle, shape):
    """The reference's int8 smoke shapes (int8_rrr_smoke.rs:442-500): the int32 fast
    cell equals the f64-accumulating interpreter over widened I32 operands, in both layouts."""
    m, n, k = shape
    a, b = _int8_patterns(m, n, k)
    ref_np = a.reshape(m, k).astype(np.int64) @ b.reshape(k, n).astype(np.int64)
    acc_rrr = oracle.gemm_s8_s32(a, b, oracle.RRR, m, n, k)
    assert np.array_equal(acc_rrr, ref_np.astype(np.int32))
    interp = oracle.contraction(oracle.I32, a.astype(np.int32), (0, k, 1), b.astype(np.int32), (0, n, 1), (1, m, n, k))
    assert np.array_equal(interp.reshape(m, n), acc_rrr)
    # same bytes read as column-major B (RCR): element (kk, j) at kk + j*ldb
    acc_rcr = oracle.gemm_s8_s32(a, b, oracle.RCR, m, n, k)
    want_rcr = a.reshape(m, k).astype(np.int64) @ b.reshape(n, k).astype(np.int64).T
    assert np.array_equal(acc_rcr, want_rcr.astype(np.int32))


def test_int_gemm_s8_out_reference_contract(oracle):
    """int8_rrr_smoke.rs:76-131, 159-172: alpha = 0.125, half-to-even saturating cast."""
    m, n, k = 64, 64, 32
    a, b = _int8_patterns(m, n, k)
    d = oracle.int_gemm_s8_out(a, b, oracle.RRR, m, n, k, alpha=0.125)
    acc = a.reshape(m, k).astype(np.int32) @ b.reshape(k, n).astype(np.int32)
    want = np.clip(np.rint(np.float32(0.125) * acc.astype(np.float32)), -128, 127).astype(np.int8)
    assert np.array_equal(d, want)
    # 12.5 -> 12 and 13.5 -> 14 (ties to even, LESSONS.md:442-478 of the reference)
    a1 = np.array([1] * 4, dtype=np.int8)
    b1 = np.array([25, 27, 0, 0, 0, 0, 0, 0], dtype=np.int8).reshape(4, 2)
    b1[:, :] = 0
    b1[0] = [25, 27]
    assert oracle.int_gemm_s8_out(a1, b1, oracle.RRR, 1, 2, 4, alpha=0.5).tolist() == [[12, 14]]


def test_w8a8_linear_fixture(oracle):
    """crates/baracuda-kernels/tests/quantized_linear_smoke.rs:82-184: quantize both sides with the
    reference's recipe, contract in int32, dequantise; within 3 % of the full-precision product."""
    kat = json.loads((GOLDEN / "reference_known_answers.json").read_text())["quantized_linear_w8a8_f32_basic"]
    a = np.array(kat["activation"], dtype=np.float32).reshape(2, 8)
    w = np.array(kat["weight"], dtype=np.float32).reshape(3, 8)
    aq, sa = oracle.quantize_rows_s8(a)
    wq, sw = oracle.quantize_rows_s8(w)
    # the row maximum always lands on +-127 and the scale is absmax/127
    assert np.all(np.abs(aq).max(axis=1) == 127) and np.all(np.abs(wq).max(axis=1) == 127)
    assert np.array_equal(sa, np.abs(a).max(axis=1) / np.float32(127))
    acc = oracle.gemm_s8_s32(aq, wq, oracle.RCR, 2, 3, 8)
    out = oracle.dequant_s32_f32(acc, sa, sw)
    want = np.array([[sum(np.float32(a[i, t]) * np.float32(w[j, t]) for t in range(8)) for j in range(3)] for i in range(2)],
                    dtype=np.float32)
    rel = np.abs(out - want) / np.maximum(np.abs(want), 1e-3)
    assert rel.max() < 0.03
    # bf16 store = RNE of that f32 value
    out_bf = oracle.dequant_s32_bf16(acc, sa, sw)
    assert np.array_equal(out_bf, torch.from_numpy(out).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))


def test_quantizer_zero_row_and_clamp(oracle):
    """baracuda_quantize_compose.cuh:183-189: an all-zero row gets scale 1 and zeros."""
    x = np.zeros((2, 16), dtype=np.float32)
    x[1, 3] = -5.0
    q, s = oracle.quantize_rows_s8(x)
    assert s[0] == 1.0 and not q[0].any()
    assert q[1, 3] == -127 and s[1] == np.float32(5.0) / np.float32(127)
    q8, s8 = oracle.quantize_rows_e4m3(x)
    assert s8[0] == 1.0 and not q8[0].any() and q8[1, 3] == 0xFE


@pytest.mark.parametrize("shape", [(64, 64, 32), (128, 128, 128), (100, 70, 50)])
def test_fp8_smoke_pattern(oracle, shape):
    """crates/baracuda-kernels/tests/fp8_e4m3_rcr_smoke.rs:66-127, 193-207: inputs on the e4m3 grid,
    alpha = 0.25; the f64-accumulated oracle agrees with the reference's f32-accumulating loop to
    within one e4m3 grid step after the e4m3 store."""
    m, n, k = shape
    av = np.array([(((i * 5) % 13) - 6) * 0.125 for i in range(m * k)], dtype=np.float32)
    bv = np.array([(((i * 7) % 11) - 5) * 0.125 for i in range(k * n)], dtype=np.float32)
    a_bits, b_bits = oracle.f32_to_e4m3(av), oracle.f32_to_e4m3(bv)
    table = oracle.e4m3_decode_table()
    assert np.array_equal(table[a_bits], av) and np.array_equal(table[b_bits], bv)  # exactly representable
    acc = oracle.gemm_e4m3_f32(a_bits, b_bits, oracle.RCR, m, n, k)
    # reference loop: f32 accumulate, K ascending, column-major B
    A = av.reshape(m, k)
    B = bv.reshape(n, k)
    want = np.zeros((m, n), dtype=np.float32)
    for kk in range(k):
        want += np.outer(A[:, kk], B[:, kk]).astype(np.float32)
    z_ref = np.float32(0.25) * want
    z_orc = np.float32(0.25) * acc
    d_ref = table[oracle.f32_to_e4m3(z_ref)]
    d_orc = table[oracle.f32_to_e4m3(z_orc)]
    mag = np.maximum(np.abs(d_ref), np.abs(d_orc))
    spacing = np.where(mag < 1.0 / 64.0, 1.0 / 512.0, 2.0 ** (np.floor(np.log2(np.maximum(mag, 1e-30))) - 3))
    assert np.all(np.abs(d_ref - d_orc) <= spacing + 1e-7)


def test_comparator(oracle):
    """docs/design/oracle.md:57-71 and oracle.rs:1998-2060 of the reference."""
    e = np.array([1.0, np.nan, 0.0, np.inf], dtype=np.float32)
    assert oracle.compare_tolerant(e, np.array([1.0 + 1e-4, np.nan, -0.0, np.inf], dtype=np.float32), 1e-3, 0.0) == -1
    assert oracle.compare_tolerant(e, np.array([1.1, np.nan, 0.0, np.inf], dtype=np.float32), 1e-3, 0.0) == 0
    assert oracle.compare_tolerant(e, np.array([1.0, np.nan, 0.0, -np.inf], dtype=np.float32), 1e-3, 0.0) == 3
    assert oracle.compare_tolerant(e, np.array([1.0, 5.0, 0.0, np.inf], dtype=np.float32), 1e-3, 0.0) == 1
    assert oracle.compare_bitexact(np.array([1, 2, 3], dtype=np.int32), np.array([1, 2, 3], dtype=np.int32)) == -1
    assert oracle.compare_bitexact(np.array([1, 2, 3], dtype=np.int32), np.array([1, 9, 3], dtype=np.int32)) == 1


def test_frozen_oracle_fixtures(oracle):
    """The committed fixtures (tests/golden/make_golden.py) still equal what the oracle computes,
    and the torch input quantizers used by the benchmark produce the oracle's bytes."""
    from baracuda_b200 import synth

    data = np.load(GOLDEN / "w8a8_fp8_cases.npz")
    for tag in ("c0s", "ragged"):
        a, b = data[f"{tag}_a_q"], data[f"{tag}_b_q"]
        m, k = a.shape
        n = b.shape[0]
        acc = oracle.gemm_s8_s32(a, b, oracle.RCR, m, n, k)
        assert np.array_equal(acc, data[f"{tag}_acc"])
        assert np.array_equal(oracle.dequant_s32_bf16(acc, data[f"{tag}_sa"], data[f"{tag}_sb"]), data[f"{tag}_out_bf16"])
    a8, b8 = data["fp8_a_q"], data["fp8_b_q"]
    m, k = a8.shape
    n = b8.shape[0]
    assert np.array_equal(oracle.gemm_e4m3_f32(a8, b8, oracle.RCR, m, n, k), data["fp8_acc"])
    # torch quantizers == oracle quantizers on the fixture's float inputs
    xf = torch.from_numpy(data["c0s_a_f32"])
    q_t, s_t = synth.quantize_rows_s8(xf)
    assert np.array_equal(q_t.numpy(), data["c0s_a_q"]) and np.array_equal(s_t.numpy(), data["c0s_sa"])
    q8_t, s8_t = synth.quantize_rows_e4m3(torch.from_numpy(data["fp8_a_f32"]))
    q8_o, s8_o = oracle.quantize_rows_e4m3(data["fp8_a_f32"])
    assert np.array_equal(q8_t.numpy(), q8_o) and np.array_equal(s8_t.numpy(), s8_o)
    qt_t, st_t = synth.quantize_tensor_e4m3(torch.from_numpy(data["fp8_a_f32"]))
    qt_o, st_o = oracle.quantize_tensor_e4m3(data["fp8_a_f32"])
    assert np.array_equal(qt_t.numpy(), qt_o) and np.array_equal(st_t.numpy(), st_o)
