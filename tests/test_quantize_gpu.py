"""GPU parity of the per-token activation quantizer and of the two-launch W8A8 linear built on it,
against the CPU oracle's restatement of the reference recipe: scales and codes bit-exact."""
import numpy as np
import pytest
import torch

import baracuda_b200 as bq
from helpers import bf16_bits, dev

pytestmark = pytest.mark.gpu


# the register-resident kernel at every threads-per-row choice (32 ... 1024), row counts that do not fill a CTA of eight
# warps, and the general kernel (columns not a whole number of vectors, rows longer than the registers hold)
@pytest.mark.parametrize("shape", [(1, 4096), (8, 4096), (128, 1024), (37, 50), (5, 8200), (3, 20000), (2048, 8192),
                                   (37, 4096), (13, 14336), (2, 40000), (2, 65536), (1, 70000), (3, 8)])
@pytest.mark.parametrize("in_dtype", ["f32", "bf16"])
def test_per_token_s8(oracle, shape, in_dtype):
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[0, :] = 0.0 if rows > 1 else x[0, :]  # an all-zero row gets scale 1 and zeros (compose.cuh:183-189)
    xt = torch.from_numpy(x)
    if in_dtype == "bf16":
        xt = xt.to(torch.bfloat16)
        x = xt.to(torch.float32).numpy()
    q_ref, s_ref = oracle.quantize_rows_s8(x)
    plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "s8"))
    scale = torch.full((rows,), float("nan"), device="cuda")
    q = torch.full((rows, cols), 99, dtype=torch.int8, device="cuda")
    plan.run(None, xt.cuda(), scale, q)
    torch.cuda.synchronize()
    assert np.array_equal(scale.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("shape", [(8, 4096), (100, 70), (512, 8192), (19, 14336), (2, 40000)])
@pytest.mark.parametrize("in_dtype", ["f32", "bf16"])
def test_per_token_e4m3(oracle, shape, in_dtype):
    rows, cols = shape
    x = (np.random.default_rng(cols).standard_normal((rows, cols)) * 3.0).astype(np.float32)
    xt = torch.from_numpy(x)
    if in_dtype == "bf16":
        xt = xt.to(torch.bfloat16)
        x = xt.to(torch.float32).numpy()
    q_ref, s_ref = oracle.quantize_rows_e4m3(x)
    plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "e4m3"))
    scale = torch.empty(rows, device="cuda")
    q = torch.empty((rows, cols), dtype=torch.uint8, device="cuda")
    plan.run(None, xt.cuda(), scale, q)
    torch.cuda.synchronize()
    assert np.array_equal(scale.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("in_dtype", ["f32", "bf16"])
def test_aligned_padded_pitches_keep_the_vector_path_inside_the_row(oracle, in_dtype):
    """Row pitches wider than the row (but 16-byte aligned, so the register-resident kernel runs): nothing beyond the
    row's columns is read into the maximum or written, and non-finite padding cannot leak into the scales."""
    rows, cols, ld_in, ld_out = 11, 4096, 4096 + 64, 4096 + 32
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, ld_in)).astype(np.float32)
    x[:, cols:] = 1e30  # padding far above every real value
    xt = torch.from_numpy(x)
    if in_dtype == "bf16":
        xt = xt.to(torch.bfloat16)
        x = xt.to(torch.float32).numpy()
    q_ref, s_ref = oracle.quantize_rows_s8(np.ascontiguousarray(x[:, :cols]))
    plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "s8"))
    scale = torch.empty(rows, device="cuda")
    q = torch.full((rows, ld_out), 77, dtype=torch.int8, device="cuda")
    plan.run(None, xt.cuda(), scale, q, ld_in=ld_in, ld_out=ld_out)
    torch.cuda.synchronize()
    got = q.cpu().numpy()
    assert np.array_equal(got[:, :cols], q_ref) and np.all(got[:, cols:] == 77)
    assert np.array_equal(scale.cpu().numpy(), s_ref)


@pytest.mark.parametrize("qrange", [(-127, 127), (-128, 127), (-7, 7), (-50, 100), (-100, 50), (0, 127)])
@pytest.mark.parametrize("in_dtype", ["f32", "bf16"])
def test_quantization_ranges_with_and_without_the_clamp(oracle, qrange, in_dtype):
    """Symmetric ranges (and -128..127) take the clamp-free rounding of the register-resident kernel, ranges the scaled
    values can leave keep the clamp; both against the oracle, on rows with ties (x.5 after scaling) in them."""
    qmin, qmax = qrange
    rows, cols = 16, 4096
    rng = np.random.default_rng(qmax - qmin)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    # rows whose scale is a power of two, so that many scaled values land exactly on .5
    x[0] = (rng.integers(-2 * qmax, 2 * qmax + 1, size=cols) * 0.5).astype(np.float32)
    x[0, 0] = float(qmax)
    x[1] = -x[0]
    xt = torch.from_numpy(x)
    if in_dtype == "bf16":
        xt = xt.to(torch.bfloat16)
        x = xt.to(torch.float32).numpy()
    q_ref, s_ref = oracle.quantize_rows_s8(x, qmin, qmax)
    plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "s8", qmin, qmax))
    scale = torch.empty(rows, device="cuda")
    q = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
    plan.run(None, xt.cuda(), scale, q)
    torch.cuda.synchronize()
    assert np.array_equal(scale.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


def test_nan_entries_are_skipped_by_the_row_maximum_on_both_paths(oracle):
    """fmaxf ignores a NaN operand; the bf16 fast path compares bit patterns and has to skip NaNs explicitly."""
    rows, cols = 4, 4096
    x = np.random.default_rng(5).standard_normal((rows, cols)).astype(np.float32)
    x[1, 17] = np.nan
    x[2, 4000] = np.nan
    clean = np.where(np.isnan(x), 0.0, x).astype(np.float32)
    _, s_ref = oracle.quantize_rows_s8(clean)
    for xt in (torch.from_numpy(x), torch.from_numpy(x).to(torch.bfloat16)):
        if xt.dtype == torch.bfloat16:
            _, s_ref = oracle.quantize_rows_s8(np.where(np.isnan(x), 0.0, xt.to(torch.float32).numpy()).astype(np.float32))
        plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "s8"))
        scale = torch.empty(rows, device="cuda")
        q = torch.empty((rows, cols), dtype=torch.int8, device="cuda")
        plan.run(None, xt.cuda(), scale, q)
        torch.cuda.synchronize()
        assert np.array_equal(scale.cpu().numpy(), s_ref)


def test_padded_pitches_and_canaries(oracle):
    rows, cols, ld_in, ld_out = 9, 100, 117, 131  # odd pitches: the scalar path
    x = np.random.default_rng(1).standard_normal((rows, ld_in)).astype(np.float32)
    q_ref, s_ref = oracle.quantize_rows_s8(x[:, :cols])
    plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(rows, cols, "s8"))
    scale = torch.empty(rows, device="cuda")
    q = torch.full((rows, ld_out), 77, dtype=torch.int8, device="cuda")
    plan.run(None, dev(x), scale, q, ld_in=ld_in, ld_out=ld_out)
    torch.cuda.synchronize()
    got = q.cpu().numpy()
    assert np.array_equal(got[:, :cols], q_ref) and np.all(got[:, cols:] == 77)
    assert np.array_equal(scale.cpu().numpy(), s_ref)


@pytest.mark.parametrize("m", [1, 4, 300])
def test_quantized_linear_two_launch_path(oracle, m):
    """QuantizedLinearPlan (quantize, then GEMV for m <= 8 or GEMM): bit-equal to the oracle's
    quantize -> int32 contraction -> (sa*sw)*acc -> bf16, and within 3 % (relative L2 error) of the
    full-precision product, the level the reference accepts (quantized_linear_smoke.rs:171-184)."""
    c_out, k = 1024, 2048
    rng = np.random.default_rng(m)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((c_out, k)) * 0.02).astype(np.float32)
    wq, sw = oracle.quantize_rows_s8(w)
    aq, sa = oracle.quantize_rows_s8(a)
    want = oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, c_out, k), sa, sw)
    plan = bq.QuantizedLinearPlan.select(None, bq.QuantizedLinearDescriptor(m, c_out, k))
    assert plan.sku().arch is bq.ArchSku.Sm100a
    out = torch.empty((m, c_out), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    plan.run(None, ws, bq.QuantizedLinearArgs(
        activation=dev(a), weight_q=dev(wq), weight_scale=dev(sw), output=out,
        act_q_scratch=torch.empty((m, k), dtype=torch.int8, device="cuda"),
        act_scale_scratch=torch.empty(m, device="cuda")))
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(out), want)
    full = a @ w.T
    got = out.to(torch.float32).cpu().numpy()
    assert np.linalg.norm(got - full) / np.linalg.norm(full) < 0.03


@pytest.mark.parametrize("m", [1, 2, 5, 8])
@pytest.mark.parametrize("nk", [(1024, 2048), (14336, 4096), (1000, 512), (4096, 8192)])
def test_decode_step_in_one_launch(oracle, m, nk):
    """bf16 activations, m <= 8: the per-token quantiser runs inside the GEMV.  The output and the scales must equal
    the two-launch path (quantize_per_token_sym_bf16_s8, then gemv_q8_m1_bf16) and the oracle bit for bit."""
    c_out, k = nk
    rng = np.random.default_rng(m * 31 + k)
    a_bf = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
    if m >= 5:
        a_bf[m - 1].zero_()  # an all-zero token: scale 1.0
    a = a_bf.to(torch.float32).numpy()
    w = (rng.standard_normal((c_out, k)) * 0.02).astype(np.float32)
    wq, sw = oracle.quantize_rows_s8(w)
    aq, sa = oracle.quantize_rows_s8(a)
    want = oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, c_out, k), sa, sw)
    plan = bq.QuantizedLinearPlan.select(None, bq.QuantizedLinearDescriptor(m, c_out, k))
    out = torch.full((m, c_out), float("nan"), dtype=torch.bfloat16, device="cuda")
    scales = torch.full((m,), float("nan"), device="cuda")
    args = bq.QuantizedLinearArgs(activation=a_bf.cuda(), weight_q=dev(wq), weight_scale=dev(sw), output=out,
                                  act_q_scratch=torch.empty((m, k), dtype=torch.int8, device="cuda"),
                                  act_scale_scratch=scales)
    assert plan.fused_decode_ok(args)
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    plan.run(None, ws, args)
    torch.cuda.synchronize()
    assert bq.device_status() == 0
    assert np.array_equal(scales.cpu().numpy(), sa)
    assert np.array_equal(bf16_bits(out), want)


def test_decode_fusion_declines_other_shapes():
    from baracuda_b200 import _lib
    can = _lib.load().baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement
    assert can(1, 14336, 4096, 4096, 4096, 14336) == 0
    assert can(1, 4096, 14336, 14336, 14336, 4096) == 3   # 28 chunks of 512 do not divide 16
    assert can(1, 1024, 4096 + 64, 4096 + 64, 4096 + 64, 1024) == 3
    assert can(9, 1024, 4096, 4096, 4096, 1024) == 2
    assert can(1, 1024, 4096, 4000, 4096, 1024) == 2      # ldx < k
    assert can(0, 1024, 4096, 4096, 4096, 1024) == 0
