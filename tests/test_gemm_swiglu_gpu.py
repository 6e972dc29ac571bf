"""GPU parity of the gated-MLP up-projection: one GEMM over the interleaved gate/up weight whose epilogue stores
silu(z_gate) * z_up as bf16 [M, F].  The reference has no such epilogue (its EpilogueKind ends at BiasSilu,
crates/baracuda-kernel-vocab/src/layout.rs:69-96), so parity is defined from its pieces: the W8A8 dequant
(sa*sb)*(float)acc (baracuda_quantize_compose.cuh:271-274), silu as its tests state it
(crates/baracuda-kernels/tests/int8_rrr_smoke.rs:60-66), the product in f32, one bf16 rounding.
Tolerance: one bf16 ulp of the expected value."""
import numpy as np
import pytest
import torch

from baracuda_b200 import (ElementKind, GatedMlpUpArgs, GatedMlpUpDescriptor, GatedMlpUpPlan, InvalidProblem,
                           MisalignedOperand, Unsupported, _lib, set_tuning, SCALE_PER_TENSOR, SCALE_PER_ROW_COL)
from helpers import dev, pad_rows

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _status_clean():
    torch.cuda.synchronize()
    assert _lib.load().baracuda_kernels_q_device_status() == 0


def _w8a8_inputs(oracle, m, f, k, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    wg = rng.integers(-127, 128, size=(f, k), dtype=np.int8)
    wu = rng.integers(-127, 128, size=(f, k), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m).astype(np.float32)
    # scales that put z_gate around +-3: both branches of silu are exercised
    sg = rng.uniform(0.0005, 0.004, size=f).astype(np.float32) * np.float32(16.0 / np.sqrt(k))
    su = rng.uniform(0.0005, 0.004, size=f).astype(np.float32) * np.float32(16.0 / np.sqrt(k))
    zg = oracle.dequant_s32_f32(oracle.gemm_s8_s32(a, wg, oracle.RCR, m, f, k), sa, sg)
    zu = oracle.dequant_s32_f32(oracle.gemm_s8_s32(a, wu, oracle.RCR, m, f, k), sa, su)
    return a, wg, wu, sa, sg, su, zg, zu


def _close(got, want, slack):
    tol = np.abs(want) * 2.0 ** -7 + slack
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside one bf16 ulp; worst {np.abs(got - want).max()}"


@pytest.mark.parametrize("shape", [(128, 32, 64), (300, 544, 256), (1024, 1024, 512), (520, 1504, 128)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_w8a8_gate_up(oracle, shape, with_bias):
    m, f, k = shape
    a, wg, wu, sa, sg, su, zg, zu = _w8a8_inputs(oracle, m, f, k, 4321 + m + int(with_bias))
    rng = np.random.default_rng(77)
    alpha = np.float32(0.75)
    zg, zu = (zg * alpha).astype(np.float32), (zu * alpha).astype(np.float32)
    bg = bu = None
    if with_bias:
        bg = rng.standard_normal(f).astype(np.float32)
        bu = rng.standard_normal(f).astype(np.float32)
        zg, zu = (zg + bg[None, :]).astype(np.float32), (zu + bu[None, :]).astype(np.float32)
    want = oracle.swiglu_f32(zg, zu)

    plan = GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(m, f, k))
    assert plan.workspace_size() == 0
    w = GatedMlpUpPlan.interleave(dev(wg), dev(wu))
    sb = GatedMlpUpPlan.interleave(dev(sg), dev(su))
    assert np.array_equal(w.cpu().numpy(), oracle.interleave_gate_up(wg, wu))
    assert np.array_equal(sb.cpu().numpy(), oracle.interleave_gate_up(sg, su))
    bias = GatedMlpUpPlan.interleave(dev(bg), dev(bu)) if with_bias else None
    ldd = f + 8
    d = torch.full((m, ldd), 7.0, dtype=torch.bfloat16, device="cuda")
    plan.run(None, None, GatedMlpUpArgs(a=dev(a), b_gate_up=w, d=d, scale_a=dev(sa), scale_b=sb, bias=bias, ldd=ldd,
                                        alpha=float(alpha)))
    _status_clean()
    got = d.float().cpu().numpy()
    _close(got[:, :f], want, 1e-6)
    assert np.all(got[:, f:] == 7.0)  # the row padding is not written


@pytest.mark.parametrize("tuning", [(0, 64), (0, 128), (0, 256), (0, 512), (2, 192), (2, 128)])
def test_w8a8_gate_up_on_every_tile_width(oracle, tuning):
    m, f, k = 640, 800, 192
    a, wg, wu, sa, sg, su, zg, zu = _w8a8_inputs(oracle, m, f, k, 99)
    want = oracle.swiglu_f32(zg, zu)
    plan = GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(m, f, k))
    w = GatedMlpUpPlan.interleave(dev(wg), dev(wu))
    sb = GatedMlpUpPlan.interleave(dev(sg), dev(su))
    d = torch.zeros((m, f), dtype=torch.bfloat16, device="cuda")
    key, value = tuning
    try:
        if key == 2:
            set_tuning(0, 512)
        set_tuning(key, value)
        plan.run(None, None, GatedMlpUpArgs(a=dev(a), b_gate_up=w, d=d, scale_a=dev(sa), scale_b=sb))
    finally:
        set_tuning(0, 0)
        set_tuning(2, 0)
    _status_clean()
    _close(d.float().cpu().numpy(), want, 1e-6)


@pytest.mark.parametrize("scale_mode", [SCALE_PER_TENSOR, SCALE_PER_ROW_COL])
def test_fp8_gate_up(oracle, scale_mode):
    m, f, k = 520, 1056, 256
    rng = np.random.default_rng(5 + scale_mode)
    a = oracle.f32_to_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    wg = oracle.f32_to_e4m3(rng.standard_normal((f, k)).astype(np.float32))
    wu = oracle.f32_to_e4m3(rng.standard_normal((f, k)).astype(np.float32))
    accg = oracle.gemm_e4m3_f32(a, wg, oracle.RCR, m, f, k)
    accu = oracle.gemm_e4m3_f32(a, wu, oracle.RCR, m, f, k)
    if scale_mode == SCALE_PER_ROW_COL:
        sa = rng.uniform(0.05, 0.2, size=m).astype(np.float32)
        sg = rng.uniform(0.05, 0.2, size=f).astype(np.float32)
        su = rng.uniform(0.05, 0.2, size=f).astype(np.float32)
        zg = ((sa[:, None] * sg[None, :]).astype(np.float32) * accg).astype(np.float32)
        zu = ((sa[:, None] * su[None, :]).astype(np.float32) * accu).astype(np.float32)
        sb = GatedMlpUpPlan.interleave(dev(sg), dev(su))
    else:
        sa = np.array([0.11], dtype=np.float32)
        sbv = np.array([0.07], dtype=np.float32)
        zg = ((sa[0] * sbv[0]).astype(np.float32) * accg).astype(np.float32)
        zu = ((sa[0] * sbv[0]).astype(np.float32) * accu).astype(np.float32)
        sb = dev(sbv)
    want = oracle.swiglu_f32(zg, zu)
    plan = GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(m, f, k, ElementKind.Fp8E4M3, scale_mode))
    w = GatedMlpUpPlan.interleave(dev(wg), dev(wu))
    d = torch.zeros((m, f), dtype=torch.bfloat16, device="cuda")
    plan.run(None, None, GatedMlpUpArgs(a=dev(a), b_gate_up=w, d=d, scale_a=dev(sa), scale_b=sb))
    _status_clean()
    # f32 accumulation order differs from the oracle's f64 sums: allow that slack on each factor
    got = d.float().cpu().numpy()
    tol = np.abs(want) * 2.0 ** -7 + 2e-3 * (np.abs(zu) + 1.0)
    assert np.all(np.abs(got - want) <= tol)


def test_k_zero_gives_zeros():
    """An empty contraction: z_gate = z_up = 0, so h = silu(0) * 0 = 0 (the GEMM family's k == 0 rule)."""
    m, f = 64, 64
    plan = GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(m, f, 0))
    d = torch.full((m, f), 3.0, dtype=torch.bfloat16, device="cuda")
    z8 = torch.zeros(4096, dtype=torch.int8, device="cuda")
    s = torch.ones(2 * f, dtype=torch.float32, device="cuda")
    plan.run(None, None, GatedMlpUpArgs(a=z8, b_gate_up=z8, d=d, scale_a=s, scale_b=s))
    _status_clean()
    assert torch.all(d == 0)


def test_status_rules():
    lib = _lib.load()
    z = torch.zeros(1 << 16, dtype=torch.int8, device="cuda")
    s = torch.ones(256, dtype=torch.float32, device="cuda")
    d = torch.zeros(1 << 14, dtype=torch.bfloat16, device="cuda")
    run = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run
    can = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement
    ok = (64, 128, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr(), 64)
    assert can(*ok) == 0
    assert can(64, 96, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr(), 48) == 3    # n2 not a multiple of 64
    assert can(64, 128, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr(), 63) == 2   # ldd < F
    assert can(64, 128, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr(), 68) == 1   # row pitch not 16 bytes
    assert can(64, 128, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr() + 2, 64) == 1
    assert can(-1, 128, 64, z.data_ptr(), 64, z.data_ptr(), 64, d.data_ptr(), 64) == 2
    assert run(*ok, None, s.data_ptr(), None, 1.0, None, 0, _stream()) == 2              # scales are required
    assert run(0, 128, 64, None, 64, None, 64, None, 64, None, None, None, 1.0, None, 0, _stream()) == 0  # empty
    il = lib.baracuda_kernels_q_interleave_gate_up_run
    assert il(48, 64, z.data_ptr(), 64, z.data_ptr(), 64, z.data_ptr(), 64, _stream()) == 3  # F not a multiple of 32
    assert il(32, 64, z.data_ptr(), 32, z.data_ptr(), 64, z.data_ptr(), 64, _stream()) == 2  # pitch < row
    with pytest.raises(Unsupported):
        GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(8, 48, 64))
    with pytest.raises(InvalidProblem):
        GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(8, 64, 64, ElementKind.S8, SCALE_PER_TENSOR))
    plan = GatedMlpUpPlan.select(None, GatedMlpUpDescriptor(64, 64, 64))
    with pytest.raises(MisalignedOperand):
        plan.run(None, None, GatedMlpUpArgs(a=z, b_gate_up=z, d=d, scale_a=s, scale_b=s, ldd=68))
    torch.cuda.synchronize()
