"""GPU parity of the fused bias / activation epilogues (the reference's EpilogueKind chain) on the 8-bit-out and
bf16-out GEMM symbols.  Inputs, bias patterns, alpha and the 128^3 shape are those of the reference's smoke tests
(crates/baracuda-kernels/tests/int8_rrr_smoke.rs:159-172,416-430,500-620; fp8_bias_smoke.rs:166-202); ragged
shapes are added.  Bias and BiasRelu must be exact; BiasGelu / BiasSilu may differ by one output code (int8),
one e4m3 grid step, or one bf16 ulp -- tighter than the reference's own +-1 / two-step rule."""
import numpy as np
import pytest
import torch

from baracuda_b200 import _lib
from helpers import dev, pad_rows

pytestmark = pytest.mark.gpu

ACTS = {1: "", 2: "_relu", 3: "_gelu", 4: "_silu"}
SHAPES = [(128, 128, 128), (100, 70, 50), (300, 520, 192)]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _status_clean():
    torch.cuda.synchronize()
    assert _lib.load().baracuda_kernels_q_device_status() == 0


def _s8_operands(m, n, k, layout):
    a = np.array([((i * 7) % 15) - 7 for i in range(m * k)], dtype=np.int8).reshape(m, k)
    if layout == "rcr":
        b = np.array([((i * 11) % 13) - 6 for i in range(k * n)], dtype=np.int8).reshape(n, k)
    else:
        b = np.array([((i * 11) % 13) - 6 for i in range(k * n)], dtype=np.int8).reshape(k, n)
    return a, b


def _weights_dev(b, layout, k, n):
    """Device copy with a 16-byte-aligned pitch, and that pitch."""
    inner = k if layout == "rcr" else n
    ld = (inner + 15) // 16 * 16
    return dev(pad_rows(b, ld)), ld


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
@pytest.mark.parametrize("bias_kind", ["f32", "i32"])
@pytest.mark.parametrize("epi", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", SHAPES)
def test_s8_bias_activation(oracle, layout, bias_kind, epi, shape):
    m, n, k = shape
    a, b = _s8_operands(m, n, k, layout)
    if bias_kind == "f32":
        bias = np.array([((j % 5) - 2) * 0.5 for j in range(n)], dtype=np.float32)
    else:
        bias = np.array([((j % 5) - 2) * 2 for j in range(n)], dtype=np.int32)
    alpha = np.float32(0.125)
    acc = oracle.gemm_s8_s32(a, b, oracle.RCR if layout == "rcr" else oracle.RRR, m, n, k)
    want = oracle.sat_s8(oracle.epilogue_chain(alpha * acc.astype(np.float32), bias, epi))
    lda = (k + 15) // 16 * 16
    bd, ldb = _weights_dev(b, layout, k, n)
    d = torch.full((m, n), 99, dtype=torch.int8, device="cuda")
    lib = _lib.load()
    sym = f"baracuda_kernels_gemm_s8_{layout}_sm100a_bias{ACTS[epi]}_{bias_kind}_run"
    ad, biasd = dev(pad_rows(a, lda)), dev(bias)
    st = getattr(lib, sym)(m, n, k, ad.data_ptr(), lda, bd.data_ptr(), ldb, None, 0, d.data_ptr(), n,
                           biasd.data_ptr(), float(alpha), 0.0, None, 0, _stream())
    assert st == 0
    _status_clean()
    got = d.cpu().numpy()
    if epi <= 2:
        assert np.array_equal(got, want)
    else:
        diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 0.01


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
def test_s8_epilogue_run_with_beta_and_generic_chain(oracle, layout):
    """z = alpha*acc + beta*C + bias through the argument-driven symbol; identity ignores the bias pointer."""
    m, n, k = 200, 136, 96
    a, b = _s8_operands(m, n, k, layout)
    c = np.array([((i * 5) % 17) - 8 for i in range(m * n)], dtype=np.int8).reshape(m, n)
    bias = np.array([((j % 5) - 2) * 0.5 for j in range(n)], dtype=np.float32)
    alpha, beta = np.float32(0.125), np.float32(0.5)
    acc = oracle.gemm_s8_s32(a, b, oracle.RCR if layout == "rcr" else oracle.RRR, m, n, k)
    z = (alpha * acc.astype(np.float32) + beta * c.astype(np.float32)).astype(np.float32)
    lda = (k + 15) // 16 * 16
    bd, ldb = _weights_dev(b, layout, k, n)
    ad, cd, biasd = dev(pad_rows(a, lda)), dev(c), dev(bias)
    run = getattr(_lib.load(), f"baracuda_kernels_gemm_s8_{layout}_sm100a_epilogue_run")
    for epi in (0, 1, 2):
        d = torch.full((m, n), 99, dtype=torch.int8, device="cuda")
        st = run(m, n, k, ad.data_ptr(), lda, bd.data_ptr(), ldb, cd.data_ptr(), n, d.data_ptr(), n,
                 biasd.data_ptr(), 1, epi, float(alpha), float(beta), None, 0, _stream())
        assert st == 0
        _status_clean()
        assert np.array_equal(d.cpu().numpy(), oracle.sat_s8(oracle.epilogue_chain(z, bias, epi)))


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
@pytest.mark.parametrize("epi", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", SHAPES[:2])
def test_e4m3_bias_activation(oracle, layout, epi, shape):
    m, n, k = shape
    av = np.array([(((i * 5) % 13) - 6) * 0.125 for i in range(m * k)], dtype=np.float32).reshape(m, k)
    bshape = (n, k) if layout == "rcr" else (k, n)
    bv = np.array([(((i * 7) % 11) - 5) * 0.125 for i in range(k * n)], dtype=np.float32).reshape(bshape)
    a_bits, b_bits = oracle.f32_to_e4m3(av), oracle.f32_to_e4m3(bv)
    bias = np.array([((j % 5) - 2) * 0.5 for j in range(n)], dtype=np.float32)
    acc = oracle.gemm_e4m3_f32(a_bits, b_bits, oracle.RCR if layout == "rcr" else oracle.RRR, m, n, k)
    want_bits = oracle.f32_to_e4m3(oracle.epilogue_chain(np.float32(0.25) * acc, bias, epi))
    lda = (k + 15) // 16 * 16
    bd, ldb = _weights_dev(b_bits, layout, k, n)
    d = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
    sym = f"baracuda_kernels_gemm_fp8_e4m3_{layout}_sm100a_bias{ACTS[epi]}_run"
    ad, biasd = dev(pad_rows(a_bits, lda)), dev(bias)
    st = getattr(_lib.load(), sym)(m, n, k, ad.data_ptr(), lda, bd.data_ptr(), ldb, None, 0,
                                   d.data_ptr(), n, biasd.data_ptr(), 0.25, 0.0, None, 0, _stream())
    assert st == 0
    _status_clean()
    got_bits = d.cpu().numpy()
    if epi <= 2:
        assert np.array_equal(got_bits, want_bits)
    else:
        # neighbouring codes of one sign differ by one grid step; +0 / -0 decode to the same value
        table = oracle.e4m3_decode_table()
        same_value = table[got_bits] == table[want_bits]
        step = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32)) <= 1
        assert np.all(same_value | step) and (~same_value).mean() < 0.01


@pytest.mark.parametrize("family", ["w8a8_s8", "fp8_e4m3"])
@pytest.mark.parametrize("layout", ["rcr", "rrr"])
@pytest.mark.parametrize("epi", [0, 1, 2, 3, 4])
def test_bf16_out_bias_activation(oracle, family, layout, epi):
    """D = bf16(act((sa*sb)*acc*alpha + bias)) on a shape that runs both the staged and the ragged store paths."""
    m, n, k = 300, 1096, 256
    rng = np.random.default_rng(1234 + epi)
    lay = oracle.RCR if layout == "rcr" else oracle.RRR
    bshape = (n, k) if layout == "rcr" else (k, n)
    if family == "w8a8_s8":
        a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
        b = rng.integers(-127, 128, size=bshape, dtype=np.int8)
        acc = oracle.gemm_s8_s32(a, b, lay, m, n, k)
        sa = rng.uniform(0.001, 0.01, size=m).astype(np.float32)
        sb = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
        y = oracle.dequant_s32_f32(acc, sa, sb)
    else:
        a = oracle.f32_to_e4m3(rng.standard_normal((m, k)).astype(np.float32))
        b = oracle.f32_to_e4m3(rng.standard_normal(bshape).astype(np.float32))
        acc = oracle.gemm_e4m3_f32(a, b, lay, m, n, k)
        sa = rng.uniform(0.05, 0.2, size=m).astype(np.float32)
        sb = rng.uniform(0.05, 0.2, size=n).astype(np.float32)
        y = ((sa[:, None] * sb[None, :]).astype(np.float32) * acc).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = oracle.epilogue_chain(y, bias, epi)
    lda = (k + 15) // 16 * 16
    bd, ldb = _weights_dev(b, layout, k, n)
    d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    sym = f"baracuda_kernels_gemm_{family}_{layout}_bf16_sm100a_epilogue_run"
    ad, sad, sbd, biasd = dev(pad_rows(a, lda)), dev(sa), dev(sb), dev(bias)
    st = getattr(_lib.load(), sym)(m, n, k, ad.data_ptr(), lda, bd.data_ptr(), ldb, None, 0,
                                   d.data_ptr(), n, sad.data_ptr(), sbd.data_ptr(), 1, biasd.data_ptr(), epi,
                                   1.0, 0.0, None, 0, _stream())
    assert st == 0
    _status_clean()
    got = d.float().cpu().numpy()
    # one bf16 ulp of the expected value (2^-7 relative), plus the f32 accumulation-order slack of the fp8 sums
    tol = np.abs(want) * 2.0 ** -7 + (1e-3 if family == "fp8_e4m3" else 1e-6)
    assert np.all(np.abs(got - want) <= tol)
    if family == "w8a8_s8" and epi <= 2:
        want_bits = oracle.f32_to_bf16_bits(want)
        assert np.array_equal(d.view(torch.int16).cpu().numpy().view(np.uint16), want_bits)


@pytest.mark.parametrize("family", ["w8a8_s8", "fp8_e4m3"])
@pytest.mark.parametrize("shape", [(300, 1096, 256), (1024, 2048, 128), (100, 70, 64)])
@pytest.mark.parametrize("in_place", [False, True])
def test_bf16_out_beta_c(oracle, family, shape, in_place):
    """D = bf16(alpha * (sa*sb) * acc + beta * C [+ bias]) with C bf16 (the residual add of an o / down projection),
    C separate with its own pitch or D itself; staged, ragged and CTA-pair store paths."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + int(in_place))
    if family == "w8a8_s8":
        a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
        b = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        acc = oracle.gemm_s8_s32(a, b, oracle.RCR, m, n, k)
        sa = rng.uniform(0.001, 0.01, size=m).astype(np.float32)
        sb = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
        y = oracle.dequant_s32_f32(acc, sa, sb)
    else:
        a = oracle.f32_to_e4m3(rng.standard_normal((m, k)).astype(np.float32))
        b = oracle.f32_to_e4m3(rng.standard_normal((n, k)).astype(np.float32))
        acc = oracle.gemm_e4m3_f32(a, b, oracle.RCR, m, n, k)
        sa = rng.uniform(0.05, 0.2, size=m).astype(np.float32)
        sb = rng.uniform(0.05, 0.2, size=n).astype(np.float32)
        y = ((sa[:, None] * sb[None, :]).astype(np.float32) * acc).astype(np.float32)
    alpha, beta = np.float32(0.5), np.float32(-1.25)
    c_bits = oracle.f32_to_bf16_bits(rng.standard_normal((m, n)).astype(np.float32))
    c = oracle.bf16_bits_to_f32(c_bits)
    bias = rng.standard_normal(n).astype(np.float32)
    z = ((y * alpha).astype(np.float32) + (beta * c).astype(np.float32)).astype(np.float32)
    want = oracle.epilogue_chain(z, bias, 1)
    lda = (k + 15) // 16 * 16
    ad, bd = dev(pad_rows(a, lda)), dev(pad_rows(b, lda))
    ldc = n if in_place else n + 3  # an odd pitch takes the scalar C loads
    cd = torch.from_numpy(pad_rows(c_bits.view(np.int16), ldc)).cuda().view(torch.bfloat16)
    d = cd if in_place else torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    sym = f"baracuda_kernels_gemm_{family}_rcr_bf16_sm100a_epilogue_run"
    sad, sbd, biasd = dev(sa), dev(sb), dev(bias)
    st = getattr(_lib.load(), sym)(m, n, k, ad.data_ptr(), lda, bd.data_ptr(), lda, cd.data_ptr(), ldc,
                                   d.data_ptr(), n, sad.data_ptr(), sbd.data_ptr(), 1, biasd.data_ptr(), 1,
                                   float(alpha), float(beta), None, 0, _stream())
    assert st == 0
    _status_clean()
    got = d.float().cpu().numpy()
    if family == "w8a8_s8":
        assert np.array_equal(d.view(torch.int16).cpu().numpy().view(np.uint16), oracle.f32_to_bf16_bits(want))
    else:
        tol = np.abs(want) * 2.0 ** -7 + 1e-3
        assert np.all(np.abs(got - want) <= tol)


def test_bf16_out_beta_c_status_rules():
    lib = _lib.load()
    z = torch.zeros(1 << 16, dtype=torch.int8, device="cuda")
    s = torch.ones(256, dtype=torch.float32, device="cuda")
    d = torch.zeros(1 << 14, dtype=torch.bfloat16, device="cuda")
    run = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run
    can = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement
    head = (64, 64, 64, z.data_ptr(), 64, z.data_ptr(), 64)
    assert can(*head, d.data_ptr(), 64, d.data_ptr(), 64) == 0
    assert can(*head, d.data_ptr(), 63, d.data_ptr(), 64) == 2                    # ldc < n
    assert can(*head, d.data_ptr() + 1, 64, d.data_ptr(), 64) == 1                # C not 2-byte aligned
    tail = (s.data_ptr(), s.data_ptr())
    assert run(*head, None, 0, d.data_ptr(), 64, *tail, 1.0, 0.5, None, 0, _stream()) == 2   # beta without C
    assert run(*head, d.data_ptr(), 64, d.data_ptr(), 64, *tail, 1.0, 0.0, None, 0, _stream()) == 0  # beta 0: C unread
    raw = lib.baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement
    assert raw(*head, d.data_ptr(), 64, d.data_ptr(), 64) == 3                    # the raw SKU takes no C
    torch.cuda.synchronize()


def test_epilogue_status_rules():
    lib = _lib.load()
    z = torch.zeros(4096, dtype=torch.int8, device="cuda")
    f = torch.zeros(64, dtype=torch.float32, device="cuda")
    run = lib.baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run
    args = (16, 16, 16, z.data_ptr(), 16, z.data_ptr(), 16, None, 0, z.data_ptr(), 16)
    assert run(*args, None, 1, 1, 1.0, 0.0, None, 0, _stream()) == 2           # bias chain without a bias
    assert run(*args, f.data_ptr(), 3, 1, 1.0, 0.0, None, 0, _stream()) == 2   # unknown bias type
    assert run(*args, f.data_ptr(), 1, 5, 1.0, 0.0, None, 0, _stream()) == 2   # unknown chain
    assert run(*args, None, 0, 0, 1.0, 0.0, None, 0, _stream()) == 0           # identity needs none
    frun = lib.baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_epilogue_run
    assert frun(*args, f.data_ptr(), 2, 1, 1.0, 0.0, None, 0, _stream()) == 2  # fp8 takes a float bias only
    torch.cuda.synchronize()


@pytest.mark.parametrize("tn", [256, 224, 192, 128])
@pytest.mark.parametrize("epi", [3, 4])
@pytest.mark.parametrize("out", ["bf16", "s8"])
def test_eight_epilogue_warps_gelu_silu_on_the_cta_pair_kernel(oracle, tn, epi, out):
    """bias + gelu / silu on the CTA-pair kernel run with eight epilogue warps (two per tensor-memory lane quadrant, each
    half of the column blocks): every tile width (224 has an odd number of 32-column blocks), ragged M / N, both the
    staged bf16 stores and the direct 8-bit stores, checked against the oracle's chain."""
    import baracuda_b200 as bq

    m, n, k = 700, 1480, 256
    rng = np.random.default_rng(tn + epi)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    b = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    bias = rng.standard_normal(n).astype(np.float32)
    acc = oracle.gemm_s8_s32(a, b, oracle.RCR, m, n, k)
    lda = (k + 15) // 16 * 16
    ad, bd, biasd = dev(pad_rows(a, lda)), dev(pad_rows(b, lda)), dev(bias)
    lib = _lib.load()
    bq.set_tuning(0, 512)
    bq.set_tuning(2, tn)
    bq.set_tuning(5, 8)
    try:
        if out == "bf16":
            sa = rng.uniform(0.001, 0.01, size=m).astype(np.float32)
            sb = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
            want = oracle.epilogue_chain(oracle.dequant_s32_f32(acc, sa, sb), bias, epi)
            d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            sad, sbd = dev(sa), dev(sb)
            st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_epilogue_run(
                m, n, k, ad.data_ptr(), lda, bd.data_ptr(), lda, None, 0, d.data_ptr(), n, sad.data_ptr(), sbd.data_ptr(), 1,
                biasd.data_ptr(), epi, 1.0, 0.0, None, 0, _stream())
            assert st == 0
            _status_clean()
            got = d.float().cpu().numpy()
            assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-6)
        else:
            alpha = np.float32(2.0 ** -9)
            want = oracle.sat_s8(oracle.epilogue_chain(alpha * acc.astype(np.float32), bias, epi))
            d = torch.full((m, n), 99, dtype=torch.int8, device="cuda")
            st = lib.baracuda_kernels_gemm_s8_rcr_sm100a_epilogue_run(
                m, n, k, ad.data_ptr(), lda, bd.data_ptr(), lda, None, 0, d.data_ptr(), n, biasd.data_ptr(), 1, epi,
                float(alpha), 0.0, None, 0, _stream())
            assert st == 0
            _status_clean()
            diff = np.abs(d.cpu().numpy().astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).mean() < 0.01
    finally:
        bq.set_tuning(0, 0)
        bq.set_tuning(2, 0)
        bq.set_tuning(5, 0)
