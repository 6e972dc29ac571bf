"""One-GPU parity of the K-sharded (row-parallel) entry points: the two K slices of a problem are run as world-1
calls without the collective, their raw accumulators are added by hand and dequantised through the library's own pass,
and a plain world-1 call must equal the unsharded GEMM bit for bit."""
import numpy as np
import pytest
import torch

import baracuda_b200 as bq
from baracuda_b200 import _lib
from baracuda_b200 import parallel as par
from helpers import bf16_bits, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["w8a8", "fp8"])
@pytest.mark.parametrize("shape", [(300, 1040, 512), (128, 70, 64), (1024, 2048, 1024)])
def test_world_one_equals_the_fused_gemm(oracle, kind, shape):
    m, n, k = shape
    rng = np.random.default_rng(21)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    if kind == "w8a8":
        aq, sa = oracle.quantize_rows_s8(a)
        wq, sb = oracle.quantize_rows_s8(w)
        y = oracle.dequant_s32_f32(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k), sa, sb)
        fused = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(m, n, k))
    else:
        aq, sa = oracle.quantize_rows_e4m3(a)
        wq, sb = oracle.quantize_rows_e4m3(w)
        y = ((sa[:, None] * sb[None, :]).astype(np.float32) * oracle.gemm_e4m3_f32(aq, wq, oracle.RCR, m, n, k)).astype(np.float32)
        fused = bq.Fp8ScaledGemmPlan.select(None, bq.QGemmDescriptor(m, n, k), scale_mode=bq.SCALE_PER_ROW_COL)
    ld = (k + 15) // 16 * 16
    pad = lambda x: np.pad(x, ((0, 0), (0, ld - k)))
    ctx = par.TensorParallelContext(0, 1)
    plan = par.RowParallelQGemmPlan(ctx, m, n, k, kind=kind, reduce=par.REDUCE_NONE)
    assert plan.workspace_size() == m * n * 4
    ws = torch.empty(plan.workspace_size(), dtype=torch.uint8, device="cuda")
    a_d, w_d, sa_d, sb_d, bias_d = dev(aq), dev(wq), dev(sa), dev(sb), dev(bias)
    if ld != k:
        pytest.skip("the plan passes tight pitches")  # shapes above keep K a multiple of 16
    y_d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    plan.forward(None, a_d, sa_d, w_d, sb_d, y_d, ws)
    ref = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    fused.run(None, None, bq.QGemmArgs(a=a_d, b=w_d, d=ref, scale_a=sa_d, scale_b=sb_d))
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(y_d), bf16_bits(ref))  # same accumulators, same product order
    # with a bias, against the oracle
    plan.forward(None, a_d, sa_d, w_d, sb_d, y_d, ws, bias=bias_d)
    torch.cuda.synchronize()
    want = oracle.f32_to_bf16_bits((y + bias[None, :]).astype(np.float32))
    if kind == "w8a8":
        assert np.array_equal(bf16_bits(y_d), want)
    else:
        got_f, want_f = oracle.bf16_bits_to_f32(bf16_bits(y_d)), oracle.bf16_bits_to_f32(want)
        assert oracle.compare_tolerant(want_f, got_f, 1e-2, 1e-4 * float(np.abs(want_f).max())) == -1
    assert bq.device_status() == 0


def test_two_k_slices_add_up_exactly(oracle):
    """What the all-reduce does between the ranks, done by hand on one GPU: int32 partial sums of the two K halves add
    to the unsharded sums."""
    m, n, k = 256, 512, 1024
    rng = np.random.default_rng(3)
    aq = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    wq = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    want = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    lib = _lib.load()
    total = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    for r in range(2):
        a_l = par.shard_cols(torch.from_numpy(aq), 2, r).cuda()
        w_l = par.shard_cols(torch.from_numpy(wq), 2, r).cuda()
        part = torch.zeros((m, n), dtype=torch.int32, device="cuda")
        st = lib.baracuda_kernels_gemm_s8_rcr_s32_sm100a_run(m, n, k // 2, a_l.data_ptr(), k // 2, w_l.data_ptr(), k // 2, None, 0,
                                                              part.data_ptr(), n, 1.0, 0.0, None, 0,
                                                              torch.cuda.current_stream().cuda_stream)
        assert st == 0
        total += part
    torch.cuda.synchronize()
    assert np.array_equal(total.cpu().numpy(), want)


def test_kshard_status_rules():
    lib = _lib.load()
    z = torch.zeros(1 << 16, dtype=torch.int8, device="cuda")
    f = torch.ones(256, dtype=torch.float32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    run = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run
    args = (64, 64, 64, z.data_ptr(), 64, z.data_ptr(), 64, z.data_ptr(), 64, f.data_ptr(), f.data_ptr(), None, 1.0)
    assert run(0, 1, None, 0, *args, None, 0, s) == 4                       # no workspace
    assert run(0, 1, None, 0, *args, z.data_ptr(), 64 * 64 * 4 - 1, s) == 4  # too small
    assert run(0, 2, None, 1, *args, z.data_ptr(), 64 * 64 * 4, s) == 2      # a collective without a communicator
    assert run(2, 2, None, 0, *args, z.data_ptr(), 64 * 64 * 4, s) == 2      # rank outside the world
    assert run(0, 1, None, 7, *args, z.data_ptr(), 64 * 64 * 4, s) == 2      # unknown reduce mode
    assert run(0, 1, None, 0, *args, z.data_ptr(), 64 * 64 * 4, s) == 0
    torch.cuda.synchronize()
