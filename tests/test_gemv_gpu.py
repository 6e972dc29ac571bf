"""GPU parity of the int8 decode GEMV, through the C ABI, against the CPU oracle.
Integer sums must match bit for bit; the bf16 outputs equal the oracle's
f32-dequant-then-RNE bit for bit as well (tolerance 0 ulp; the contract allows 1)."""
import numpy as np
import pytest
import torch

import baracuda_b200 as bq
from helpers import bf16_bits, dev, pad_rows, w8a8_case

pytestmark = pytest.mark.gpu

LAYOUTS = {"rcr": bq.LayoutSku.Rcr, "rrr": bq.LayoutSku.Rrr}


def _weights_for(layout, wq_nk):
    """wq_nk is the weight as [N,K]; RRR stores it [K,N]."""
    return wq_nk if layout is bq.LayoutSku.Rcr else np.ascontiguousarray(wq_nk.T)


def _run(m, n, k, layout, aq, wq_nk, sa, sb, raw, dependent_launch=False, **kw):
    desc = bq.GemvQ8Descriptor(m, n, k, batch=1, layout=layout)
    plan = bq.GemvQ8Plan.select(None, desc, raw_accumulators=raw)
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    d = torch.full((m, n), -7 if raw else float("nan"), dtype=torch.int32 if raw else torch.bfloat16, device="cuda")
    args = bq.GemvQ8Args(a=dev(aq), b=dev(_weights_for(layout, wq_nk)), d=d,
                         scale_a=None if raw else dev(sa), scale_b=None if raw else dev(sb), **kw)
    plan.run(None, ws, args, dependent_launch=dependent_launch)
    torch.cuda.synchronize()
    return d


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_decode_shape_bit_exact(oracle, layout, m):
    """K=4096, N=14336, m in {1,2,4,8}: the decode configuration at full size."""
    n, k = 14336, 4096
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=1235)
    acc_ref = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    lay = LAYOUTS[layout]
    acc = _run(m, n, k, lay, aq, wq, sa, sb, raw=True).cpu().numpy()
    assert oracle.compare_bitexact(acc_ref, acc) == -1
    out = _run(m, n, k, lay, aq, wq, sa, sb, raw=False)
    assert oracle.compare_bitexact(oracle.dequant_s32_bf16(acc_ref, sa, sb), bf16_bits(out)) == -1


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
@pytest.mark.parametrize("shape", [(1, 70, 50), (3, 100, 77), (1, 64, 32), (5, 1040, 2064), (8, 16, 16), (1, 1, 1),
                                   (2, 4112, 8208), (7, 528, 6000)])
def test_ragged_and_small_shapes(oracle, layout, shape):
    """Ragged shapes in the spirit of the reference's 100x70x50 case; both the streaming and the byte-load kernels."""
    m, n, k = shape
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=77 + n)
    acc_ref = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    lay = LAYOUTS[layout]
    acc = _run(m, n, k, lay, aq, wq, sa, sb, raw=True).cpu().numpy()
    assert oracle.compare_bitexact(acc_ref, acc) == -1
    out = _run(m, n, k, lay, aq, wq, sa, sb, raw=False)
    assert oracle.compare_bitexact(oracle.dequant_s32_bf16(acc_ref, sa, sb), bf16_bits(out)) == -1


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
def test_byte_load_kernel_equals_streaming_kernel(oracle, layout):
    m, n, k = 4, 2048, 1024
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=5)
    lay = LAYOUTS[layout]
    fast = _run(m, n, k, lay, aq, wq, sa, sb, raw=True).cpu().numpy()
    bq.set_tuning(1, 9)
    try:
        slow = _run(m, n, k, lay, aq, wq, sa, sb, raw=True).cpu().numpy()
    finally:
        bq.set_tuning(1, 0)
    assert np.array_equal(fast, slow)
    assert np.array_equal(fast, oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k))


@pytest.mark.parametrize("variant", [0, 1, 2, 3])  # automatic, bulk-copy dp4a, register streaming, tensor-core streaming
@pytest.mark.parametrize("shape", [(1, 300, 512), (2, 149, 4096), (3, 1000, 4112), (4, 2048, 9000 // 16 * 16), (1, 7, 16),
                                   (8, 520, 2048), (5, 1187, 8192), (7, 3000, 1088), (6, 2048, 1536), (2, 4096, 3072)])
def test_both_k_contiguous_kernels_on_the_same_shapes(oracle, shape, variant):
    """The bulk-copy streaming kernel (variant 1) and the register-streaming kernel (variant 2) are both
    exercised on shapes that include partial K chunks, several chunks per row and fewer columns than SMs; K = 1536 and
    3072 (three / six 512-byte chunks, which do not divide the warp count) and 1088 take the tensor-core kernel's
    staged-activation configuration, the other K its register-activation one."""
    m, n, k = shape
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=31 + n)
    acc_ref = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    bq.set_tuning(1, variant)
    try:
        acc = _run(m, n, k, bq.LayoutSku.Rcr, aq, wq, sa, sb, raw=True).cpu().numpy()
        out = _run(m, n, k, bq.LayoutSku.Rcr, aq, wq, sa, sb, raw=False)
    finally:
        bq.set_tuning(1, 0)
    assert bq.device_status() == 0
    assert oracle.compare_bitexact(acc_ref, acc) == -1
    assert oracle.compare_bitexact(oracle.dequant_s32_bf16(acc_ref, sa, sb), bf16_bits(out)) == -1


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("layout", ["rcr", "rrr"])
def test_padded_leading_dims_batch_broadcast_and_canaries(oracle, layout, variant):
    """Padded lda/ldb/ldd, strided batch with the weights broadcast (stride_b == 0, the reference's GQA use,
    gemv_dense_smoke.rs), and untouched padding between output rows and batch slots."""
    lay = LAYOUTS[layout]
    m, n, k, batch = 2, 272, 160, 3
    lda, ldd = k + 16, n + 24
    stride_a, stride_d, stride_sa = m * lda + 32, m * ldd + 40, m
    rng = np.random.default_rng(3)
    aq_all, sa_all = [], []
    for g in range(batch):
        aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=100 + g)
        aq_all.append(aq)
        sa_all.append(sa)
    _, wq, _, sb = w8a8_case(oracle, m, n, k, seed=100)
    a_buf = np.zeros(batch * stride_a, dtype=np.int8)
    for g in range(batch):
        a_buf[g * stride_a: g * stride_a + m * lda] = pad_rows(aq_all[g], lda, fill=55).ravel()
    if lay is bq.LayoutSku.Rcr:
        ldb = k + 32
        b_buf = pad_rows(wq, ldb, fill=-99).ravel()
    else:
        ldb = n + 16
        b_buf = pad_rows(np.ascontiguousarray(wq.T), ldb, fill=-99).ravel()
    d = torch.full((batch * stride_d,), 123.0, dtype=torch.bfloat16, device="cuda")
    desc = bq.GemvQ8Descriptor(m, n, k, batch=batch, layout=lay)
    plan = bq.GemvQ8Plan.select(None, desc)
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    args = bq.GemvQ8Args(a=dev(a_buf), b=dev(b_buf), d=d, scale_a=dev(np.concatenate(sa_all)), scale_b=dev(sb),
                         lda=lda, ldb=ldb, ldd=ldd, stride_a=stride_a, stride_b=0, stride_d=stride_d,
                         stride_scale_a=stride_sa, stride_scale_b=0)
    bq.set_tuning(1, variant)
    try:
        plan.run(None, ws, args)
        torch.cuda.synchronize()
    finally:
        bq.set_tuning(1, 0)
    got = bf16_bits(d)
    canary = bf16_bits(torch.tensor([123.0], dtype=torch.bfloat16))[0]
    touched = np.zeros(batch * stride_d, dtype=bool)
    for g in range(batch):
        acc = oracle.gemm_s8_s32(aq_all[g], wq, oracle.RCR, m, n, k)
        want = oracle.dequant_s32_bf16(acc, sa_all[g], sb)
        for r in range(m):
            lo = g * stride_d + r * ldd
            assert np.array_equal(got[lo: lo + n], want[r]), (g, r)
            touched[lo: lo + n] = True
    assert np.all(got[~touched] == canary), "padding between rows / batch slots was clobbered"


def test_alpha_beta(oracle):
    """D = alpha*(sa*sb*acc) + beta*D, each product and the sum rounded in f32 (gemv_dense.cu FFI contract)."""
    m, n, k = 2, 512, 256
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=9)
    acc = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    d0 = (np.random.default_rng(1).standard_normal((m, n))).astype(np.float32)
    d0_bf = torch.from_numpy(d0).to(torch.bfloat16)
    alpha, beta = np.float32(0.75), np.float32(-1.5)
    y = (sa[:, None] * sb[None, :]) * acc.astype(np.float32)
    y = (y * alpha).astype(np.float32) + (beta * d0_bf.to(torch.float32).numpy()).astype(np.float32)
    want = bf16_bits(torch.from_numpy(y.astype(np.float32)).to(torch.bfloat16))
    for lay in (bq.LayoutSku.Rcr, bq.LayoutSku.Rrr):
        plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=lay))
        ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
        d = d0_bf.clone().cuda()
        b = wq if lay is bq.LayoutSku.Rcr else np.ascontiguousarray(wq.T)
        plan.run(None, ws, bq.GemvQ8Args(a=dev(aq), b=dev(b), d=d, scale_a=dev(sa), scale_b=dev(sb),
                                         alpha=float(alpha), beta=float(beta)))
        torch.cuda.synchronize()
        assert np.array_equal(bf16_bits(d), want)


def test_workspace_contract():
    plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(1, 14336, 4096, layout=bq.LayoutSku.Rrr))
    assert plan.workspace_size() > 0
    z8 = torch.zeros(14336 * 4096, dtype=torch.int8, device="cuda")
    args = bq.GemvQ8Args(a=z8[:4096], b=z8, d=torch.zeros(14336, dtype=torch.bfloat16, device="cuda"),
                         scale_a=torch.ones(1, device="cuda"), scale_b=torch.ones(14336, device="cuda"))
    with pytest.raises(bq.WorkspaceTooSmall):
        plan.run(None, None, args)
    # the flat symbol reports status 4 as well
    from baracuda_b200 import _lib
    st = _lib.load().baracuda_kernels_gemv_q8_m1_bf16_sm100a_run(
        1, 14336, 4096, 1, 0, 1.0, 0.0, args.a.data_ptr(), 4096, 0, args.b.data_ptr(), 14336, 0,
        args.scale_a.data_ptr(), 0, args.scale_b.data_ptr(), 0, args.d.data_ptr(), 14336, 0, None, 0,
        torch.cuda.current_stream().cuda_stream)
    assert st == 4


def test_dependent_launch_mode_gives_the_same_results(oracle):
    """Programmatic dependent launch, selected per call (the *_pdl_run symbols): a chain of GEMVs on one stream over
    static weights equals the same chain launched normally."""
    m, n, k = 2, 4096, 4096
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=44)
    want = oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k), sa, sb)
    plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=bq.LayoutSku.Rcr))
    a_d, b_d, sa_d, sb_d = dev(aq), dev(wq), dev(sa), dev(sb)
    outs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(6)]
    for d in outs:
        plan.run(None, None, bq.GemvQ8Args(a=a_d, b=b_d, d=d, scale_a=sa_d, scale_b=sb_d), dependent_launch=True)
    torch.cuda.synchronize()
    assert bq.device_status() == 0
    for d in outs:
        assert np.array_equal(bf16_bits(d), want)


@pytest.mark.parametrize("variant", [0, 8])  # automatic (row-run streaming kernel), direct-load split-K kernel
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (2, 1040, 2064), (3, 272, 1000), (5, 14336, 512), (8, 2048, 4100),
                                   (7, 528, 8192), (1, 16, 16400), (4, 14336, 4096), (2, 32768, 8192), (1, 65536, 8192),
                                   (3, 1040, 30), (2, 2064, 33), (6, 48, 20000)])
def test_both_row_major_weight_kernels_on_the_same_shapes(oracle, shape, variant):
    """Weights row-major [K, N] (the reference GEMV's layout, gemv_dense.cu:128-171): int32 sums are exact whichever
    kernel runs; ragged K (not a multiple of the 32-row stage, shorter than one stage), N that is not a multiple of the
    1024-column strip, K so long that the run crosses several strips' worth of stages, and 65536 x 8192, which the
    streaming kernel serves with two waves of CTAs."""
    m, n, k = shape
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=m * 1000 + n + k)
    want = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    bq.set_tuning(1, variant)
    try:
        got = _run(m, n, k, bq.LayoutSku.Rrr, aq, wq, sa, sb, raw=True).cpu().numpy()
        got_bf = bf16_bits(_run(m, n, k, bq.LayoutSku.Rrr, aq, wq, sa, sb, raw=False))
    finally:
        bq.set_tuning(1, 0)
    assert bq.device_status() == 0
    assert np.array_equal(got, want)
    assert np.array_equal(got_bf, oracle.dequant_s32_bf16(want, sa, sb))


@pytest.mark.parametrize("shape", [(4, 14336, 4096), (8, 1024, 640), (1, 4096, 14336)])
def test_row_major_weights_tensor_core_kernel_in_a_dependent_chain(oracle, shape):
    """The tcgen05 kernel and its reduce kernel chained with programmatic stream serialization, several launches with
    different activations sharing one workspace: a launch may not overwrite partial rows the previous reduce still reads."""
    m, n, k = shape
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=31 + m)
    rng = np.random.default_rng(m)
    acts = [aq] + [rng.integers(-127, 128, size=(m, k), dtype=np.int8) for _ in range(3)]
    wants = [oracle.dequant_s32_bf16(oracle.gemm_s8_s32(a, wq, oracle.RCR, m, n, k), sa, sb) for a in acts]
    plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=bq.LayoutSku.Rrr))
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    b_d, sa_d, sb_d = dev(np.ascontiguousarray(wq.T)), dev(sa), dev(sb)
    a_ds = [dev(a) for a in acts]
    for pdl in (0, 1):
        outs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in acts]
        for rep in range(3):
            for a_d, d in zip(a_ds, outs):
                plan.run(None, ws, bq.GemvQ8Args(a=a_d, b=b_d, d=d, scale_a=sa_d, scale_b=sb_d), dependent_launch=bool(pdl))
        torch.cuda.synchronize()
        assert bq.device_status() == 0
        for d, want in zip(outs, wants):
            assert np.array_equal(bf16_bits(d), want), pdl


def test_row_major_weights_strided_batch_and_dependent_launches(oracle):
    """Distinct weights per batch entry (stride_b = K * ldb) through the streaming kernel, launched as a chain with
    programmatic stream serialization on one shared workspace."""
    m, n, k, batch = 2, 1024, 1024, 3
    cases = [w8a8_case(oracle, m, n, k, seed=700 + g) for g in range(batch)]
    a_buf = np.concatenate([c[0].ravel() for c in cases])
    b_buf = np.concatenate([np.ascontiguousarray(c[1].T).ravel() for c in cases])
    sa_buf = np.concatenate([c[2] for c in cases])
    sb_buf = np.concatenate([c[3] for c in cases])
    plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, batch=batch, layout=bq.LayoutSku.Rrr))
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    a_d, b_d, sa_d, sb_d = dev(a_buf), dev(b_buf), dev(sa_buf), dev(sb_buf)
    outs = [torch.full((batch, m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    for pdl in (0, 1):
        for d in outs:
            d.fill_(float("nan"))
            plan.run(None, ws, bq.GemvQ8Args(a=a_d, b=b_d, d=d, scale_a=sa_d, scale_b=sb_d, stride_a=m * k,
                                             stride_b=k * n, stride_d=m * n, stride_scale_a=m, stride_scale_b=n),
                     dependent_launch=bool(pdl))
        torch.cuda.synchronize()
        assert bq.device_status() == 0
        for d in outs:
            for g, (aq, wq, sa, sb) in enumerate(cases):
                want = oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k), sa, sb)
                assert np.array_equal(bf16_bits(d[g]), want), (pdl, g)


def test_bounded_wait_gives_up_and_the_context_survives(oracle):
    """Failure detection without a fault: a barrier wait that nothing completes runs out of its (short) cycle budget,
    the kernel records status 299 and ends, and the next launches on the same context work and report no status."""
    from baracuda_b200 import _lib
    lib = _lib.load()
    s = torch.cuda.current_stream().cuda_stream
    assert lib.baracuda_kernels_q_selftest_bounded_wait(0, s) == 2          # budget out of range
    assert lib.baracuda_kernels_q_selftest_bounded_wait(1 << 40, s) == 2
    assert lib.baracuda_kernels_q_selftest_bounded_wait(2_000_000, s) == 0  # about a millisecond
    torch.cuda.synchronize()
    assert bq.device_status() == 299
    assert bq.device_status() == 0  # read-and-clear
    m, n, k = 1, 1024, 1024
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=5)
    got = bf16_bits(_run(m, n, k, bq.LayoutSku.Rcr, aq, wq, sa, sb, raw=False))
    assert np.array_equal(got, oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k), sa, sb))
    assert bq.device_status() == 0


@pytest.mark.parametrize("layout", ["rcr", "rrr"])
def test_graph_capture_and_replay(oracle, layout):
    """The reason the reference's GEMV exists (gemv_dense.cu:6-12; tests/capture_replay_gather_gemv.rs): the call records
    into a CUDA graph -- no allocation, no host sync -- and replays read the buffers' current contents."""
    lay = LAYOUTS[layout]
    m, n, k = 1, 4096, 4096
    cases = [w8a8_case(oracle, m, n, k, seed=900 + i) for i in range(2)]
    wq, sb = cases[0][1], cases[0][3]
    plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=lay))
    ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
    a_d, sa_d = dev(cases[0][0]), dev(cases[0][2])
    b_d, sb_d = dev(_weights_for(lay, wq)), dev(sb)
    d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    args = bq.GemvQ8Args(a=a_d, b=b_d, d=d, scale_a=sa_d, scale_b=sb_d)
    plan.run(None, ws, args)  # first call outside the capture: one-time function attributes
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            plan.run(side, ws, args)
    for aq, _, sa, _ in cases[::-1]:
        a_d.copy_(dev(aq))
        sa_d.copy_(dev(sa))
        d.zero_()
        graph.replay()
        torch.cuda.synchronize()
        want = oracle.dequant_s32_bf16(oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k), sa, sb)
        assert np.array_equal(bf16_bits(d), want)
    assert bq.device_status() == 0


@pytest.mark.parametrize("shape", [(2, 1024, 14336), (8, 4096, 14336), (3, 520, 16384), (4, 1000, 7168), (1, 2048, 14336)])
def test_k_contiguous_weights_long_k(oracle, shape):
    """K = 14336 / 16384 (two K chunks per warp in the register-activation kernel) and 7168 (448-byte chunks), with and
    without dependent launch (which also routes m = 1 to that kernel)."""
    m, n, k = shape
    aq, wq, sa, sb = w8a8_case(oracle, m, n, k, seed=n + k + m)
    acc = oracle.gemm_s8_s32(aq, wq, oracle.RCR, m, n, k)
    want = oracle.dequant_s32_bf16(acc, sa, sb)
    for pdl in (0, 1):
        got_raw = _run(m, n, k, bq.LayoutSku.Rcr, aq, wq, sa, sb, raw=True, dependent_launch=bool(pdl)).cpu().numpy()
        got = bf16_bits(_run(m, n, k, bq.LayoutSku.Rcr, aq, wq, sa, sb, raw=False, dependent_launch=bool(pdl)))
        assert bq.device_status() == 0
        assert np.array_equal(got_raw, acc), (shape, pdl)
        assert np.array_equal(got, want), (shape, pdl)
