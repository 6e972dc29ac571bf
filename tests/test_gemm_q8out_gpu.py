"""GPU parity of the 8-bit-out GEMM symbols that keep the reference's own IntGemm / Fp8Gemm contract
(D = sat(alpha*(A x B) + beta*C), D in the input type), on the reference's smoke patterns and shapes.
The reference accepts +-1 code (int8) / one e4m3 grid step against its in-file CPU loop; here the int8 output
must equal the oracle's restatement of that loop exactly, and the e4m3 output must sit within one grid step."""
import numpy as np
import pytest
import torch

from baracuda_b200 import _lib
from helpers import dev, pad_rows

pytestmark = pytest.mark.gpu


def _call(sym, m, n, k, a, lda, b, ldb, c, ldc, d, ldd, alpha, beta):
    lib = _lib.load()
    st = getattr(lib, sym)(m, n, k, a.data_ptr(), lda, b.data_ptr(), ldb, None if c is None else c.data_ptr(), ldc,
                           d.data_ptr(), ldd, alpha, beta, None, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert lib.baracuda_kernels_q_device_status() == 0
    return st


@pytest.mark.parametrize("shape", [(64, 64, 32), (128, 128, 128), (256, 128, 64), (100, 70, 50), (1024, 1536, 512)])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_s8_out_reference_contract(oracle, shape, beta):
    """crates/baracuda-kernels/tests/int8_rrr_smoke.rs:159-172, 442-500 (patterns, alpha = 0.125) read as RCR
    operands (crates/baracuda-cutlass/tests/int8_smoke.rs:85-124)."""
    m, n, k = shape
    a = np.array([((i * 7) % 15) - 7 for i in range(m * k)], dtype=np.int8).reshape(m, k)
    b = np.array([((i * 11) % 13) - 6 for i in range(k * n)], dtype=np.int8).reshape(n, k)
    c = np.array([((i * 5) % 17) - 8 for i in range(m * n)], dtype=np.int8).reshape(m, n)
    ld = (k + 15) // 16 * 16
    want = oracle.int_gemm_s8_out(a, b, oracle.RCR, m, n, k, alpha=0.125, beta=beta, c=c if beta else None)
    d = torch.full((m, n), 99, dtype=torch.int8, device="cuda")
    st = _call("baracuda_kernels_gemm_s8_rcr_sm100a_run", m, n, k, dev(pad_rows(a, ld)), ld, dev(pad_rows(b, ld)), ld,
               dev(c) if beta else None, n, d, n, 0.125, beta)
    assert st == 0
    assert np.array_equal(d.cpu().numpy(), want)


def test_s8_out_saturates(oracle):
    m, n, k = 128, 128, 256
    a = np.full((m, k), 127, dtype=np.int8)
    b = np.full((n, k), 127, dtype=np.int8)
    b[::2] = -127
    d = torch.zeros((m, n), dtype=torch.int8, device="cuda")
    assert _call("baracuda_kernels_gemm_s8_rcr_sm100a_run", m, n, k, dev(a), k, dev(b), k, None, 0, d, n, 1.0, 0.0) == 0
    got = d.cpu().numpy()
    assert np.all(got[:, 1::2] == 127) and np.all(got[:, 0::2] == -128)


@pytest.mark.parametrize("shape", [(64, 64, 32), (128, 128, 128), (256, 128, 64), (100, 70, 50)])
def test_e4m3_out_reference_contract(oracle, shape):
    """crates/baracuda-kernels/tests/fp8_e4m3_rcr_smoke.rs:66-127, 193-247: alpha = 0.25, tolerance one e4m3 grid step."""
    m, n, k = shape
    av = np.array([(((i * 5) % 13) - 6) * 0.125 for i in range(m * k)], dtype=np.float32).reshape(m, k)
    bv = np.array([(((i * 7) % 11) - 5) * 0.125 for i in range(k * n)], dtype=np.float32).reshape(n, k)
    a_bits, b_bits = oracle.f32_to_e4m3(av), oracle.f32_to_e4m3(bv)
    ld = (k + 15) // 16 * 16
    acc = oracle.gemm_e4m3_f32(a_bits, b_bits, oracle.RCR, m, n, k)
    want_bits = oracle.f32_to_e4m3(np.float32(0.25) * acc)
    d = torch.zeros((m, n), dtype=torch.uint8, device="cuda")
    st = _call("baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run", m, n, k, dev(pad_rows(a_bits, ld)), ld,
               dev(pad_rows(b_bits, ld)), ld, None, 0, d, n, 0.25, 0.0)
    assert st == 0
    table = oracle.e4m3_decode_table()
    got_f, want_f = table[d.cpu().numpy()], table[want_bits]
    # the sums are exact in f32 for these patterns, so the codes are in fact equal; the reference's rule is one grid step
    assert np.array_equal(got_f, want_f)


def test_q8_out_status_rules():
    lib = _lib.load()
    z = torch.zeros(4096, dtype=torch.int8, device="cuda")
    run = lib.baracuda_kernels_gemm_s8_rcr_sm100a_run
    s = torch.cuda.current_stream().cuda_stream
    assert run(16, 16, 16, z.data_ptr(), 16, z.data_ptr(), 16, None, 0, z.data_ptr(), 16, 1.0, 0.5, None, 0, s) == 2  # beta needs C
    assert run(16, 16, 16, z.data_ptr(), 16, z.data_ptr(), 16, z.data_ptr(), 8, z.data_ptr(), 16, 1.0, 0.5, None, 0, s) == 2  # ldc < n
    assert run(0, 16, 16, None, 16, None, 16, None, 0, None, 16, 1.0, 0.0, None, 0, s) == 0  # empty
    assert lib.baracuda_kernels_gemm_s8_rcr_sm100a_workspace_size(16, 16, 16) == 0
