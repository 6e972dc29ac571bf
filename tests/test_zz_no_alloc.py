"""The allocation-free GEMV entry point (scratch inside the library image) against the regular
workspace entry point and the CPU oracle, through the C ABI.  Collected last on purpose: if it
fails, every other test has already run."""
import ctypes

import numpy as np
import pytest
import torch

import baracuda_b200 as bq
from baracuda_b200 import _lib

pytestmark = pytest.mark.gpu

REGULAR = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_run"
STATIC = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run"
WS_SIZE = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size"


def _case(m, n, k, seed, batch=1, device="cuda"):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randint(-127, 128, (batch, m, k), dtype=torch.int8, device=device, generator=g)
    w = torch.randint(-127, 128, (batch, k, n), dtype=torch.int8, device=device, generator=g)  # row-major [K, N] per slot
    sa = torch.rand((batch, m), device=device, generator=g) * 0.01
    sb = torch.rand((batch, n), device=device, generator=g) * 0.001
    return x, w, sa, sb


def _args(m, n, k, batch, x, w, sa, sb, d):
    return (m, n, k, batch, 0, 1.0, 0.0, x.data_ptr(), k, m * k, w.data_ptr(), n, k * n, sa.data_ptr(), m,
            sb.data_ptr(), n, d.data_ptr(), n, m * n)


def _call_regular(lib, m, n, k, x, w, sa, sb, batch=1):
    need = getattr(lib, WS_SIZE)(m, n, k, batch, 0)
    assert need > 0, "the shape must be one that uses scratch"
    ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    d = torch.full((batch, m, n), float("nan"), dtype=torch.bfloat16, device=x.device)
    st = getattr(lib, REGULAR)(*_args(m, n, k, batch, x, w, sa, sb, d), ws.data_ptr(), need,
                               torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return d


def _call_static(lib, m, n, k, x, w, sa, sb, batch=1, d=None):
    if d is None:
        d = torch.full((batch, m, n), float("nan"), dtype=torch.bfloat16, device=x.device)
    st = getattr(lib, STATIC)(*_args(m, n, k, batch, x, w, sa, sb, d), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return d


def _oracle_bits(oracle, m, n, k, x, w, sa, sb):
    """bf16 bit patterns the CPU oracle gives for batch slot 0."""
    w_nk = np.ascontiguousarray(w[0].cpu().numpy().T)
    acc = oracle.gemm_s8_s32(x[0].cpu().numpy(), w_nk, oracle.RCR, m, n, k)
    return oracle.dequant_s32_bf16(acc, sa[0].cpu().numpy(), sb[0].cpu().numpy())


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _free_bytes():
    free, _ = torch.cuda.mem_get_info()
    return free


def test_static_scratch_entry_matches_workspace_entry_and_oracle_twice_in_a_row(oracle):
    """Two different problems back to back through the allocation-free entry point: the second call
    inherits the first call's scratch contents and must still be exact (0 differing bf16 bit patterns,
    the tolerance of the other GEMV tests), against the regular entry point and against the oracle."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    for seed, (m, n, k) in enumerate([(1, 14336, 4096), (4, 4096, 14336)]):
        x, w, sa, sb = _case(m, n, k, seed)
        want = _call_regular(lib, m, n, k, x, w, sa, sb)
        got = _call_static(lib, m, n, k, x, w, sa, sb)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, n, k)
        assert np.array_equal(_bits(got[0]), _oracle_bits(oracle, m, n, k, x, w, sa, sb)), (m, n, k)
    # same problem again: stale partial sums and tickets from the previous call must not leak in
    again = _call_static(lib, m, n, k, x, w, sa, sb)
    torch.cuda.synchronize()
    assert torch.equal(again.view(torch.int16), want.view(torch.int16))
    assert bq.device_status() == 0


def test_static_scratch_entry_allocates_nothing():
    """The claim itself: after one warm call, the device's free memory (the driver's figure, which sees allocations by
    any route) is the same before and after a run of calls."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    m, n, k = 2, 14336, 4096
    x, w, sa, sb = _case(m, n, k, 7)
    d = torch.empty((1, m, n), dtype=torch.bfloat16, device="cuda")
    _call_static(lib, m, n, k, x, w, sa, sb, d=d)  # first call on the device: address lookup, module load
    torch.cuda.synchronize()
    before = _free_bytes()
    for _ in range(16):
        _call_static(lib, m, n, k, x, w, sa, sb, d=d)
    torch.cuda.synchronize()
    assert _free_bytes() == before


@pytest.mark.parametrize("variant", [0, 8])  # automatic (streaming kernel), direct-load kernel (tickets in the scratch)
def test_static_scratch_every_row_major_kernel_twice(oracle, variant):
    """Every kernel that takes scratch, twice in a row on the shared array: the direct-load kernel keeps tickets
    there that must be cleared per call, the streaming kernels partial rows."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    m, n, k = 3, 2048, 4096
    x, w, sa, sb = _case(m, n, k, 11 + variant)
    want = _oracle_bits(oracle, m, n, k, x, w, sa, sb)
    bq.set_tuning(1, variant)
    try:
        for _ in range(2):
            got = _call_static(lib, m, n, k, x, w, sa, sb)
            torch.cuda.synchronize()
            assert np.array_equal(_bits(got[0]), want), variant
    finally:
        bq.set_tuning(1, 0)
    assert bq.device_status() == 0


def test_static_scratch_strided_batch(oracle):
    """Distinct weights per batch slot (stride_b = K * N): the batched path, through the static scratch."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    m, n, k, batch = 2, 1024, 1024, 3
    x, w, sa, sb = _case(m, n, k, 21, batch=batch)
    want = _call_regular(lib, m, n, k, x, w, sa, sb, batch=batch)
    got = _call_static(lib, m, n, k, x, w, sa, sb, batch=batch)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert np.array_equal(_bits(got[0]), _oracle_bits(oracle, m, n, k, x, w, sa, sb))


def test_static_scratch_on_a_second_device(oracle):
    """The array's address is looked up per device: a call with device 1 current uses device 1's copy."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = _lib.load()
    m, n, k = 1, 4096, 4096
    with torch.cuda.device(1):
        x, w, sa, sb = _case(m, n, k, 31, device="cuda:1")
        got = _call_static(lib, m, n, k, x, w, sa, sb)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(got[0]), _oracle_bits(oracle, m, n, k, x, w, sa, sb))
    torch.cuda.set_device(0)


def test_static_scratch_limit_is_enforced():
    lib = _lib.load()
    cap = lib.baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity()
    assert cap == 8 << 20
    m, n, k = 8, 65536, 8192  # needs more split-K scratch than the fixed array holds
    assert getattr(lib, WS_SIZE)(m, n, k, 1, 0) > cap
    st = getattr(lib, STATIC)(m, n, k, 1, 0, 1.0, 0.0, 16, k, 0, 16, n, 0, 16, 0, 16, 0, 16, n, 0, None)
    assert st == 4
    # the envelope the header states: the decode shapes of an 8B-class model fit at every m <= 8
    for shape in ((8, 14336, 4096), (8, 4096, 14336), (8, 28672, 4096), (8, 6144, 4096)):
        assert getattr(lib, WS_SIZE)(*shape, 1, 0) <= cap, shape
