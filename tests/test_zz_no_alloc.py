"""The allocation-free GEMV entry point (scratch inside the library image) against the regular
workspace entry point, through the C ABI.  Collected last on purpose: if it fails, every other
test has already run."""
import numpy as np
import pytest
import torch

from baracuda_b200 import _lib

pytestmark = pytest.mark.gpu

REGULAR = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_run"
STATIC = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run"


def _case(m, n, k, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    x = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)
    w = torch.randint(-127, 128, (k, n), dtype=torch.int8, device="cuda", generator=g)  # row-major [K, N]
    sa = torch.rand(m, device="cuda", generator=g) * 0.01
    sb = torch.rand(n, device="cuda", generator=g) * 0.001
    return x, w, sa, sb


def _call_regular(lib, m, n, k, x, w, sa, sb):
    need = lib.baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(m, n, k, 1, 0)
    assert need > 0, "the shape must be one that uses scratch"
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    st = getattr(lib, REGULAR)(m, n, k, 1, 0, 1.0, 0.0, x.data_ptr(), k, 0, w.data_ptr(), n, 0, sa.data_ptr(), 0,
                               sb.data_ptr(), 0, d.data_ptr(), n, 0, ws.data_ptr(), need,
                               torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return d


def _call_static(lib, m, n, k, x, w, sa, sb):
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    st = getattr(lib, STATIC)(m, n, k, 1, 0, 1.0, 0.0, x.data_ptr(), k, 0, w.data_ptr(), n, 0, sa.data_ptr(), 0,
                              sb.data_ptr(), 0, d.data_ptr(), n, 0, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return d


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    """Two different problems back to back through the allocation-free entry point: the second call
    inherits the first call's scratch contents and must still be exact (0 differing bf16 bit patterns,
    the tolerance of the other GEMV tests)."""
    lib = _lib.load()
    torch.cuda.set_device(0)
    for seed, (m, n, k) in enumerate([(1, 14336, 4096), (4, 4096, 14336)]):
        x, w, sa, sb = _case(m, n, k, seed)
        want = _call_regular(lib, m, n, k, x, w, sa, sb)
        got = _call_static(lib, m, n, k, x, w, sa, sb)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, n, k)
        assert not torch.isnan(got.float()).any()
    # same problem again: stale partial sums and tickets from the previous call must not leak in
    again = _call_static(lib, m, n, k, x, w, sa, sb)
    torch.cuda.synchronize()
    assert torch.equal(again.view(torch.int16), want.view(torch.int16))


def test_static_scratch_limit_is_enforced():
    lib = _lib.load()
    cap = lib.baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity()
    assert cap == 8 << 20
    m, n, k = 8, 65536, 8192  # needs more split-K scratch than the fixed array holds
    assert lib.baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size(m, n, k, 1, 0) > cap
    st = getattr(lib, STATIC)(m, n, k, 1, 0, 1.0, 0.0, 16, k, 0, 16, n, 0, 16, 0, 16, 0, 16, n, 0, None)
    assert st == 4
