"""Host-side checks that need no GPU: the C-ABI library loads and exports every
symbol the header declares, the pure-host validators follow the reference's
status contract, and the typed plans validate / identify themselves."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import baracuda_b200 as bq
from baracuda_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
W8A8 = "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a"
GEMV = "baracuda_kernels_gemv_q8_m1_bf16_sm100a"


def _declared_symbols():
    text = (ROOT / "include" / "baracuda_kernels_q.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(baracuda_\w+)\s*\(", text))
    # whole prototypes declared through a BARACUDA_Q_DECLARE_*_RUN(symbol) macro
    names.update(re.findall(r"^BARACUDA_Q_DECLARE_\w*RUN\((baracuda_\w+)\)", text, flags=re.M))
    # the _workspace_size / _can_implement pair declared through BARACUDA_Q_DECLARE_GEMM_TAIL(NAME)
    for base in re.findall(r"^BARACUDA_Q_DECLARE_GEMM_TAIL\((baracuda_\w+)\)", text, flags=re.M):
        names.update({base + "_workspace_size", base + "_can_implement"})
    return sorted(names)


def test_library_exports_every_declared_symbol(qlib):
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(qlib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes prototype"
    assert sorted(_lib.SIGNATURES) == names


def test_gemm_can_implement_status_table(qlib):
    can = getattr(qlib, W8A8 + "_can_implement")
    A, B, D = 0x10000, 0x20000, 0x30000
    assert can(128, 256, 512, A, 512, B, 512, None, 0, D, 256) == 0
    assert can(-1, 256, 512, A, 512, B, 512, None, 0, D, 256) == 2          # negative dim
    assert can(128, 256, 512, A, 511, B, 512, None, 0, D, 256) == 2         # lda < k
    assert can(128, 256, 512, A, 512, B, 100, None, 0, D, 256) == 2         # ldb < k
    assert can(128, 256, 512, A, 512, B, 512, None, 0, D, 255) == 2         # ldd < n
    assert can(128, 256, 512, A + 4, 512, B, 512, None, 0, D, 256) == 1     # a not 16-byte aligned
    assert can(128, 256, 500, A, 500, B, 512, None, 0, D, 256) == 1         # lda not a multiple of 16
    assert can(128, 256, 500, A, 512, B, 512, None, 0, D, 256) == 0         # ragged k with padded pitch is fine
    assert can(128, 256, 512, A, 512, B, 512, D, 256, D, 256) == 0          # C (bf16, may be D) is accepted
    assert can(128, 256, 512, A, 512, B, 512, D, 255, D, 256) == 2          # ldc < n
    assert can(128, 256, 512, A, 512, B, 512, D + 1, 256, D, 256) == 1      # C not 2-byte aligned
    assert can(0, 0, 0, None, 1, None, 1, None, 0, None, 1) == 0            # empty
    assert getattr(qlib, W8A8 + "_workspace_size")(128, 256, 512) == 0


def test_gemv_can_implement_status_table(qlib):
    """Mirrors the rejection table of crates/baracuda-kernels/tests/gemv_dense_smoke.rs:399-432."""
    can = getattr(qlib, GEMV + "_can_implement")
    ok = dict(m=1, n=64, k=32, batch=1, layout=0, lda=32, ldb=64, ldd=64, sa=0, sb=0, sd=0)

    def call(**kw):
        a = {**ok, **kw}
        return can(a["m"], a["n"], a["k"], a["batch"], a["layout"], a["lda"], a["ldb"], a["ldd"], a["sa"], a["sb"], a["sd"])

    assert call() == 0
    assert call(m=0) == 0 and call(n=0, ldb=1, ldd=1) == 0
    assert call(m=8) == 0 and call(m=9) == 2
    assert call(m=-1) == 2 and call(batch=-1) == 2
    assert call(layout=2) == 2
    assert call(lda=31) == 2 and call(ldb=63) == 2 and call(ldd=63) == 2
    assert call(layout=1, ldb=32) == 0 and call(layout=1, ldb=31) == 2      # RCR: ldb >= k
    assert call(batch=4, sd=0) == 2 and call(batch=4, sd=64) == 0          # overlapping outputs
    ws = getattr(qlib, GEMV + "_workspace_size")
    assert ws(1, 14336, 4096, 1, 1) == 0                                    # K-contiguous weights: no scratch
    assert ws(1, 14336, 4096, 1, 0) > 0                                     # row-major weights: split-K scratch
    assert ws(0, 14336, 4096, 1, 0) == 0


def test_run_rejects_and_empty_without_a_gpu(qlib):
    run = getattr(qlib, W8A8 + "_run")
    # empty problem: status 0, nothing launched (no CUDA call is made)
    assert run(0, 256, 512, None, 512, None, 512, None, 0, None, 256, None, None, 1.0, 0.0, None, 0, None) == 0
    # null operands on a non-empty problem
    assert run(128, 256, 512, None, 512, None, 512, None, 0, None, 256, None, None, 1.0, 0.0, None, 0, None) == 2
    # beta != 0 needs C
    assert run(128, 256, 512, 0x1000, 512, 0x2000, 512, None, 0, 0x3000, 256, 0x4000, 0x5000, 1.0, 0.5, None, 0, None) == 2
    assert qlib.baracuda_kernels_q_set_tuning(0, 100) == 2
    assert qlib.baracuda_kernels_q_set_tuning(0, 0) == 0


def test_plan_select_and_sku():
    desc = bq.QGemmDescriptor(m=128, n=1024, k=1024)
    p = bq.W8A8GemmPlan.select(None, desc)
    s = p.sku()
    assert s.arch is bq.ArchSku.Sm100a and s.backend is bq.BackendKind.Bespoke
    assert s.layout is bq.LayoutSku.Rcr and s.element is bq.ElementKind.S8 and s.aux_element is bq.ElementKind.Bf16
    g = p.precision_guarantee()
    assert g.accumulator is bq.ElementKind.I32 and g.bit_stable_on_same_hardware and g.deterministic
    # sku is a usable cache key
    assert {s: 1}[bq.W8A8GemmPlan.select(None, desc).sku()] == 1
    assert bq.W8A8GemmPlan.select(None, desc, raw_accumulators=True).sku() != s
    f = bq.Fp8ScaledGemmPlan.select(None, desc, scale_mode=bq.SCALE_PER_ROW_COL)
    assert f.sku().element is bq.ElementKind.Fp8E4M3 and f.precision_guarantee().accumulator is bq.ElementKind.F32
    rrr = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(1, 1, 1, layout=bq.LayoutSku.Rrr))
    assert rrr.sku().layout is bq.LayoutSku.Rrr and rrr._run_symbol.endswith("s8_rrr_bf16_sm100a_run")
    with pytest.raises(bq.Unsupported):
        bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(1, 1, 1, epilogue=bq.EpilogueKind.BiasRelu), raw_accumulators=True)
    fused = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(1, 1, 1, epilogue=bq.EpilogueKind.BiasRelu))
    assert fused.sku().epilogue is bq.EpilogueKind.BiasRelu and fused.sku() != bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(1, 1, 1)).sku()
    with pytest.raises(bq.Unsupported):
        bq.W8A8GemmPlan.select(None, desc, bq.PlanPreference(prefer_backend=bq.BackendKind.Cublas))
    with pytest.raises(bq.InvalidProblem):
        bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(-1, 1, 1))
    gv = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(1, 14336, 4096, layout=bq.LayoutSku.Rcr))
    assert gv.workspace_size() == 0 and gv.sku().layout is bq.LayoutSku.Rcr
    with pytest.raises(bq.InvalidProblem):
        bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(9, 64, 64))
    with pytest.raises(bq.Unsupported):
        bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(1, 14336, 4096), bq.PlanPreference(max_workspace_bytes=16))


def test_typed_layer_refuses_short_buffers():
    """The typed layer owns buffer-length soundness (gemv_dense.rs:218-268)."""
    FakeCuda = _FakeCuda
    p = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(128, 256, 512))
    good = dict(a=FakeCuda(128 * 512, torch.int8), b=FakeCuda(256 * 512, torch.int8), d=FakeCuda(128 * 256, torch.bfloat16),
                scale_a=FakeCuda(128, torch.float32), scale_b=FakeCuda(256, torch.float32))
    p.can_implement(bq.QGemmArgs(**good))
    with pytest.raises(bq.BufferTooSmall):
        p.can_implement(bq.QGemmArgs(**{**good, "b": FakeCuda(256 * 512 - 1, torch.int8)}))
    with pytest.raises(bq.BufferTooSmall):
        p.can_implement(bq.QGemmArgs(**{**good, "scale_b": FakeCuda(255, torch.float32)}))
    with pytest.raises(bq.InvalidProblem):
        p.can_implement(bq.QGemmArgs(**{**good, "d": FakeCuda(128 * 256, torch.float16)}))
    with pytest.raises(bq.MisalignedOperand):
        p.can_implement(bq.QGemmArgs(**{**good, "lda": 520}))


class _FakeCuda:
    """Shape/dtype stand-in so the typed layer's checks run without a device."""
    def __init__(self, n, dtype, cuda=True):
        self._n, self.dtype, self.is_cuda = n, dtype, cuda
    def numel(self):
        return self._n
    def data_ptr(self):
        return 0x10000
    def element_size(self):
        return 1


def test_gemv_typed_layer_checks_scale_dtypes():
    """A bf16 scale vector of the right LENGTH is half the bytes the kernel reads: it must be refused, not overrun."""
    m, n, k = 4, 256, 512
    p = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=bq.LayoutSku.Rcr))
    good = dict(a=_FakeCuda(m * k, torch.int8), b=_FakeCuda(n * k, torch.int8), d=_FakeCuda(m * n, torch.bfloat16),
                scale_a=_FakeCuda(m, torch.float32), scale_b=_FakeCuda(n, torch.float32))
    p.can_implement(bq.GemvQ8Args(**good))
    for name, bad in (("scale_b", _FakeCuda(n, torch.bfloat16)), ("scale_a", _FakeCuda(m, torch.float16)),
                      ("scale_b", _FakeCuda(n, torch.float32, cuda=False)), ("scale_a", None)):
        with pytest.raises(bq.InvalidProblem):
            p.can_implement(bq.GemvQ8Args(**{**good, name: bad}))
    with pytest.raises(bq.BufferTooSmall):
        p.can_implement(bq.GemvQ8Args(**{**good, "scale_b": _FakeCuda(n - 1, torch.float32)}))


def test_fused_decode_branch_checks_dtypes(monkeypatch):
    m, n, k = 1, 1024, 4096
    lin = bq.QuantizedLinearPlan.select(None, bq.QuantizedLinearDescriptor(m, n, k))
    monkeypatch.setattr(lin, "fused_decode_ok", lambda args: True)
    good = dict(activation=_FakeCuda(m * k, torch.bfloat16), weight_q=_FakeCuda(n * k, torch.int8),
                weight_scale=_FakeCuda(n, torch.float32), output=_FakeCuda(m * n, torch.bfloat16),
                act_q_scratch=_FakeCuda(m * k, torch.int8), act_scale_scratch=_FakeCuda(m, torch.float32))
    for name, bad in (("weight_scale", _FakeCuda(n, torch.bfloat16)), ("weight_q", _FakeCuda(n * k, torch.uint8)),
                      ("act_scale_scratch", _FakeCuda(m, torch.float16)), ("output", _FakeCuda(m * n, torch.float32))):
        with pytest.raises(bq.InvalidProblem):
            lin.run(0, None, bq.QuantizedLinearArgs(**{**good, name: bad}))


def test_parallel_forwards_check_dtypes_and_scale_lengths():
    from baracuda_b200 import parallel as par

    ctx = par.TensorParallelContext(0, 2, comm=None)
    m, n, k = 64, 512, 256
    col = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind="w8a8")
    good = dict(a=_FakeCuda(m * k, torch.int8), scale_a=_FakeCuda(m, torch.float32), w_local=_FakeCuda(n // 2 * k, torch.int8),
                scale_b_local=_FakeCuda(n // 2, torch.float32), y_local=_FakeCuda(m * n // 2, torch.bfloat16))
    for name, bad in (("scale_a", _FakeCuda(m, torch.bfloat16)), ("scale_b_local", _FakeCuda(n // 2, torch.float16)),
                      ("y_local", _FakeCuda(m * n // 2, torch.float16)), ("a", _FakeCuda(m * k, torch.uint8))):
        with pytest.raises(bq.InvalidProblem):
            col.forward(0, **{**good, name: bad})
    with pytest.raises(bq.BufferTooSmall):
        col.forward(0, **{**good, "scale_b_local": _FakeCuda(n // 2 - 1, torch.float32)})
    with pytest.raises(bq.BufferTooSmall):
        col.forward(0, **{**good, "scale_a": _FakeCuda(m - 1, torch.float32)})
    row = par.RowParallelQGemmPlan(ctx, m, n, k, kind="w8a8")
    rgood = dict(a_local=_FakeCuda(m * k // 2, torch.int8), scale_a=_FakeCuda(m, torch.float32),
                 w_local=_FakeCuda(n * k // 2, torch.int8), scale_b=_FakeCuda(n, torch.float32),
                 y=_FakeCuda(m * n, torch.bfloat16), workspace=_FakeCuda(m * n * 4, torch.uint8))
    for name, bad in (("scale_b", _FakeCuda(n, torch.bfloat16)), ("y", _FakeCuda(m * n, torch.float32))):
        with pytest.raises(bq.InvalidProblem):
            row.forward(0, **{**rgood, name: bad})
    with pytest.raises(bq.BufferTooSmall):
        row.forward(0, **{**rgood, "scale_a": _FakeCuda(m - 1, torch.float32)})


def test_static_scratch_entry_validates_before_the_size_limit(qlib):
    """Invalid problems report the regular entry point's status (2), not the size limit's (4)."""
    run = qlib.baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run
    P = 0x10000
    n, k = 14336, 4096
    assert run(9, n, k, 1, 0, 1.0, 0.0, P, k, 0, P, n, 0, P, 0, P, 0, P, n, 0, None) == 2          # m > 8
    assert run(1, n, k, 1, 0, 1.0, 0.0, None, k, 0, P, n, 0, P, 0, P, 0, P, n, 0, None) == 2       # null a
    assert run(1, n, k, 1, 0, 1.0, 0.0, P, k, 0, P, n - 1, 0, P, 0, P, 0, P, n, 0, None) == 2      # ldb < n
    assert run(0, n, k, 1, 0, 1.0, 0.0, None, k, 0, None, n, 0, None, 0, None, 0, None, n, 0, None) == 0  # empty
    assert run(8, 65536, 8192, 1, 0, 1.0, 0.0, P, 8192, 0, P, 65536, 0, P, 0, P, 0, P, 65536, 0, None) == 4  # too large


def test_set_tuning_is_per_thread(qlib):
    """The test hooks are thread-local: a value forced on one thread is invisible to another."""
    import threading

    assert qlib.baracuda_kernels_q_set_tuning(3, 1) == 2  # the old process-wide dependent-launch switch is gone
    assert qlib.baracuda_kernels_q_set_tuning(1, 33) == 2  # removed experimental GEMV configurations
    assert qlib.baracuda_kernels_q_set_tuning(1, 9) == 0
    seen = []
    t = threading.Thread(target=lambda: seen.append(qlib.baracuda_kernels_q_set_tuning(1, 0)))
    t.start()
    t.join()
    assert seen == [0]
    assert qlib.baracuda_kernels_q_set_tuning(1, 0) == 0


def test_set_tuning_accepts_only_documented_values(qlib):
    """Every key of the test hook: the documented values return 0 (and are reset), anything else 2."""
    allowed = {0: (0, 64, 128, 256, 512), 1: (0, 1, 2, 3, 8, 9), 2: (0, 2, 256, 224, 192, 128), 4: (0, 1, 2), 5: (0, 4, 8),
               6: (0, 1, 2, 4, 256)}
    for key, values in allowed.items():
        for v in values:
            assert qlib.baracuda_kernels_q_set_tuning(key, v) == 0, (key, v)
        for v in (-1, 3 if key not in (1,) else 4, 7, 100, 1 << 20):
            if v not in values:
                assert qlib.baracuda_kernels_q_set_tuning(key, v) == 2, (key, v)
        assert qlib.baracuda_kernels_q_set_tuning(key, 0) == 0
    for key in (-1, 3, 7, 8, 99):
        assert qlib.baracuda_kernels_q_set_tuning(key, 0) == 2


def test_int8_symbols_refuse_k_that_could_overflow_32_bits(qlib):
    A, B, D = 0x10000, 0x20000, 0x30000
    k_ok, k_bad = 131056, 131072  # multiples of 16 either side of the 131 071 bound
    s8 = getattr(qlib, W8A8 + "_can_implement")
    fp8 = qlib.baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement
    assert s8(128, 256, k_ok, A, k_ok, B, k_ok, None, 0, D, 256) == 0
    assert s8(128, 256, k_bad, A, k_bad, B, k_bad, None, 0, D, 256) == 3
    assert fp8(128, 256, k_bad, A, k_bad, B, k_bad, None, 0, D, 256) == 0          # f32 accumulators: no such bound
    assert qlib.baracuda_kernels_gemm_s8_rrr_sm100a_can_implement(128, 256, k_bad, A, k_bad, B, 256, None, 0, D, 256) == 3
    gemv = getattr(qlib, GEMV + "_can_implement")
    assert gemv(1, 64, k_ok, 1, 1, k_ok, k_ok, 64, 0, 0, 0) == 0
    assert gemv(1, 64, k_bad, 1, 1, k_bad, k_bad, 64, 0, 0, 0) == 3
    with pytest.raises(bq.Unsupported):
        p = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(128, 256, k_bad))
        p.can_implement(bq.QGemmArgs(a=_FakeCuda(128 * k_bad, torch.int8), b=_FakeCuda(256 * k_bad, torch.int8),
                                     d=_FakeCuda(128 * 256, torch.bfloat16), scale_a=_FakeCuda(128, torch.float32),
                                     scale_b=_FakeCuda(256, torch.float32)))


def test_smoothquant_plan_surface():
    p = bq.SmoothQuantLinearPlan.select(None, bq.SmoothQuantLinearDescriptor(128, 256, 512, act_scale=0.02))
    assert p.workspace_size() == 0 and p.sku().arch is bq.ArchSku.Sm100a and p.sku().element is bq.ElementKind.S8
    good = dict(act_q=_FakeCuda(128 * 512, torch.int8), weight_q=_FakeCuda(256 * 512, torch.int8),
                weight_scale=_FakeCuda(256, torch.float32), output=_FakeCuda(128 * 256, torch.bfloat16))
    p.can_implement(bq.SmoothQuantLinearArgs(**good))
    with pytest.raises(bq.InvalidProblem):
        p.can_implement(bq.SmoothQuantLinearArgs(**{**good, "weight_scale": _FakeCuda(256, torch.float64)}))
    with pytest.raises(bq.InvalidProblem):
        bq.SmoothQuantLinearPlan.select(None, bq.SmoothQuantLinearDescriptor(1, 1, 1, act_scale=float("nan")))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_cpp_plan_layer(qlib, tmp_path):
    """Compiles and runs the host-only checks of include/baracuda_kernels_q_plan.hpp against the library."""
    import subprocess

    exe = tmp_path / "plan_host_test"
    libdir = _lib.LIB_PATH.parent
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(ROOT / "tests" / "cpp" / "plan_host_test.cpp"),
                    "-o", str(exe), "-L", str(libdir), "-lbaracuda_kernels_q", f"-Wl,-rpath,{libdir}"], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "plan_host_test ok" in res.stdout
