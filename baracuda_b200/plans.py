"""Typed Plan facade over the flat C ABI — the host-side mirror of the
reference's Plan triple (`select` → `can_implement` → `workspace_size` → `run`,
plus `sku()` / `precision_guarantee()`; ARCHITECTURE.md:67-110 of the reference,
crates/baracuda-kernels/src/gemm/int_gemm.rs:48-637, fp8_gemm.rs:36-741,
gemv_dense.rs:48-412).

The plans are plain data: a validated descriptor plus the SKU fixed at
`select`.  Tensors are torch CUDA tensors used purely as device-buffer
handles (pointer, length, dtype); all compute happens in the CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from .vocab import (
    OP_FP8_SCALED_GEMM,
    OP_GEMV_Q8,
    OP_W8A8_GEMM,
    ArchSku,
    BackendKind,
    BufferTooSmall,
    ElementKind,
    EpilogueKind,
    InvalidProblem,
    KernelSku,
    LayoutSku,
    MathPrecision,
    OpCategory,
    PlanPreference,
    PrecisionGuarantee,
    Unsupported,
    WorkspaceTooSmall,
    status_to_result,
)

SCALE_PER_TENSOR = 0
SCALE_PER_ROW_COL = 1

_INT_GUARANTEE = PrecisionGuarantee(MathPrecision.Int8, ElementKind.I32, True, True)
# tcgen05 accumulates each tile in a fixed order; one CTA owns one output tile
_FP8_GUARANTEE = PrecisionGuarantee(MathPrecision.Fp8E4M3, ElementKind.F32, True, True)


def _stream_ptr(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, elems: int, name: str) -> None:
    """The typed layer is the soundness boundary for buffer lengths
    (gemv_dense.rs:218-268): refuse a launch that would run off a buffer."""
    if t.numel() < elems:
        raise BufferTooSmall(f"{name}: need {elems} elements, buffer holds {t.numel()}")


def _check_backend(pref: PlanPreference) -> None:
    if pref.prefer_backend not in (None, BackendKind.Bespoke):
        raise Unsupported("these plans are bespoke-only")


def _need_typed(t: Optional[torch.Tensor], dtype, elems: int, name: str) -> None:
    """A device vector or matrix of exactly `dtype` with at least `elems` elements: the kernels read typed storage, so a
    buffer of another element size would be read past its end even when its element count looks sufficient."""
    if t is None:
        raise InvalidProblem(f"{name} is required")
    dtypes = dtype if isinstance(dtype, tuple) else (dtype,)
    if t.dtype not in dtypes:
        raise InvalidProblem(f"{name}: expected {' or '.join(str(d) for d in dtypes)}, got {t.dtype}")
    if not t.is_cuda:
        raise InvalidProblem(f"{name}: expected a device buffer")
    _need(t, elems, name)


def _span(rows: int, cols: int, ld: int) -> int:
    return 0 if rows == 0 or cols == 0 else (rows - 1) * ld + cols


# --------------------------------------------------------------------------- GEMM
@dataclass(frozen=True)
class QGemmDescriptor:
    """Shape and layout of an 8-bit GEMM (IntGemmDescriptor, types.rs:187-198)."""
    m: int
    n: int
    k: int
    layout: LayoutSku = LayoutSku.Rcr
    epilogue: EpilogueKind = EpilogueKind.Identity


@dataclass
class QGemmArgs:
    """Device views for one run.  `a` is [M,K] with row pitch lda, `b` is the
    weight stored [N,K] with row pitch ldb (column-major [K,N]), `d` is [M,N]."""
    a: torch.Tensor
    b: torch.Tensor
    d: torch.Tensor
    scale_a: Optional[torch.Tensor] = None
    scale_b: Optional[torch.Tensor] = None
    lda: Optional[int] = None
    ldb: Optional[int] = None
    ldd: Optional[int] = None
    alpha: float = 1.0
    beta: float = 0.0
    c: Optional[torch.Tensor] = None
    ldc: int = 0
    bias: Optional[torch.Tensor] = None  # [N] float32 (or int32 on the s8 8-bit-out plan) when the epilogue has one


# EpilogueKind -> the `epilogue` argument of the *_epilogue_run symbols
_EPILOGUE_CODE = {EpilogueKind.Identity: 0, EpilogueKind.Bias: 1, EpilogueKind.BiasRelu: 2, EpilogueKind.BiasGelu: 3,
                  EpilogueKind.BiasSilu: 4}


class _QGemmPlanBase:
    _run_symbol = ""
    _can_symbol = ""
    _ws_symbol = ""
    _in_dtypes: tuple = ()
    _out_dtype = torch.bfloat16
    _needs_scales = True
    _bias_dtypes: tuple = (torch.float32,)

    def __init__(self, desc: QGemmDescriptor, sku: KernelSku):
        self.desc = desc
        self._sku = sku

    @classmethod
    def _validate_desc(cls, desc: QGemmDescriptor, pref: PlanPreference) -> None:
        _check_backend(pref)
        if desc.m < 0 or desc.n < 0 or desc.k < 0:
            raise InvalidProblem("negative dimension")
        if max(desc.m, desc.n, desc.k) >= 2**31:
            raise InvalidProblem("dimension exceeds int32")
        if desc.epilogue not in _EPILOGUE_CODE:
            raise InvalidProblem("unknown epilogue")

    def sku(self) -> KernelSku:
        return self._sku

    def precision_guarantee(self) -> PrecisionGuarantee:
        return self._sku.precision_guarantee

    def workspace_size(self) -> int:
        lib = _lib.load()
        return int(getattr(lib, self._ws_symbol)(self.desc.m, self.desc.n, self.desc.k))

    def _lds(self, args: QGemmArgs):
        d = self.desc
        lda = args.lda if args.lda is not None else max(d.k, 1)
        ldb = args.ldb if args.ldb is not None else max(d.k if d.layout is LayoutSku.Rcr else d.n, 1)
        ldd = args.ldd if args.ldd is not None else max(d.n, 1)
        return lda, ldb, ldd

    def can_implement(self, args: QGemmArgs) -> None:
        d = self.desc
        lda, ldb, ldd = self._lds(args)
        for t, name in ((args.a, "a"), (args.b, "b")):
            if t.dtype not in self._in_dtypes:
                raise InvalidProblem(f"{name}: dtype {t.dtype} not accepted by this plan")
        if args.d.dtype != self._out_dtype:
            raise InvalidProblem(f"d: expected {self._out_dtype}")
        if not (args.a.is_cuda and args.b.is_cuda and args.d.is_cuda):
            raise InvalidProblem("operands must be device buffers")
        lib = _lib.load()
        ldc = args.ldc or max(d.n, 1)
        st = getattr(lib, self._can_symbol)(d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb,
                                            _ptr(args.c), ldc, _ptr(args.d), ldd)
        status_to_result(st, type(self).__name__)
        if d.m == 0 or d.n == 0:
            return  # empty problem: nothing is read or written
        if args.c is not None:
            if args.c.dtype != args.d.dtype or not args.c.is_cuda:
                raise InvalidProblem("c: expected a device buffer of the output type")
            _need(args.c, _span(d.m, d.n, ldc), "c")
        _need(args.a, _span(d.m, d.k, lda), "a")
        _need(args.b, _span(d.n, d.k, ldb) if d.layout is LayoutSku.Rcr else _span(d.k, d.n, ldb), "b")
        _need(args.d, _span(d.m, d.n, ldd), "d")
        if self._needs_scales:
            self._check_scales(args)
        if d.epilogue.requires_bias():
            if args.bias is None:
                raise InvalidProblem(f"epilogue {d.epilogue.value} needs a bias vector")
            if args.bias.dtype not in self._bias_dtypes or not args.bias.is_cuda:
                raise InvalidProblem(f"bias: expected a device vector of {self._bias_dtypes}")
            _need(args.bias, d.n, "bias")

    def _bias_kind(self, args: QGemmArgs) -> int:
        return 2 if args.bias is not None and args.bias.dtype == torch.int32 else 1

    def _check_scales(self, args: QGemmArgs) -> None:
        raise NotImplementedError

    def _call(self, lib, args: QGemmArgs, lda: int, ldb: int, ldd: int, ws_ptr, ws_bytes, stream) -> int:
        raise NotImplementedError

    def run(self, stream, workspace: Optional[torch.Tensor], args: QGemmArgs, dependent_launch: bool = False) -> None:
        """`dependent_launch=True` (bf16-out plans only) selects the *_pdl_run symbol: the kernel may start while the
        previous kernel of the stream finishes and prefetches weight tiles meanwhile; pass it only when that previous
        kernel does not write `b`."""
        self.can_implement(args)
        need = self.workspace_size()
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        if need > ws_bytes:
            raise WorkspaceTooSmall(need, ws_bytes)
        lib = _lib.load()
        lda, ldb, ldd = self._lds(args)
        if dependent_launch:
            st = self._call_dependent(lib, args, lda, ldb, ldd, _ptr(workspace), ws_bytes, _stream_ptr(stream))
        else:
            st = self._call(lib, args, lda, ldb, ldd, _ptr(workspace), ws_bytes, _stream_ptr(stream))
        status_to_result(st, type(self).__name__)

    def _call_dependent(self, lib, args: QGemmArgs, lda: int, ldb: int, ldd: int, ws_ptr, ws_bytes, stream) -> int:
        raise Unsupported(f"{type(self).__name__} has no dependent-launch form")


class W8A8GemmPlan(_QGemmPlanBase):
    """s8 x s8 -> s32 on tcgen05 with the fused per-token x per-channel dequant
    to bf16 (or, with `raw_accumulators`, the int32 sums themselves)."""

    _in_dtypes = (torch.int8,)

    def __init__(self, desc, sku, raw: bool):
        super().__init__(desc, sku)
        self.raw = raw
        lay = desc.layout.value
        base = f"baracuda_kernels_gemm_s8_{lay}_s32_sm100a" if raw else f"baracuda_kernels_gemm_w8a8_s8_{lay}_bf16_sm100a"
        self._run_symbol, self._can_symbol, self._ws_symbol = base + "_run", base + "_can_implement", base + "_workspace_size"
        self._out_dtype = torch.int32 if raw else torch.bfloat16
        self._needs_scales = not raw

    @classmethod
    def select(cls, stream, desc: QGemmDescriptor, pref: PlanPreference = PlanPreference(),
               raw_accumulators: bool = False) -> "W8A8GemmPlan":
        cls._validate_desc(desc, pref)
        if raw_accumulators and desc.epilogue is not EpilogueKind.Identity:
            raise Unsupported("the raw-accumulator SKU has the identity epilogue only")
        sku = KernelSku(OpCategory.Gemm, OP_W8A8_GEMM, ElementKind.S8,
                        ElementKind.I32 if raw_accumulators else ElementKind.Bf16,
                        desc.layout, desc.epilogue, ArchSku.Sm100a, BackendKind.Bespoke, _INT_GUARANTEE)
        return cls(desc, sku, raw_accumulators)

    def _check_scales(self, args):
        if args.scale_a is None or args.scale_b is None:
            raise InvalidProblem("scale_a and scale_b are required")
        for t, n, name in ((args.scale_a, self.desc.m, "scale_a"), (args.scale_b, self.desc.n, "scale_b")):
            if t.dtype != torch.float32:
                raise InvalidProblem(f"{name}: expected float32")
            _need(t, n, name)

    def _call(self, lib, args, lda, ldb, ldd, ws_ptr, ws_bytes, stream):
        d = self.desc
        if self.raw:
            return getattr(lib, self._run_symbol)(
                d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
                args.alpha, args.beta, ws_ptr, ws_bytes, stream)
        if d.epilogue is not EpilogueKind.Identity:
            return getattr(lib, self._run_symbol.replace("_run", "_epilogue_run"))(
                d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
                _ptr(args.scale_a), _ptr(args.scale_b), SCALE_PER_ROW_COL, _ptr(args.bias), _EPILOGUE_CODE[d.epilogue],
                args.alpha, args.beta, ws_ptr, ws_bytes, stream)
        return getattr(lib, self._run_symbol)(
            d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
            _ptr(args.scale_a), _ptr(args.scale_b), args.alpha, args.beta, ws_ptr, ws_bytes, stream)


    def _call_dependent(self, lib, args, lda, ldb, ldd, ws_ptr, ws_bytes, stream):
        d = self.desc
        if self.raw:
            raise Unsupported("the raw-accumulator SKU has no dependent-launch form")
        return getattr(lib, self._run_symbol.replace("_run", "_pdl_run"))(
            d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
            _ptr(args.scale_a), _ptr(args.scale_b), SCALE_PER_ROW_COL, _ptr(args.bias), _EPILOGUE_CODE[d.epilogue],
            args.alpha, args.beta, ws_ptr, ws_bytes, stream)


class Fp8ScaledGemmPlan(_QGemmPlanBase):
    """e4m3 x e4m3 -> f32 on tcgen05 with f32 scales (per tensor, or per row and
    per column) fused into a bf16 store; `raw_accumulators` writes the f32 sums."""

    _in_dtypes = (torch.uint8, torch.float8_e4m3fn)

    def __init__(self, desc, sku, raw: bool, scale_mode: int):
        super().__init__(desc, sku)
        self.raw = raw
        self.scale_mode = scale_mode
        if raw and desc.layout is not LayoutSku.Rcr:
            raise Unsupported("raw f32 accumulators are exported for the RCR layout only")
        base = ("baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a" if raw
                else f"baracuda_kernels_gemm_fp8_e4m3_{desc.layout.value}_bf16_sm100a")
        self._run_symbol, self._can_symbol, self._ws_symbol = base + "_run", base + "_can_implement", base + "_workspace_size"
        self._out_dtype = torch.float32 if raw else torch.bfloat16
        self._needs_scales = not raw

    @classmethod
    def select(cls, stream, desc: QGemmDescriptor, pref: PlanPreference = PlanPreference(),
               scale_mode: int = SCALE_PER_TENSOR, raw_accumulators: bool = False) -> "Fp8ScaledGemmPlan":
        cls._validate_desc(desc, pref)
        if scale_mode not in (SCALE_PER_TENSOR, SCALE_PER_ROW_COL):
            raise InvalidProblem("scale_mode must be 0 (per tensor) or 1 (per row / per column)")
        if raw_accumulators and desc.epilogue is not EpilogueKind.Identity:
            raise Unsupported("the raw-accumulator SKU has the identity epilogue only")
        sku = KernelSku(OpCategory.Gemm, OP_FP8_SCALED_GEMM, ElementKind.Fp8E4M3,
                        ElementKind.F32 if raw_accumulators else ElementKind.Bf16,
                        desc.layout, desc.epilogue, ArchSku.Sm100a, BackendKind.Bespoke, _FP8_GUARANTEE)
        return cls(desc, sku, raw_accumulators, scale_mode)

    def _check_scales(self, args):
        if args.scale_a is None or args.scale_b is None:
            raise InvalidProblem("scale_a and scale_b are required")
        na = self.desc.m if self.scale_mode == SCALE_PER_ROW_COL else 1
        nb = self.desc.n if self.scale_mode == SCALE_PER_ROW_COL else 1
        for t, n, name in ((args.scale_a, na, "scale_a"), (args.scale_b, nb, "scale_b")):
            if t.dtype != torch.float32:
                raise InvalidProblem(f"{name}: expected float32")
            _need(t, n, name)

    def _call(self, lib, args, lda, ldb, ldd, ws_ptr, ws_bytes, stream):
        d = self.desc
        if self.raw:
            return lib.baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run(
                d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
                args.alpha, args.beta, ws_ptr, ws_bytes, stream)
        if d.epilogue is not EpilogueKind.Identity:
            return getattr(lib, self._run_symbol.replace("_run", "_epilogue_run"))(
                d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
                _ptr(args.scale_a), _ptr(args.scale_b), self.scale_mode, _ptr(args.bias), _EPILOGUE_CODE[d.epilogue],
                args.alpha, args.beta, ws_ptr, ws_bytes, stream)
        return getattr(lib, self._run_symbol)(
            d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
            _ptr(args.scale_a), _ptr(args.scale_b), self.scale_mode, args.alpha, args.beta, ws_ptr, ws_bytes, stream)


    def _call_dependent(self, lib, args, lda, ldb, ldd, ws_ptr, ws_bytes, stream):
        d = self.desc
        if self.raw:
            raise Unsupported("the raw-accumulator SKU has no dependent-launch form")
        return getattr(lib, self._run_symbol.replace("_run", "_pdl_run"))(
            d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1), _ptr(args.d), ldd,
            _ptr(args.scale_a), _ptr(args.scale_b), self.scale_mode, _ptr(args.bias), _EPILOGUE_CODE[d.epilogue],
            args.alpha, args.beta, ws_ptr, ws_bytes, stream)


# --------------------------------------------------------------------------- GEMV
@dataclass(frozen=True)
class GemvQ8Descriptor:
    """GemvDenseDescriptor (gemv_dense.rs:48-75) for int8 weights; m may be 1..8."""
    m: int
    n: int
    k: int
    batch: int = 1
    layout: LayoutSku = LayoutSku.Rrr


@dataclass
class GemvQ8Args:
    """GemvDenseArgs (gemv_dense.rs:77-110) plus the two scale vectors."""
    a: torch.Tensor
    b: torch.Tensor
    d: torch.Tensor
    scale_a: Optional[torch.Tensor] = None
    scale_b: Optional[torch.Tensor] = None
    lda: Optional[int] = None
    ldb: Optional[int] = None
    ldd: Optional[int] = None
    stride_a: int = 0
    stride_b: int = 0
    stride_d: int = 0
    stride_scale_a: int = 0
    stride_scale_b: int = 0
    alpha: float = 1.0
    beta: float = 0.0


class GemvQ8Plan:
    """Decode GEMV with int8 weights, bf16 out (or the int32 sums)."""

    def __init__(self, desc: GemvQ8Descriptor, sku: KernelSku, raw: bool):
        self.desc, self._sku, self.raw = desc, sku, raw
        self._base = "baracuda_kernels_gemv_q8_m1_s32_sm100a" if raw else "baracuda_kernels_gemv_q8_m1_bf16_sm100a"

    @classmethod
    def select(cls, stream, desc: GemvQ8Descriptor, pref: PlanPreference = PlanPreference(),
               raw_accumulators: bool = False) -> "GemvQ8Plan":
        _check_backend(pref)
        if min(desc.m, desc.n, desc.k, desc.batch) < 0:
            raise InvalidProblem("negative dimension")
        if desc.m > 8:
            raise InvalidProblem("the GEMV family serves m <= 8; larger m belongs on the GEMM plans")
        sku = KernelSku(OpCategory.Gemm, OP_GEMV_Q8, ElementKind.S8,
                        ElementKind.I32 if raw_accumulators else ElementKind.Bf16,
                        desc.layout, None, ArchSku.Sm100a, BackendKind.Bespoke, _INT_GUARANTEE)
        plan = cls(desc, sku, raw_accumulators)
        if plan.workspace_size() > pref.max_workspace_bytes:
            raise Unsupported("workspace budget too small for this shape")
        return plan

    def sku(self) -> KernelSku:
        return self._sku

    def precision_guarantee(self) -> PrecisionGuarantee:
        return self._sku.precision_guarantee

    def _layout_code(self) -> int:
        return 0 if self.desc.layout is LayoutSku.Rrr else 1

    def workspace_size(self) -> int:
        lib = _lib.load()
        d = self.desc
        return int(getattr(lib, self._base + "_workspace_size")(d.m, d.n, d.k, d.batch, self._layout_code()))

    def _lds(self, args: GemvQ8Args):
        d = self.desc
        lda = args.lda if args.lda is not None else max(d.k, 1)
        ldb_min = d.n if d.layout is LayoutSku.Rrr else d.k
        ldb = args.ldb if args.ldb is not None else max(ldb_min, 1)
        ldd = args.ldd if args.ldd is not None else max(d.n, 1)
        return lda, ldb, ldd

    def can_implement(self, args: GemvQ8Args) -> None:
        d = self.desc
        lda, ldb, ldd = self._lds(args)
        if args.a.dtype != torch.int8 or args.b.dtype != torch.int8:
            raise InvalidProblem("a and b must be int8")
        if args.d.dtype != (torch.int32 if self.raw else torch.bfloat16):
            raise InvalidProblem("d has the wrong dtype for this plan")
        if not (args.a.is_cuda and args.b.is_cuda and args.d.is_cuda):
            raise InvalidProblem("operands must be device buffers")
        lib = _lib.load()
        st = getattr(lib, self._base + "_can_implement")(d.m, d.n, d.k, d.batch, self._layout_code(), lda, ldb, ldd,
                                                         args.stride_a, args.stride_b, args.stride_d)
        status_to_result(st, "GemvQ8Plan")
        if min(args.stride_a, args.stride_b, args.stride_d) < 0:
            raise InvalidProblem("negative batch stride")
        last = max(d.batch - 1, 0)
        b_rows, b_cols = (d.k, d.n) if d.layout is LayoutSku.Rrr else (d.n, d.k)
        if d.batch > 0 and d.m > 0 and d.n > 0:
            _need(args.a, last * args.stride_a + _span(d.m, d.k, lda), "a")
            _need(args.b, last * args.stride_b + _span(b_rows, b_cols, ldb), "b")
            _need(args.d, last * args.stride_d + _span(d.m, d.n, ldd), "d")
            if not self.raw:
                if min(args.stride_scale_a, args.stride_scale_b) < 0:
                    raise InvalidProblem("negative scale stride")
                # the kernels read float[...]: a bf16 or f16 scale vector of the right length would be overrun
                _need_typed(args.scale_a, torch.float32, last * args.stride_scale_a + d.m, "scale_a")
                _need_typed(args.scale_b, torch.float32, last * args.stride_scale_b + d.n, "scale_b")

    def run(self, stream, workspace: Optional[torch.Tensor], args: GemvQ8Args, dependent_launch: bool = False) -> None:
        """`dependent_launch=True` selects the *_pdl_run symbol: the kernel may start while the previous kernel of the
        stream drains and prefetches weights meanwhile; pass it only when that previous kernel does not write `b`."""
        self.can_implement(args)
        need = self.workspace_size()
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        if need > ws_bytes:
            raise WorkspaceTooSmall(need, ws_bytes)
        lib = _lib.load()
        d = self.desc
        lda, ldb, ldd = self._lds(args)
        s = _stream_ptr(stream)
        suffix = "_pdl_run" if dependent_launch else "_run"
        if self.raw:
            st = getattr(lib, "baracuda_kernels_gemv_q8_m1_s32_sm100a" + suffix)(
                d.m, d.n, d.k, d.batch, self._layout_code(), args.alpha, args.beta,
                _ptr(args.a), lda, args.stride_a, _ptr(args.b), ldb, args.stride_b,
                _ptr(args.d), ldd, args.stride_d, _ptr(workspace), ws_bytes, s)
        else:
            st = getattr(lib, "baracuda_kernels_gemv_q8_m1_bf16_sm100a" + suffix)(
                d.m, d.n, d.k, d.batch, self._layout_code(), args.alpha, args.beta,
                _ptr(args.a), lda, args.stride_a, _ptr(args.b), ldb, args.stride_b,
                _ptr(args.scale_a), args.stride_scale_a, _ptr(args.scale_b), args.stride_scale_b,
                _ptr(args.d), ldd, args.stride_d, _ptr(workspace), ws_bytes, s)
        status_to_result(st, "GemvQ8Plan")


def device_status() -> int:
    """Read-and-clear the word a kernel sets when a bounded wait ran out (0 = none)."""
    return int(_lib.load().baracuda_kernels_q_device_status())


def set_tuning(key: int, value: int) -> None:
    """Test hook: forces a kernel choice for the calling thread (see the header); 0 restores the automatic choice."""
    status_to_result(_lib.load().baracuda_kernels_q_set_tuning(key, value), "set_tuning")


# --------------------------------------------------------------------------- activation quantizer
@dataclass(frozen=True)
class QuantizePerTokenDescriptor:
    """Per-token symmetric quantizer (DynamicRangeQuantizeDescriptor of the reference's quantize family,
    crates/baracuda-kernels/src/quantize/dynamic_range.rs): `out` is "s8" or "e4m3"."""
    rows: int
    cols: int
    out: str = "s8"
    q_min: int = -127
    q_max: int = 127


class QuantizePerTokenPlan:
    """scale[r] = absmax/qmax (1.0 for a zero row); q = clamp(rint(x * (1/scale))) — f32 or bf16 in, f32 scales out."""

    def __init__(self, desc: QuantizePerTokenDescriptor):
        self.desc = desc

    @classmethod
    def select(cls, stream, desc: QuantizePerTokenDescriptor, pref: PlanPreference = PlanPreference()):
        _check_backend(pref)
        if desc.rows < 0 or desc.cols < 0:
            raise InvalidProblem("negative dimension")
        if desc.out not in ("s8", "e4m3"):
            raise InvalidProblem("out must be 's8' or 'e4m3'")
        if desc.out == "s8" and (desc.q_min > desc.q_max or desc.q_max <= 0):
            raise InvalidProblem("bad quantization range")
        return cls(desc)

    def workspace_size(self) -> int:
        return 0

    def run(self, stream, x: torch.Tensor, scale: torch.Tensor, q: torch.Tensor,
            ld_in: Optional[int] = None, ld_out: Optional[int] = None) -> None:
        d = self.desc
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise InvalidProblem("input must be float32 or bfloat16")
        if scale.dtype != torch.float32:
            raise InvalidProblem("scale must be float32")
        ld_in = ld_in if ld_in is not None else max(d.cols, 1)
        ld_out = ld_out if ld_out is not None else max(d.cols, 1)
        _need(x, _span(d.rows, d.cols, ld_in), "input")
        _need(q, _span(d.rows, d.cols, ld_out), "output")
        _need(scale, d.rows, "scale")
        lib = _lib.load()
        tin = "f32" if x.dtype == torch.float32 else "bf16"
        fn = getattr(lib, f"baracuda_kernels_quantize_per_token_sym_{tin}_{d.out}_sm100a_run")
        if d.out == "s8":
            st = fn(d.rows, d.cols, d.q_min, d.q_max, _ptr(x), ld_in, _ptr(scale), _ptr(q), ld_out, None, 0,
                    _stream_ptr(stream))
        else:
            st = fn(d.rows, d.cols, _ptr(x), ld_in, _ptr(scale), _ptr(q), ld_out, None, 0, _stream_ptr(stream))
        status_to_result(st, "QuantizePerTokenPlan")


# --------------------------------------------------------------------------- W8A8 linear (quantize + GEMM)
@dataclass(frozen=True)
class QuantizedLinearDescriptor:
    """QuantizedLinearDescriptor (crates/baracuda-kernels/src/quantize/quantized_linear.rs:55-80)."""
    m: int
    c_out: int
    k: int
    q_min: int = -127
    q_max: int = 127


@dataclass
class QuantizedLinearArgs:
    """QuantizedLinearArgs (quantized_linear.rs:82-120): f32/bf16 activation, offline-quantized int8 weight
    [C_out, K] with per-channel f32 scales, bf16 output, caller-owned scratch for the quantized activation."""
    activation: torch.Tensor
    weight_q: torch.Tensor
    weight_scale: torch.Tensor
    output: torch.Tensor
    act_q_scratch: torch.Tensor
    act_scale_scratch: torch.Tensor


class QuantizedLinearPlan:
    """The reference's two-launch W8A8 linear (quantized_linear.rs:262-355) on the sm_100a kernels:
    per-token quantize, then the tcgen05 GEMM (m > 8) or the streaming GEMV (m <= 8), bf16 out."""

    def __init__(self, desc: QuantizedLinearDescriptor, quant: QuantizePerTokenPlan, mm):
        self.desc, self._quant, self._mm = desc, quant, mm

    @classmethod
    def select(cls, stream, desc: QuantizedLinearDescriptor, pref: PlanPreference = PlanPreference()):
        quant = QuantizePerTokenPlan.select(stream, QuantizePerTokenDescriptor(desc.m, desc.k, "s8", desc.q_min, desc.q_max), pref)
        if 0 < desc.m <= 8:
            mm = GemvQ8Plan.select(stream, GemvQ8Descriptor(desc.m, desc.c_out, desc.k, layout=LayoutSku.Rcr), pref)
        else:
            mm = W8A8GemmPlan.select(stream, QGemmDescriptor(desc.m, desc.c_out, desc.k), pref)
        return cls(desc, quant, mm)

    def sku(self) -> KernelSku:
        return self._mm.sku()

    def precision_guarantee(self) -> PrecisionGuarantee:
        return self._mm.precision_guarantee()

    def workspace_size(self) -> int:
        return self._mm.workspace_size()

    def fused_decode_ok(self, args: QuantizedLinearArgs) -> bool:
        """True when the whole step runs as one launch: bf16 activation, m <= 8, and a K the fused-quantiser GEMV serves."""
        d = self.desc
        if not isinstance(self._mm, GemvQ8Plan) or args.activation.dtype != torch.bfloat16:
            return False
        st = _lib.load().baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement(d.m, d.c_out, d.k, max(d.k, 1),
                                                                                          max(d.k, 1), max(d.c_out, 1))
        return st == 0 and args.activation.data_ptr() % 16 == 0 and args.weight_q.data_ptr() % 16 == 0

    def run(self, stream, workspace: Optional[torch.Tensor], args: QuantizedLinearArgs,
            dependent_launch: bool = False) -> None:
        """`dependent_launch` as in GemvQ8Plan.run / the GEMM plans' run: the matrix kernel prefetches weights while the
        kernel before it on the stream (here: the quantiser, which never writes weights) finishes."""
        if args.act_q_scratch.dtype != torch.int8:
            raise InvalidProblem("act_q_scratch must be int8")
        d = self.desc
        if self.fused_decode_ok(args):
            # decode: quantiser and GEMV in one kernel; the scales still land in act_scale_scratch
            _need_typed(args.activation, torch.bfloat16, _span(d.m, d.k, d.k), "activation")
            _need_typed(args.weight_q, torch.int8, _span(d.c_out, d.k, d.k), "weight_q")
            _need_typed(args.weight_scale, torch.float32, d.c_out, "weight_scale")
            _need_typed(args.act_scale_scratch, torch.float32, d.m, "act_scale_scratch")
            _need_typed(args.output, torch.bfloat16, _span(d.m, d.c_out, d.c_out), "output")
            sym = "baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16" + ("_pdl_run" if dependent_launch else "_run")
            st = getattr(_lib.load(), sym)(
                d.m, d.c_out, d.k, d.q_min, d.q_max, 1.0, 0.0, _ptr(args.activation), d.k, _ptr(args.weight_q), d.k,
                _ptr(args.weight_scale), _ptr(args.act_scale_scratch), _ptr(args.output), d.c_out, None, 0,
                _stream_ptr(stream))
            status_to_result(st, "QuantizedLinearPlan")
            return
        self._quant.run(stream, args.activation, args.act_scale_scratch, args.act_q_scratch)
        if isinstance(self._mm, GemvQ8Plan):
            # the quantiser launched just before writes activations and scales, never the weights
            self._mm.run(stream, workspace, GemvQ8Args(a=args.act_q_scratch, b=args.weight_q, d=args.output,
                                                       scale_a=args.act_scale_scratch, scale_b=args.weight_scale),
                         dependent_launch=dependent_launch)
        else:
            self._mm.run(stream, workspace, QGemmArgs(a=args.act_q_scratch, b=args.weight_q, d=args.output,
                                                      scale_a=args.act_scale_scratch, scale_b=args.weight_scale),
                         dependent_launch=dependent_launch)


# --------------------------------------------------------------------------- SmoothQuant linear (per-tensor activation scale)
OP_SMOOTHQUANT_LINEAR = "smoothquant_linear_w8a8"


@dataclass(frozen=True)
class SmoothQuantLinearDescriptor:
    """SmoothQuantLinearDescriptor (crates/baracuda-kernels/src/quantize/smoothquant.rs:70-118): the per-tensor
    activation scale is frozen model metadata and lives in the descriptor."""
    m: int
    n: int
    k: int
    act_scale: float


@dataclass
class SmoothQuantLinearArgs:
    """SmoothQuantLinearArgs (smoothquant.rs:120-150): pre-quantized int8 activation [M, K], smoothed-then-quantized
    int8 weight [N, K], per-output-channel f32 weight scales, bf16 output.  `act_scale_scratch` is kept for source
    compatibility with the reference and is not touched: the scale travels by value."""
    act_q: torch.Tensor
    weight_q: torch.Tensor
    weight_scale: torch.Tensor
    output: torch.Tensor
    act_scale_scratch: Optional[torch.Tensor] = None


class SmoothQuantLinearPlan:
    """y[m, n] = bf16((act_scale * weight_scale[n]) * sum_k a_q[m, k] * w_q[n, k]) on the tcgen05 GEMM
    (SmoothQuantLinearPlan, smoothquant.rs:152-330, whose two launches -- fill + W8A8 kernel -- become one)."""

    _base = "baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a"

    def __init__(self, desc: SmoothQuantLinearDescriptor, sku: KernelSku):
        self.desc, self._sku = desc, sku

    @classmethod
    def select(cls, stream, desc: SmoothQuantLinearDescriptor, pref: PlanPreference = PlanPreference()):
        _check_backend(pref)
        if desc.m < 0 or desc.n < 0 or desc.k < 0:
            raise InvalidProblem("negative dimension")
        if max(desc.m, desc.n, desc.k) >= 2**31:
            raise InvalidProblem("dimension exceeds int32")
        if not (desc.act_scale == desc.act_scale) or desc.act_scale in (float("inf"), float("-inf")):
            raise InvalidProblem("act_scale must be finite")
        sku = KernelSku(OpCategory.Gemm, OP_SMOOTHQUANT_LINEAR, ElementKind.S8, ElementKind.Bf16, LayoutSku.Rcr,
                        EpilogueKind.Identity, ArchSku.Sm100a, BackendKind.Bespoke, _INT_GUARANTEE)
        return cls(desc, sku)

    def sku(self) -> KernelSku:
        return self._sku

    def precision_guarantee(self) -> PrecisionGuarantee:
        return self._sku.precision_guarantee

    def workspace_size(self) -> int:
        return 0

    def can_implement(self, args: SmoothQuantLinearArgs) -> None:
        d = self.desc
        st = getattr(_lib.load(), self._base + "_can_implement")(d.m, d.n, d.k, _ptr(args.act_q), max(d.k, 1),
                                                                 _ptr(args.weight_q), max(d.k, 1), _ptr(args.output),
                                                                 max(d.n, 1))
        status_to_result(st, "SmoothQuantLinearPlan")
        if d.m == 0 or d.n == 0:
            return
        _need_typed(args.act_q, torch.int8, _span(d.m, d.k, d.k), "act_q")
        _need_typed(args.weight_q, torch.int8, _span(d.n, d.k, d.k), "weight_q")
        _need_typed(args.weight_scale, torch.float32, d.n, "weight_scale")
        _need_typed(args.output, torch.bfloat16, _span(d.m, d.n, d.n), "output")

    def run(self, stream, workspace: Optional[torch.Tensor], args: SmoothQuantLinearArgs) -> None:
        self.can_implement(args)
        d = self.desc
        st = getattr(_lib.load(), self._base + "_run")(
            d.m, d.n, d.k, _ptr(args.act_q), max(d.k, 1), _ptr(args.weight_q), max(d.k, 1), float(d.act_scale),
            _ptr(args.weight_scale), _ptr(args.output), max(d.n, 1), None, 0, _stream_ptr(stream))
        status_to_result(st, "SmoothQuantLinearPlan")


# --------------------------------------------------------------------------- gated-MLP up-projection
OP_GATED_MLP_UP = "gemm_gate_up_swiglu"


@dataclass(frozen=True)
class GatedMlpUpDescriptor:
    """One launch for the first half of a gated MLP: h[M, F] = silu(x Wg^T) * (x Wu^T) from 8-bit operands.
    `element` is ElementKind.S8 (per-token x per-channel scales) or ElementKind.Fp8E4M3 (scales per `scale_mode`)."""
    m: int
    f: int
    k: int
    element: ElementKind = ElementKind.S8
    scale_mode: int = SCALE_PER_ROW_COL


@dataclass
class GatedMlpUpArgs:
    """`b_gate_up` is the interleaved [2F, K] weight, `scale_b` (and `bias`) the interleaved [2F] vectors built by
    GatedMlpUpPlan.interleave; `d` is bf16 [M, F]."""
    a: torch.Tensor
    b_gate_up: torch.Tensor
    d: torch.Tensor
    scale_a: torch.Tensor
    scale_b: torch.Tensor
    bias: Optional[torch.Tensor] = None
    lda: Optional[int] = None
    ldb: Optional[int] = None
    ldd: Optional[int] = None
    alpha: float = 1.0


class GatedMlpUpPlan:
    """Gate and up projections plus SiLU-and-multiply in the GEMM epilogue.  The reference's EpilogueKind
    (crates/baracuda-kernel-vocab/src/layout.rs:69-96) ends at BiasSilu, so there a gated MLP is the GEMM(s) followed
    by an elementwise pass over [M, 2F]; here that intermediate stays in tensor memory."""

    def __init__(self, desc: GatedMlpUpDescriptor, sku: KernelSku):
        self.desc = desc
        self._sku = sku
        fam = "w8a8_s8" if desc.element is ElementKind.S8 else "fp8_e4m3"
        self._base = f"baracuda_kernels_gemm_{fam}_rcr_bf16_sm100a_swiglu"

    @classmethod
    def select(cls, stream, desc: GatedMlpUpDescriptor, pref: PlanPreference = PlanPreference()) -> "GatedMlpUpPlan":
        _check_backend(pref)
        if desc.m < 0 or desc.f < 0 or desc.k < 0:
            raise InvalidProblem("negative dimension")
        if max(desc.m, 2 * desc.f, desc.k) >= 2**31:
            raise InvalidProblem("dimension exceeds int32")
        if desc.element not in (ElementKind.S8, ElementKind.Fp8E4M3):
            raise Unsupported("gated-MLP up-projection takes s8 or e4m3 operands")
        if desc.element is ElementKind.S8 and desc.scale_mode != SCALE_PER_ROW_COL:
            raise InvalidProblem("the s8 SKU takes per-token and per-channel scales")
        if desc.scale_mode not in (SCALE_PER_TENSOR, SCALE_PER_ROW_COL):
            raise InvalidProblem("scale_mode must be 0 (per tensor) or 1 (per row / per column)")
        if desc.f % 32 != 0:
            raise Unsupported("F must be a multiple of 32 (gate and up rows are interleaved in blocks of 32)")
        guarantee = _INT_GUARANTEE if desc.element is ElementKind.S8 else _FP8_GUARANTEE
        sku = KernelSku(OpCategory.Gemm, OP_GATED_MLP_UP, desc.element, ElementKind.Bf16, LayoutSku.Rcr,
                        EpilogueKind.Identity, ArchSku.Sm100a, BackendKind.Bespoke, guarantee)
        return cls(desc, sku)

    def sku(self) -> KernelSku:
        return self._sku

    def precision_guarantee(self) -> PrecisionGuarantee:
        return self._sku.precision_guarantee

    def workspace_size(self) -> int:
        return int(getattr(_lib.load(), self._base + "_workspace_size")(self.desc.m, 2 * self.desc.f, self.desc.k))

    @staticmethod
    def interleave(gate: torch.Tensor, up: torch.Tensor, stream=None) -> torch.Tensor:
        """Rows (2-D weights) or entries (1-D scale / bias vectors) of `gate` and `up` interleaved in blocks of 32."""
        if gate.shape != up.shape or gate.dtype != up.dtype or gate.dim() not in (1, 2):
            raise InvalidProblem("gate and up must have the same shape and dtype (1-D or 2-D)")
        if not (gate.is_cuda and up.is_cuda):
            raise InvalidProblem("operands must be device buffers")
        gate, up = gate.contiguous(), up.contiguous()
        f_rows = gate.shape[0]
        row_bytes = gate.element_size() * (gate.shape[1] if gate.dim() == 2 else 1)
        out = torch.empty((2 * f_rows,) + tuple(gate.shape[1:]), dtype=gate.dtype, device=gate.device)
        st = _lib.load().baracuda_kernels_q_interleave_gate_up_run(
            f_rows, row_bytes, _ptr(gate), row_bytes, _ptr(up), row_bytes, _ptr(out), row_bytes, _stream_ptr(stream))
        status_to_result(st, "GatedMlpUpPlan.interleave")
        return out

    def _lds(self, args: GatedMlpUpArgs):
        d = self.desc
        return (args.lda if args.lda is not None else max(d.k, 1), args.ldb if args.ldb is not None else max(d.k, 1),
                args.ldd if args.ldd is not None else max(d.f, 1))

    def can_implement(self, args: GatedMlpUpArgs) -> None:
        d = self.desc
        lda, ldb, ldd = self._lds(args)
        ok_in = (torch.int8,) if d.element is ElementKind.S8 else (torch.uint8, torch.float8_e4m3fn)
        for t, name in ((args.a, "a"), (args.b_gate_up, "b_gate_up")):
            if t.dtype not in ok_in:
                raise InvalidProblem(f"{name}: dtype {t.dtype} not accepted by this plan")
        if args.d.dtype != torch.bfloat16:
            raise InvalidProblem("d: expected bfloat16")
        if not (args.a.is_cuda and args.b_gate_up.is_cuda and args.d.is_cuda):
            raise InvalidProblem("operands must be device buffers")
        st = getattr(_lib.load(), self._base + "_can_implement")(d.m, 2 * d.f, d.k, _ptr(args.a), lda,
                                                                 _ptr(args.b_gate_up), ldb, _ptr(args.d), ldd)
        status_to_result(st, type(self).__name__)
        if d.m == 0 or d.f == 0:
            return
        _need(args.a, _span(d.m, d.k, lda), "a")
        _need(args.b_gate_up, _span(2 * d.f, d.k, ldb), "b_gate_up")
        _need(args.d, _span(d.m, d.f, ldd), "d")
        per_vec = d.scale_mode == SCALE_PER_ROW_COL
        for t, n, name in ((args.scale_a, d.m if per_vec else 1, "scale_a"),
                           (args.scale_b, 2 * d.f if per_vec else 1, "scale_b")):
            if t is None or t.dtype != torch.float32:
                raise InvalidProblem(f"{name}: expected a float32 device vector")
            _need(t, n, name)
        if args.bias is not None:
            if args.bias.dtype != torch.float32 or not args.bias.is_cuda:
                raise InvalidProblem("bias: expected a float32 device vector")
            _need(args.bias, 2 * d.f, "bias")

    def run(self, stream, workspace: Optional[torch.Tensor], args: GatedMlpUpArgs) -> None:
        self.can_implement(args)
        d = self.desc
        lda, ldb, ldd = self._lds(args)
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        lib = _lib.load()
        head = (d.m, 2 * d.f, d.k, _ptr(args.a), lda, _ptr(args.b_gate_up), ldb, _ptr(args.d), ldd, _ptr(args.scale_a),
                _ptr(args.scale_b))
        tail = (_ptr(args.bias), args.alpha, _ptr(workspace), ws_bytes, _stream_ptr(stream))
        if d.element is ElementKind.S8:
            st = getattr(lib, self._base + "_run")(*head, *tail)
        else:
            st = getattr(lib, self._base + "_run")(*head, d.scale_mode, *tail)
        status_to_result(st, type(self).__name__)


# --------------------------------------------------------------------------- the reference's 8-bit-out plans
class IntGemmPlan(_QGemmPlanBase):
    """`IntGemmPlan<S8>` of the reference (crates/baracuda-kernels/src/gemm/int_gemm.rs:48-637), Rcr layout,
    on tcgen05: D[s8] = sat(rint(act(alpha * acc + beta * C + bias))), every EpilogueKind, f32 or i32 bias."""

    _in_dtypes = (torch.int8,)
    _out_dtype = torch.int8
    _needs_scales = False
    _bias_dtypes = (torch.float32, torch.int32)
    _base = "baracuda_kernels_gemm_s8_rcr_sm100a"
    _element = ElementKind.S8
    _guarantee = _INT_GUARANTEE
    _op = OP_W8A8_GEMM

    def __init__(self, desc, sku):
        super().__init__(desc, sku)
        base = self._base.replace("_rcr_", f"_{desc.layout.value}_")
        self._run_symbol, self._can_symbol, self._ws_symbol = base + "_run", base + "_can_implement", base + "_workspace_size"

    @classmethod
    def select(cls, stream, desc: QGemmDescriptor, pref: PlanPreference = PlanPreference()):
        cls._validate_desc(desc, pref)
        sku = KernelSku(OpCategory.Gemm, cls._op, cls._element, None, desc.layout, desc.epilogue, ArchSku.Sm100a,
                        BackendKind.Bespoke, cls._guarantee)
        return cls(desc, sku)

    def _call(self, lib, args, lda, ldb, ldd, ws_ptr, ws_bytes, stream):
        d = self.desc
        if d.epilogue is not EpilogueKind.Identity:
            return getattr(lib, self._run_symbol.replace("_run", "_epilogue_run"))(
                d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c), args.ldc or max(d.n, 1),
                _ptr(args.d), ldd, _ptr(args.bias), self._bias_kind(args), _EPILOGUE_CODE[d.epilogue], args.alpha,
                args.beta, ws_ptr, ws_bytes, stream)
        return getattr(lib, self._run_symbol)(d.m, d.n, d.k, _ptr(args.a), lda, _ptr(args.b), ldb, _ptr(args.c),
                                              args.ldc or max(d.n, 1), _ptr(args.d), ldd, args.alpha, args.beta,
                                              ws_ptr, ws_bytes, stream)


class Fp8GemmPlan(IntGemmPlan):
    """`Fp8GemmPlan<Fp8E4M3>` of the reference (crates/baracuda-kernels/src/gemm/fp8_gemm.rs:36-741), Rcr layout,
    D[e4m3] = sat(act(alpha * acc + beta * dequant(C) + bias)), every EpilogueKind, f32 bias."""

    _in_dtypes = (torch.uint8, torch.float8_e4m3fn)
    _out_dtype = torch.uint8
    _bias_dtypes = (torch.float32,)
    _base = "baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a"
    _element = ElementKind.Fp8E4M3
    _guarantee = _FP8_GUARANTEE
    _op = OP_FP8_SCALED_GEMM
