"""Plan-surface vocabulary, mirroring the reference's shared enums and structs
(crates/baracuda-kernel-vocab/src/layout.rs:17-96, sku.rs:123-285, plan.rs:19-86,
crates/baracuda-cutlass/src/error.rs:23-93).  Pure data: hashable, comparable,
usable as autotuner cache keys exactly like the reference's `Copy + Eq + Hash`
types."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Optional


class LayoutSku(enum.Enum):
    """Operand storage order (layout.rs:17-34)."""
    Rcr = "rcr"  # A row-major, B column-major, D row-major
    Rrr = "rrr"  # all row-major


class ArchSku(enum.Enum):
    """Compute capability a kernel was compiled for (layout.rs:43-53); Sm100a is new."""
    Sm80 = "sm80"
    Sm89 = "sm89"
    Sm90a = "sm90a"
    Sm100a = "sm100a"


class EpilogueKind(enum.Enum):
    """Fused epilogue chain (layout.rs:69-96)."""
    Identity = "identity"
    Bias = "bias"
    BiasRelu = "bias_relu"
    BiasGelu = "bias_gelu"
    BiasSilu = "bias_silu"

    def requires_bias(self) -> bool:
        return self is not EpilogueKind.Identity


class BackendKind(enum.Enum):
    """Which compute path serves a SKU (sku.rs:123-204); only Bespoke exists here."""
    Bespoke = "bespoke"
    Cutlass = "cutlass"
    Cublas = "cublas"


class OpCategory(enum.Enum):
    Gemm = "gemm"
    Quantization = "quantization"


class ElementKind(enum.Enum):
    """Subset of element.rs:1014 used on this path."""
    S8 = "s8"
    Fp8E4M3 = "fp8_e4m3"
    Bf16 = "bf16"
    F32 = "f32"
    I32 = "i32"


class MathPrecision(enum.Enum):
    """element.rs:1124-1160."""
    Int8 = "int8"
    Fp8E4M3 = "fp8_e4m3"


@dataclass(frozen=True)
class PrecisionGuarantee:
    """plan.rs:68-86."""
    math_precision: MathPrecision
    accumulator: ElementKind
    bit_stable_on_same_hardware: bool
    deterministic: bool


@dataclass(frozen=True)
class PlanPreference:
    """plan.rs:19-57 (allow_sm90a kept for signature parity; it selects nothing here)."""
    max_workspace_bytes: int = 2**63 - 1
    allow_sm90a: bool = True
    prefer_backend: Optional[BackendKind] = None


@dataclass(frozen=True)
class KernelSku:
    """sku.rs:259-285 — the telemetry / cache-key identity `Plan.sku()` returns."""
    category: OpCategory
    op: int
    element: ElementKind
    aux_element: Optional[ElementKind]
    layout: Optional[LayoutSku]
    epilogue: Optional[EpilogueKind]
    arch: ArchSku
    backend: BackendKind
    precision_guarantee: PrecisionGuarantee


# category-local op discriminants of the new SKUs
OP_W8A8_GEMM = 100
OP_FP8_SCALED_GEMM = 101
OP_GEMV_Q8 = 102


class BaracudaError(Exception):
    """Typed error of the Plan layer (crates/baracuda-cutlass/src/error.rs:23-70)."""


class Unsupported(BaracudaError):
    pass


class InvalidProblem(BaracudaError):
    pass


class MisalignedOperand(BaracudaError):
    pass


class WorkspaceTooSmall(BaracudaError):
    def __init__(self, needed: int, got: int):
        super().__init__(f"workspace too small: need {needed} bytes, got {got}")
        self.needed, self.got = needed, got


class BufferTooSmall(BaracudaError):
    pass


class LaunchFailure(BaracudaError):
    pass


def status_to_result(status: int, what: str) -> None:
    """Map a C status to the typed error (error.rs:83-93, int_gemm.rs:640-653)."""
    if status == 0:
        return
    if status == 1:
        raise MisalignedOperand(f"{what}: misaligned operand")
    if status == 2:
        raise InvalidProblem(f"{what}: invalid problem")
    if status == 3:
        raise Unsupported(f"{what}: unsupported")
    if status == 4:
        raise WorkspaceTooSmall(0, 0)
    if status == 5:
        raise LaunchFailure(f"{what}: kernel launch failed")
    raise BaracudaError(f"{what}: unknown status {status}")
