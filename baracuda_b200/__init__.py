"""B200-native quantized-GEMM hot path behind baracuda's Plan surface.

Three hand-written sm_100a kernels (W8A8 s8 GEMM, FP8 e4m3 GEMM, int8 decode
GEMV) exported as flat C symbols (include/baracuda_kernels_q.h) and wrapped by
typed plans that mirror the reference's `select / can_implement /
workspace_size / run / sku` contract.
"""
from .vocab import (  # noqa: F401
    ArchSku,
    BackendKind,
    BaracudaError,
    BufferTooSmall,
    ElementKind,
    EpilogueKind,
    InvalidProblem,
    KernelSku,
    LaunchFailure,
    LayoutSku,
    MathPrecision,
    MisalignedOperand,
    OpCategory,
    PlanPreference,
    PrecisionGuarantee,
    Unsupported,
    WorkspaceTooSmall,
)
from .plans import (  # noqa: F401
    SCALE_PER_ROW_COL,
    SCALE_PER_TENSOR,
    Fp8GemmPlan,
    GatedMlpUpArgs,
    GatedMlpUpDescriptor,
    GatedMlpUpPlan,
    Fp8ScaledGemmPlan,
    IntGemmPlan,
    GemvQ8Args,
    GemvQ8Descriptor,
    GemvQ8Plan,
    QGemmArgs,
    QGemmDescriptor,
    QuantizedLinearArgs,
    QuantizedLinearDescriptor,
    QuantizedLinearPlan,
    QuantizePerTokenDescriptor,
    QuantizePerTokenPlan,
    SmoothQuantLinearArgs,
    SmoothQuantLinearDescriptor,
    SmoothQuantLinearPlan,
    W8A8GemmPlan,
    device_status,
    set_tuning,
)
