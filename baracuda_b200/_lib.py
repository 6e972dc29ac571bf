"""ctypes binding of the flat C ABI (include/baracuda_kernels_q.h).

The library is the product: if it is missing this module raises — there is no
Python, torch or CPU fallback for any of the kernels.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libbaracuda_kernels_q.so"

_i32, _i64, _f32, _vp, _sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

_GEMM_PREFIX = [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64]
_GEMM_CAN = (_i32, _GEMM_PREFIX)
_GEMM_WS = (_sz, [_i32, _i32, _i32])
_TAIL = [_vp, _sz, _vp]  # workspace, workspace_bytes, stream

_GEMV_HEAD = [_i32, _i32, _i32, _i32, _i32, _f32, _f32, _vp, _i64, _i64, _vp, _i64, _i64]
_GEMV_CAN = (_i32, [_i32] * 5 + [_i64] * 6)
_GEMV_WS = (_sz, [_i32] * 5)

# symbol -> (restype, argtypes); every symbol the header declares is listed here
SIGNATURES: dict[str, tuple] = {
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_run": (_i32, _GEMM_PREFIX + [_vp, _vp, _f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_run": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _f32, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_smoothquant_linear_w8a8_bf16_sm100a_can_implement": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64]),
    "baracuda_kernels_gemm_s8_rcr_s32_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_s8_rcr_s32_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_s8_rcr_s32_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_s8_rcr_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_s8_rcr_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_s8_rcr_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_run": (_i32, _GEMM_PREFIX + [_vp, _vp, _i32, _f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_run": (_i32, _GEMM_PREFIX + [_vp, _vp, _f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_run": (_i32, _GEMM_PREFIX + [_vp, _vp, _i32, _f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_s8_rrr_s32_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_s8_rrr_s32_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_s8_rrr_s32_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_s8_rrr_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_s8_rrr_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_s8_rrr_sm100a_can_implement": _GEMM_CAN,
    "baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_run": (_i32, _GEMM_PREFIX + [_f32, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_workspace_size": _GEMM_WS,
    "baracuda_kernels_gemm_fp8_e4m3_rrr_sm100a_can_implement": _GEMM_CAN,
    **{f"baracuda_kernels_gemm_{fam}_{lay}_sm100a_epilogue_run":
           (_i32, _GEMM_PREFIX + [_vp, _i32, _i32, _f32, _f32] + _TAIL)
       for fam in ("s8", "fp8_e4m3") for lay in ("rcr", "rrr")},
    **{f"baracuda_kernels_gemm_s8_{lay}_sm100a_bias{act}_{bk}_run": (_i32, _GEMM_PREFIX + [_vp, _f32, _f32] + _TAIL)
       for lay in ("rcr", "rrr") for act in ("", "_relu", "_gelu", "_silu") for bk in ("f32", "i32")},
    **{f"baracuda_kernels_gemm_fp8_e4m3_{lay}_sm100a_bias{act}_run": (_i32, _GEMM_PREFIX + [_vp, _f32, _f32] + _TAIL)
       for lay in ("rcr", "rrr") for act in ("", "_relu", "_gelu", "_silu")},
    **{f"baracuda_kernels_gemm_{fam}_{lay}_bf16_sm100a_epilogue_run":
           (_i32, _GEMM_PREFIX + [_vp, _vp, _i32, _vp, _i32, _f32, _f32] + _TAIL)
       for fam in ("w8a8_s8", "fp8_e4m3") for lay in ("rcr", "rrr")},
    **{f"baracuda_kernels_gemm_{fam}_{lay}_bf16_sm100a_pdl_run":
           (_i32, _GEMM_PREFIX + [_vp, _vp, _i32, _vp, _i32, _f32, _f32] + _TAIL)
       for fam in ("w8a8_s8", "fp8_e4m3") for lay in ("rcr", "rrr")},
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_run": (
        _i32, _GEMV_HEAD + [_vp, _i64, _vp, _i64, _vp, _i64, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_pdl_run": (
        _i32, _GEMV_HEAD + [_vp, _i64, _vp, _i64, _vp, _i64, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_can_implement": _GEMV_CAN,
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_workspace_size": _GEMV_WS,
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_run": (
        _i32, _GEMV_HEAD + [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp]),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_static_ws_capacity": (_sz, []),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_run": (
        _i32, [_i32, _i32, _i32, _i32, _i32, _f32, _f32, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_pdl_run": (
        _i32, [_i32, _i32, _i32, _i32, _i32, _f32, _f32, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_bf16_sm100a_quant_bf16_can_implement": (_i32, [_i32, _i32, _i32, _i64, _i64, _i64]),
    "baracuda_kernels_gemv_q8_m1_s32_sm100a_run": (_i32, _GEMV_HEAD + [_vp, _i64, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_s32_sm100a_pdl_run": (_i32, _GEMV_HEAD + [_vp, _i64, _i64] + _TAIL),
    "baracuda_kernels_gemv_q8_m1_s32_sm100a_can_implement": _GEMV_CAN,
    "baracuda_kernels_gemv_q8_m1_s32_sm100a_workspace_size": _GEMV_WS,
    "baracuda_kernels_quantize_per_token_sym_f32_s8_sm100a_run": (_i32, [_i32, _i32, _i32, _i32, _vp, _i64, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_quantize_per_token_sym_bf16_s8_sm100a_run": (_i32, [_i32, _i32, _i32, _i32, _vp, _i64, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_quantize_per_token_sym_f32_e4m3_sm100a_run": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_quantize_per_token_sym_bf16_e4m3_sm100a_run": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_nshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _f32,
               _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _f32,
               _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_nshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _f32,
               _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_nshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _f32,
               _vp, _vp, _i64] + _TAIL),
    "baracuda_kernels_q_selftest_bounded_wait": (_i32, [_i64, _vp]),
    "baracuda_kernels_gemm_q8_kshard_workspace_size": (_sz, [_i32, _i32]),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _vp, _f32] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _f32, _vp, _vp, _vp]),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run": (
        _i32, [_i32, _i32, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _vp, _f32, _vp, _vp, _vp]),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run": (
        _i32, [_i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _f32, _vp, _vp, _vp]),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run": (
        _i32, [_i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _vp, _f32, _vp, _vp, _vp]),
    "baracuda_q_peer_barrier_run": (_i32, [_vp, _i32, _i32, _i64, _vp]),
    "baracuda_q_peer_barrier_flag_bytes": (_sz, []),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_run": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _f32] + _TAIL),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_workspace_size": (_sz, [_i32, _i32, _i32]),
    "baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_swiglu_can_implement": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64]),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_run": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i32, _vp, _f32] + _TAIL),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_workspace_size": (_sz, [_i32, _i32, _i32]),
    "baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_swiglu_can_implement": (
        _i32, [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64]),
    "baracuda_kernels_q_interleave_gate_up_run": (_i32, [_i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "baracuda_q_nccl_version": (_i32, []),
    "baracuda_q_nccl_unique_id": (_i32, [_vp]),
    "baracuda_q_nccl_comm_init_rank": (_i32, [C.POINTER(_vp), _i32, _vp, _i32]),
    "baracuda_q_nccl_comm_destroy": (_i32, [_vp]),
    "baracuda_q_nccl_stream_barrier": (_i32, [_vp, _vp, _vp]),
    "baracuda_q_nccl_all_gather_bytes": (_i32, [_vp, _i32, _vp, _vp, _sz, _vp]),
    "baracuda_kernels_q_device_status": (_i32, []),
    "baracuda_kernels_q_set_tuning": (_i32, [_i32, _i32]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library and attach the prototypes; raise if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m baracuda_b200.build`. "
            "The kernels have no fallback path."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the ABI and the binding disagree
        fn.restype = res
        fn.argtypes = list(args)
    _lib = lib
    return lib
