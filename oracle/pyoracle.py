"""numpy/ctypes front end of the C oracle (oracle/oracle.c) — TEST INFRASTRUCTURE.

Builds ``oracle/liboracle.so`` on first use (gcc via the Makefile beside it) and
exposes the restated reference functions over numpy arrays.  Nothing in the
product path imports this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"

F32, F64, BF16, I32, S8, I64 = 0, 1, 2, 3, 4, 5
EPI_IDENTITY, EPI_RELU, EPI_BIAS, EPI_BIAS_RELU = 0, 1, 2, 3
RRR, RCR = 0, 1

_NP_OF = {F32: np.float32, F64: np.float64, BF16: np.uint16, I32: np.int32, S8: np.int8, I64: np.int64}

_lib = None


def build(force: bool = False) -> Path:
    src_m = max((HERE / "oracle.c").stat().st_mtime, (HERE / "oracle.h").stat().st_mtime)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src_m:
        subprocess.run(["make", "-C", str(HERE), "-B"], check=True, capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB_PATH))
        vp, i32, i64, f32, f64 = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_double
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.restype = None
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_f32_to_bf16_bits.restype = C.c_uint16
        L.orc_f32_to_bf16_bits.argtypes = [f32]
        L.orc_bf16_bits_to_f32.restype = f32
        L.orc_bf16_bits_to_f32.argtypes = [C.c_uint16]
        L.orc_e4m3_to_f32.restype = f32
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3_satfinite.restype = C.c_uint8
        L.orc_f32_to_e4m3_satfinite.argtypes = [f32]
        L.orc_contraction.restype = C.c_int
        L.orc_contraction.argtypes = [C.c_int, i64, i64, i64, i64, vp, C.POINTER(i64), vp, C.POINTER(i64), vp, vp,
                                      C.POINTER(i64), C.c_int]
        L.orc_gemm_s8_s32.restype = C.c_int
        L.orc_gemm_s8_s32.argtypes = [i32, i32, i32, vp, i64, vp, i64, C.c_int, vp, i64]
        L.orc_dequant_s32_bf16.restype = None
        L.orc_dequant_s32_bf16.argtypes = [i32, i32, vp, i64, vp, vp, vp, i64]
        L.orc_dequant_s32_f32.restype = None
        L.orc_dequant_s32_f32.argtypes = [i32, i32, vp, i64, vp, vp, vp, i64]
        L.orc_gemm_e4m3_f32.restype = C.c_int
        L.orc_gemm_e4m3_f32.argtypes = [i32, i32, i32, vp, i64, vp, i64, C.c_int, vp, i64]
        L.orc_scale_f32_bf16.restype = None
        L.orc_scale_f32_bf16.argtypes = [i32, i32, vp, i64, vp, C.c_int, vp, C.c_int, vp, i64]
        L.orc_int_gemm_s8_out.restype = C.c_int
        L.orc_int_gemm_s8_out.argtypes = [i32, i32, i32, vp, i64, vp, i64, C.c_int, vp, i64, vp, f32, f32, vp, i64]
        L.orc_quantize_rows_s8.restype = None
        L.orc_quantize_rows_s8.argtypes = [i32, i32, i32, i32, vp, i64, vp, vp, i64]
        L.orc_quantize_rows_e4m3.restype = None
        L.orc_quantize_rows_e4m3.argtypes = [i32, i32, vp, i64, vp, vp, i64]
        L.orc_quantize_tensor_e4m3.restype = None
        L.orc_quantize_tensor_e4m3.argtypes = [i64, vp, vp, vp]
        L.orc_compare_bitexact.restype = i64
        L.orc_compare_bitexact.argtypes = [vp, vp, C.c_size_t, i64]
        L.orc_compare_tolerant_f32.restype = i64
        L.orc_compare_tolerant_f32.argtypes = [vp, vp, i64, f64, f64]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Thread count of the following calls; overrides an OMP_NUM_THREADS a launcher exported for its ranks."""
    lib().orc_set_num_threads(int(n))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    L = lib()
    return np.array([L.orc_f32_to_bf16_bits(float(v)) for v in x.ravel()], dtype=np.uint16).reshape(x.shape)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    L = lib()
    return np.array([L.orc_f32_to_e4m3_satfinite(float(v)) for v in x.ravel()], dtype=np.uint8).reshape(x.shape)


def contraction(dtype: int, lhs: np.ndarray, lhs_strides, rhs: np.ndarray, rhs_strides, shape, out_strides=None,
                bias=None, epilogue: int = EPI_IDENTITY) -> np.ndarray:
    """shape = (bdim, m, n, k); stride triples are (batch, row, col) in elements over the flat buffers."""
    bdim, m, n, k = shape
    npdt = _NP_OF[dtype]
    lhs = _c(lhs, npdt).ravel()
    rhs = _c(rhs, npdt).ravel()
    if out_strides is None:
        out_strides = (m * n, n, 1)
    out = np.zeros(bdim * m * n, dtype=npdt)
    arr = lambda s: (C.c_int64 * 3)(*s)
    bias_keep = None if bias is None else _c(bias, npdt)
    st = lib().orc_contraction(dtype, bdim, m, n, k, _p(lhs), arr(lhs_strides), _p(rhs), arr(rhs_strides),
                               None if bias_keep is None else _p(bias_keep), _p(out), arr(out_strides), epilogue)
    if st != 0:
        raise ValueError(f"orc_contraction status {st}")
    return out


def gemm_s8_s32(a: np.ndarray, b: np.ndarray, layout: int, m: int, n: int, k: int, lda=None, ldb=None) -> np.ndarray:
    a = _c(a, np.int8)
    b = _c(b, np.int8)
    lda = k if lda is None else lda
    ldb = (k if layout == RCR else n) if ldb is None else ldb
    out = np.zeros((m, n), dtype=np.int32)
    st = lib().orc_gemm_s8_s32(m, n, k, _p(a), lda, _p(b), ldb, layout, _p(out), n)
    if st != 0:
        raise ValueError(f"orc_gemm_s8_s32 status {st}")
    return out


def dequant_s32_bf16(acc: np.ndarray, sa: np.ndarray, sb: np.ndarray) -> np.ndarray:
    acc = _c(acc, np.int32)
    m, n = acc.shape
    sa, sb = _c(sa, np.float32), _c(sb, np.float32)
    out = np.zeros((m, n), dtype=np.uint16)
    lib().orc_dequant_s32_bf16(m, n, _p(acc), n, _p(sa), _p(sb), _p(out), n)
    return out


def dequant_s32_f32(acc: np.ndarray, sa: np.ndarray, sb: np.ndarray) -> np.ndarray:
    acc = _c(acc, np.int32)
    m, n = acc.shape
    sa, sb = _c(sa, np.float32), _c(sb, np.float32)
    out = np.zeros((m, n), dtype=np.float32)
    lib().orc_dequant_s32_f32(m, n, _p(acc), n, _p(sa), _p(sb), _p(out), n)
    return out


def gemm_e4m3_f32(a: np.ndarray, b: np.ndarray, layout: int, m: int, n: int, k: int, lda=None, ldb=None) -> np.ndarray:
    a = _c(a, np.uint8)
    b = _c(b, np.uint8)
    lda = k if lda is None else lda
    ldb = (k if layout == RCR else n) if ldb is None else ldb
    out = np.zeros((m, n), dtype=np.float32)
    st = lib().orc_gemm_e4m3_f32(m, n, k, _p(a), lda, _p(b), ldb, layout, _p(out), n)
    if st != 0:
        raise ValueError(f"orc_gemm_e4m3_f32 status {st}")
    return out


def scale_f32_bf16(acc: np.ndarray, sa: np.ndarray, sb: np.ndarray) -> np.ndarray:
    acc = _c(acc, np.float32)
    m, n = acc.shape
    sa, sb = _c(np.atleast_1d(sa), np.float32), _c(np.atleast_1d(sb), np.float32)
    out = np.zeros((m, n), dtype=np.uint16)
    # a one-element scale is a broadcast scalar (for m == 1 or n == 1 the two readings coincide)
    lib().orc_scale_f32_bf16(m, n, _p(acc), n, _p(sa), int(sa.size > 1), _p(sb), int(sb.size > 1), _p(out), n)
    return out


def int_gemm_s8_out(a, b, layout, m, n, k, alpha, beta=0.0, c=None, bias=None, lda=None, ldb=None) -> np.ndarray:
    a, b = _c(a, np.int8), _c(b, np.int8)
    lda = k if lda is None else lda
    ldb = (k if layout == RCR else n) if ldb is None else ldb
    cc = None if c is None else _c(c, np.int8)
    bb = None if bias is None else _c(bias, np.float32)
    out = np.zeros((m, n), dtype=np.int8)
    st = lib().orc_int_gemm_s8_out(m, n, k, _p(a), lda, _p(b), ldb, layout, None if cc is None else _p(cc), n,
                                   None if bb is None else _p(bb), alpha, beta, _p(out), n)
    if st != 0:
        raise ValueError(f"orc_int_gemm_s8_out status {st}")
    return out


EPILOGUE_IDENTITY, EPILOGUE_BIAS, EPILOGUE_BIAS_RELU, EPILOGUE_BIAS_GELU, EPILOGUE_BIAS_SILU = range(5)


def epilogue_chain(z: np.ndarray, bias, kind: int) -> np.ndarray:
    """z + bias[j], then the activation, as the reference's CPU loops state it
    (crates/baracuda-kernels/tests/int8_rrr_smoke.rs:31-66,108-131; fp8_bias_smoke.rs:30-64,154):
    relu = max(x, 0), gelu = 0.5*x*(1 + erf(x/sqrt 2)), silu = x/(1 + exp(-x)).
    The bias add is one f32 rounding (bit-exact for Bias / BiasRelu); gelu and silu are evaluated in f64 and
    rounded once to f32 -- the reference accepts +-1 output code (int8) / 2 grid steps (fp8) for those two."""
    z = np.asarray(z, dtype=np.float32)
    if kind == EPILOGUE_IDENTITY:
        return z
    b = np.asarray(bias)
    assert b.shape == (z.shape[1],) and b.dtype in (np.float32, np.int32)
    z = (z + b.astype(np.float32)[None, :]).astype(np.float32)
    if kind == EPILOGUE_BIAS:
        return z
    if kind == EPILOGUE_BIAS_RELU:
        return np.maximum(z, np.float32(0.0))
    z64 = z.astype(np.float64)
    if kind == EPILOGUE_BIAS_GELU:
        import math
        erf = np.vectorize(math.erf, otypes=[np.float64])
        return (0.5 * z64 * (1.0 + erf(z64 / math.sqrt(2.0)))).astype(np.float32)
    if kind == EPILOGUE_BIAS_SILU:
        return (z64 / (1.0 + np.exp(-z64))).astype(np.float32)
    raise ValueError(f"epilogue kind {kind}")


def interleave_gate_up(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """Rows (or entries) of gate and up interleaved in blocks of 32: out[64b + i] = gate[32b + i] for i < 32,
    up[32b + i - 32] otherwise -- the operand layout of the gated-MLP GEMM (no counterpart in the reference)."""
    gate, up = np.asarray(gate), np.asarray(up)
    assert gate.shape == up.shape and gate.shape[0] % 32 == 0
    f = gate.shape[0]
    g = gate.reshape((f // 32, 32) + gate.shape[1:])
    u = up.reshape((f // 32, 32) + up.shape[1:])
    return np.concatenate([g, u], axis=1).reshape((2 * f,) + gate.shape[1:])


def swiglu_f32(z_gate: np.ndarray, z_up: np.ndarray) -> np.ndarray:
    """silu(z_gate) * z_up with silu = x / (1 + exp(-x)) as the reference states it
    (crates/baracuda-kernels/tests/int8_rrr_smoke.rs:60-66), evaluated in f64 and rounded once to f32."""
    g = np.asarray(z_gate, dtype=np.float32).astype(np.float64)
    u = np.asarray(z_up, dtype=np.float32).astype(np.float64)
    with np.errstate(over="ignore"):
        return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)


def sat_s8(z: np.ndarray) -> np.ndarray:
    """Round half to even, clamp to [-128, 127] (int8_rrr_smoke.rs:76-78)."""
    return np.clip(np.rint(np.asarray(z, dtype=np.float32)), -128, 127).astype(np.int8)


def quantize_rows_s8(x: np.ndarray, qmin: int = -127, qmax: int = 127):
    x = _c(x, np.float32)
    rows, cols = x.shape
    scale = np.zeros(rows, dtype=np.float32)
    q = np.zeros((rows, cols), dtype=np.int8)
    lib().orc_quantize_rows_s8(rows, cols, qmin, qmax, _p(x), cols, _p(scale), _p(q), cols)
    return q, scale


def quantize_rows_e4m3(x: np.ndarray):
    x = _c(x, np.float32)
    rows, cols = x.shape
    scale = np.zeros(rows, dtype=np.float32)
    q = np.zeros((rows, cols), dtype=np.uint8)
    lib().orc_quantize_rows_e4m3(rows, cols, _p(x), cols, _p(scale), _p(q), cols)
    return q, scale


def quantize_tensor_e4m3(x: np.ndarray):
    x = _c(x, np.float32)
    scale = np.zeros(1, dtype=np.float32)
    q = np.zeros(x.shape, dtype=np.uint8)
    lib().orc_quantize_tensor_e4m3(x.size, _p(x), _p(scale), _p(q))
    return q, scale


def compare_bitexact(expected: np.ndarray, actual: np.ndarray) -> int:
    e = np.ascontiguousarray(expected)
    a = np.ascontiguousarray(actual)
    assert e.dtype == a.dtype and e.shape == a.shape, (e.dtype, a.dtype, e.shape, a.shape)
    return int(lib().orc_compare_bitexact(_p(e), _p(a), e.dtype.itemsize, e.size))


def compare_tolerant(expected: np.ndarray, actual: np.ndarray, rel: float, abs_tol: float) -> int:
    e, a = _c(expected, np.float32), _c(actual, np.float32)
    assert e.shape == a.shape
    return int(lib().orc_compare_tolerant_f32(_p(e), _p(a), e.size, rel, abs_tol))
