"""Shared helpers of the GPU parity tests: seeded inputs in the benchmark's
distributions (quantized with the CPU oracle so both sides consume the same
bytes) and small torch<->numpy conveniences."""
import numpy as np
import torch


def dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def w8a8_case(oracle, m, n, k, seed, lda=None, ldb=None):
    """Activations N(0,1) per-token int8, weights N(0,0.02) per-channel int8 stored [N,K]."""
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    aq, sa = oracle.quantize_rows_s8(a)
    wq, sb = oracle.quantize_rows_s8(w)
    return aq, wq, sa, sb


def fp8_case(oracle, m, n, k, seed, per_tensor=False):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if per_tensor:
        aq, sa = oracle.quantize_tensor_e4m3(a)
        wq, sb = oracle.quantize_tensor_e4m3(w)
    else:
        aq, sa = oracle.quantize_rows_e4m3(a)
        wq, sb = oracle.quantize_rows_e4m3(w)
    return aq, wq, sa, sb


def pad_rows(x: np.ndarray, ld: int, fill=0) -> np.ndarray:
    """Row-major [R,C] -> flat buffer with row pitch ld (padding filled)."""
    r, c = x.shape
    out = np.full((r, ld), fill, dtype=x.dtype)
    out[:, :c] = x
    return out
