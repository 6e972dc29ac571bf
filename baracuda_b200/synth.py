"""Seeded synthetic inputs for the benchmark configurations.

The quantizers follow the reference's input recipe — symmetric absmax scale,
multiply by the reciprocal, round half to even, clamp
(crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:160-200;
crates/baracuda-kernels/tests/quantized_linear_smoke.rs:35-61) — written with
torch ops so large inputs can be prepared on the GPU.  Input preparation is not
part of the timed or parity-checked kernels: both the kernels and the CPU
checker consume the bytes produced here.
"""
from __future__ import annotations

import torch


def normal(shape, std: float, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std


def quantize_rows_s8(x: torch.Tensor, qmax: int = 127):
    """Per-row symmetric int8: returns (q int8 [R,C], scale f32 [R])."""
    amax = x.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / float(qmax), torch.ones_like(amax))
    inv = 1.0 / scale
    q = torch.round(x * inv[:, None]).clamp_(-qmax, qmax).to(torch.int8)
    return q, scale


def quantize_rows_e4m3(x: torch.Tensor):
    """Per-row e4m3: scale = absmax/448, q = e4m3(x * (1/scale)) saturating; returns uint8 bytes."""
    amax = x.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    inv = 1.0 / scale
    q = (x * inv[:, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, scale


def quantize_tensor_e4m3(x: torch.Tensor):
    """Per-tensor e4m3: one dequant scale absmax/448."""
    amax = x.abs().amax()
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax)).reshape(1)
    inv = 1.0 / scale
    q = (x * inv).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, scale
