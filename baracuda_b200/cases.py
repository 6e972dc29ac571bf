"""Runs one kernel of the library a few times on seeded random operands.

    python -m baracuda_b200.cases gemv --layout rcr --m 1 --n 14336 --k 4096 --iters 3
    python -m baracuda_b200.cases gemm --kind fp8 --m 8192 --n 8192 --k 4096 --iters 3
    python -m baracuda_b200.cases quantize --m 8192 --k 4096 --in bf16 --kind s8 --iters 3

Meant as the small, self-terminating command to put under a profiler (one
kernel, a handful of launches, a few hundred MB on the device) and as a usage
example of the Plan API.  Prints the mean device time per launch.
"""
from __future__ import annotations

import argparse

import torch

import baracuda_b200 as bq


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemv", "gemm", "quantize"])
    ap.add_argument("--layout", default="rcr", choices=["rcr", "rrr"])
    ap.add_argument("--kind", default="s8", choices=["s8", "fp8"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--buffers", type=int, default=3, help="distinct weight buffers rotated through (defeats L2 reuse)")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--in", dest="in_dtype", default="bf16", choices=["bf16", "f32"],
                    help="quantize only: the activation type ([m, k] in, --kind s8 or fp8 codes out)")
    ap.add_argument("--epilogue", default="identity", choices=["identity", "bias_gelu", "gated"],
                    help="gemm --kind s8 only: fused bias + gelu, or the gated-MLP epilogue (n counts gate and up rows)")
    a = ap.parse_args()

    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    m, n, k = a.m, a.n, a.k
    sa = torch.rand(m, device="cuda", generator=g)
    sb = torch.rand(n, device="cuda", generator=g)
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ws = None
    if a.kernel == "quantize":
        dt = torch.bfloat16 if a.in_dtype == "bf16" else torch.float32
        plan = bq.QuantizePerTokenPlan.select(None, bq.QuantizePerTokenDescriptor(m, k, "s8" if a.kind == "s8" else "e4m3"))
        xs = [torch.randn(m, k, device="cuda", generator=g).to(dt) for _ in range(a.buffers)]
        q = torch.empty((m, k), dtype=torch.int8 if a.kind == "s8" else torch.uint8, device="cuda")
        launch = lambda i: plan.run(None, xs[i % len(xs)], sa, q)
    elif a.kernel == "gemv":
        layout = bq.LayoutSku.Rcr if a.layout == "rcr" else bq.LayoutSku.Rrr
        plan = bq.GemvQ8Plan.select(None, bq.GemvQ8Descriptor(m, n, k, layout=layout))
        ws = torch.empty(max(plan.workspace_size(), 16), dtype=torch.uint8, device="cuda")
        x = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)
        weights = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device="cuda", generator=g) for _ in range(a.buffers)]
        calls = [bq.GemvQ8Args(a=x, b=w, d=d, scale_a=sa, scale_b=sb) for w in weights]
        launch = lambda i: plan.run(None, ws, calls[i % len(calls)])
    else:
        bq.set_tuning(0, a.block_n)
        if a.kind == "s8":
            plan = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(m, n, k))
            mk = lambda r: torch.randint(-127, 128, (r, k), dtype=torch.int8, device="cuda", generator=g)
        else:
            plan = bq.Fp8ScaledGemmPlan.select(None, bq.QGemmDescriptor(m, n, k), scale_mode=bq.SCALE_PER_ROW_COL)
            mk = lambda r: torch.randn(r, k, device="cuda", generator=g).to(torch.float8_e4m3fn).view(torch.uint8)
        x = mk(m)
        weights = [mk(n) for _ in range(a.buffers)]
        if a.epilogue == "gated" and a.kind == "s8":
            plan = bq.GatedMlpUpPlan.select(None, bq.GatedMlpUpDescriptor(m, n // 2, k))
            d = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
            calls = [bq.GatedMlpUpArgs(a=x, b_gate_up=w, d=d, scale_a=sa, scale_b=sb) for w in weights]
        elif a.epilogue == "bias_gelu" and a.kind == "s8":
            plan = bq.W8A8GemmPlan.select(None, bq.QGemmDescriptor(m, n, k, epilogue=bq.EpilogueKind.BiasGelu))
            bias = torch.randn(n, device="cuda", generator=g)
            calls = [bq.QGemmArgs(a=x, b=w, d=d, scale_a=sa, scale_b=sb, bias=bias) for w in weights]
        else:
            calls = [bq.QGemmArgs(a=x, b=w, d=d, scale_a=sa, scale_b=sb) for w in weights]
        launch = lambda i: plan.run(None, None, calls[i % len(calls)])

    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(a.iters):
        launch(i)
    e.record()
    torch.cuda.synchronize()
    print(f"{a.kernel} m={m} n={n} k={k}: {s.elapsed_time(e) / a.iters * 1e3:.1f} us per launch, "
          f"device status {bq.device_status()}")


if __name__ == "__main__":
    main()
