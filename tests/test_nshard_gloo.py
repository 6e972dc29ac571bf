"""World-size-2 checks of the column-parallel host logic on CPU (gloo): shard bounds, the rank-major
gather layout and its row-major reassembly, and the unique-id hand-off, with the CPU oracle standing in
for the per-rank GEMM.  No GPU is involved."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from baracuda_b200 import parallel as par
from baracuda_b200.vocab import InvalidProblem


def test_shard_range_rules():
    assert par.shard_range(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert par.shard_range(16, 1, 0) == (0, 16)
    with pytest.raises(InvalidProblem):
        par.shard_range(10, 4, 0)          # N must divide evenly (lib.rs:781-785 of the reference)
    with pytest.raises(InvalidProblem):
        par.shard_range(16, 4, 4)
    with pytest.raises(InvalidProblem):
        par.TensorParallelContext(2, 2)
    w = torch.arange(24).reshape(6, 4)
    assert torch.equal(par.shard_rows(w, 3, 1), w[2:4])
    y = torch.arange(2 * 3 * 4).reshape(2, 3, 4)   # [G=2, M=3, N/G=4]
    full = par.gathered_to_row_major(y)
    assert full.shape == (3, 8) and torch.equal(full[:, :4], y[0]) and torch.equal(full[:, 4:], y[1])
    with pytest.raises(InvalidProblem):
        par.ColumnParallelQGemmPlan(par.TensorParallelContext(0, 2), 4, 7, 16)
    with pytest.raises(InvalidProblem):
        par.ColumnParallelQGemmPlan(par.TensorParallelContext(0, 2), 4, 8, 16, kind="bf16")
    plan = par.ColumnParallelQGemmPlan(par.TensorParallelContext(1, 2), 4, 8, 16, kind="w8a8", gather=par.GATHER_NCCL)
    assert (plan.n_local, plan.col0) == (4, 4)
    # K-sharded (row-parallel) plan: in_features must divide, each rank owns a column slice
    assert torch.equal(par.shard_cols(w, 2, 1), w[:, 2:4])
    with pytest.raises(InvalidProblem):
        par.RowParallelQGemmPlan(par.TensorParallelContext(0, 2), 4, 8, 15)
    with pytest.raises(InvalidProblem):
        par.RowParallelQGemmPlan(par.TensorParallelContext(0, 2), 4, 8, 16, reduce=5)
    rp = par.RowParallelQGemmPlan(par.TensorParallelContext(1, 2), 4, 8, 16)
    assert (rp.k_local, rp.k0) == (8, 8) and rp.workspace_size() == 4 * 8 * 4


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import ctypes as C

        from baracuda_b200 import _lib
        from oracle import pyoracle as orc

        m, n, k = 12, 40, 64
        rng = np.random.default_rng(99)  # same seed on every rank: replicated activations, full weight
        aq, sa = orc.quantize_rows_s8(rng.standard_normal((m, k)).astype(np.float32))
        wq, sb = orc.quantize_rows_s8((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        w_local = par.shard_rows(torch.from_numpy(wq), world, rank).numpy()
        sb_local = par.shard_rows(torch.from_numpy(sb), world, rank).numpy()
        n_local = n // world
        acc = orc.gemm_s8_s32(aq, w_local, orc.RCR, m, n_local, k)
        # gloo has no 16-bit integer transport: carry the bf16 bit patterns widened to int32
        y_local = torch.from_numpy(orc.dequant_s32_bf16(acc, sa, sb_local).astype(np.int32))
        parts = [torch.empty((m, n_local), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(parts, y_local.contiguous())
        y_full = torch.stack(parts)  # rank-major [G, M, N/G], what ncclAllGather writes
        got = par.gathered_to_row_major(y_full).numpy().astype(np.uint16)
        want = orc.dequant_s32_bf16(orc.gemm_s8_s32(aq, wq, orc.RCR, m, n, k), sa, sb)
        assert np.array_equal(got, want), "sharded + gathered result differs from the unsharded one"

        # K-sharded: every rank multiplies its K slice, the int32 partial sums are all-reduced (exact), one dequant
        a_k = par.shard_cols(torch.from_numpy(aq), world, rank).numpy()
        w_k = par.shard_cols(torch.from_numpy(wq), world, rank).numpy()
        part = torch.from_numpy(orc.gemm_s8_s32(a_k, w_k, orc.RCR, m, n, k // world))
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        assert np.array_equal(orc.dequant_s32_bf16(part.numpy(), sa, sb), want), "K-sharded result differs"
        st = lib_status = _lib.load().baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(
            rank, world, None, 1, m, n, k // world, None, k, None, k, None, n, None, None, None, 1.0, None, 0, None)
        assert st == 2  # no output, no scales

        # the unique id made on rank 0 reaches every rank unchanged
        lib = _lib.load()
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            assert lib.baracuda_q_nccl_unique_id(buf) == 0
        t = torch.tensor(list(buf), dtype=torch.uint8)
        dist.broadcast(t, src=0)
        ids = [torch.empty(128, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(ids, t)
        assert all(torch.equal(ids[0], x) for x in ids) and int(ids[0].sum()) > 0
        # argument validation of the sharded C entry point needs no GPU
        st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run(
            world, world, None, 0, m, n_local, k, None, k, None, k, None, n_local, None, None, 1.0, None, None, 0,
            None, 0, None)
        assert st == 2  # rank out of range
        st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run(
            rank, world, None, 1, m, n_local, k, None, k, None, k, None, n_local + 8, None, None, 1.0, None, None, 0,
            None, 0, None)
        assert st == 2  # the NCCL gather needs a d_full and a contiguous d_local
        with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
