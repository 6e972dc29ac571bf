"""Multi-GPU parity of the column-parallel and row-parallel GEMMs at every power-of-two world size the box offers (2, 4,
8): each rank computes its N-slice with the tcgen05 kernel; the sharded output, the NCCL-gathered output (rank-major)
and the fused peer-store output (row-major) must all equal the unsharded oracle result, and so must the K-sharded
forward in both its forms.  Skipped with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import baracuda_b200 as bq
        from baracuda_b200 import parallel as par
        from oracle import pyoracle as orc

        ctx = par.TensorParallelContext.from_torch_distributed()
        dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
        bits = lambda t: t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
        for kind, (m, n, k) in (("w8a8", (300, 1024, 512)), ("fp8", (1024, 2048, 1024)), ("w8a8", (300, 224 * 4 * world, 512)),
                                ("fp8", (512, 256 * 3 * world, 640))):
            rng = np.random.default_rng(5)
            a = rng.standard_normal((m, k)).astype(np.float32)
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            if kind == "w8a8":
                aq, sa = orc.quantize_rows_s8(a)
                wq, sb = orc.quantize_rows_s8(w)
                want = orc.dequant_s32_bf16(orc.gemm_s8_s32(aq, wq, orc.RCR, m, n, k), sa, sb)
            else:
                aq, sa = orc.quantize_rows_e4m3(a)
                wq, sb = orc.quantize_rows_e4m3(w)
                want = orc.scale_f32_bf16(orc.gemm_e4m3_f32(aq, wq, orc.RCR, m, n, k), sa, sb)
            want_f = orc.bf16_bits_to_f32(want)
            w_local = par.shard_rows(torch.from_numpy(wq), world, rank).cuda()
            sb_local = par.shard_rows(torch.from_numpy(sb), world, rank).cuda()
            n_local = n // world
            lo = rank * n_local

            def check(got_bits, ref_bits, what):
                if kind == "w8a8":
                    assert np.array_equal(got_bits, ref_bits), f"{kind} {what} rank {rank}"
                else:
                    g, r = orc.bf16_bits_to_f32(got_bits), orc.bf16_bits_to_f32(ref_bits)
                    assert orc.compare_tolerant(r, g, 1e-2, 1e-4 * float(np.abs(want_f).max())) == -1, f"{kind} {what}"

            # sharded output
            y_local = torch.zeros((m, n_local), dtype=torch.bfloat16, device="cuda")
            plan = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind=kind, gather=par.GATHER_NONE)
            plan.forward(None, dev(aq), dev(sa), w_local, sb_local, y_local)
            torch.cuda.synchronize()
            check(bits(y_local), want[:, lo:lo + n_local], "sharded")
            if m % world == 0:
                # activations uploaded as M/G rows per rank and replicated over NVLink before the GEMM
                rows = m // world
                a_full = torch.zeros((m, k), dtype=torch.from_numpy(aq).dtype, device="cuda")
                sa_full = torch.zeros(m, dtype=torch.float32, device="cuda")
                plan.replicate_activations(None, dev(aq[rank * rows:(rank + 1) * rows]), dev(sa[rank * rows:(rank + 1) * rows]),
                                           a_full, sa_full)
                y_local.zero_()
                plan.forward(None, a_full, sa_full, w_local, sb_local, y_local)
                torch.cuda.synchronize()
                assert np.array_equal(a_full.cpu().numpy(), aq) and np.array_equal(sa_full.cpu().numpy(), sa)
                check(bits(y_local), want[:, lo:lo + n_local], "sharded, replicated activations")
            # NCCL all-gather, rank-major [G, M, N/G]
            y_full = torch.zeros((world, m, n_local), dtype=torch.bfloat16, device="cuda")
            plan = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind=kind, gather=par.GATHER_NCCL)
            plan.forward(None, dev(aq), dev(sa), w_local, sb_local, y_local, y_full=y_full)
            torch.cuda.synchronize()
            check(bits(par.gathered_to_row_major(y_full)), want, "nccl gather")
            # fused: the epilogue stores into every rank's row-major [M, N] buffer
            full_rm, ptrs = par.alloc_peer_buffers((m, n))
            full_rm.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            plan = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind=kind, gather=par.GATHER_FUSED_PEER_STORE)
            plan.forward(None, dev(aq), dev(sa), w_local, sb_local, y_local, peer_ptrs=ptrs, ldd_full=n)
            scratch = torch.zeros(1, device="cuda")
            ctx.stream_barrier(scratch)
            torch.cuda.synchronize()
            dist.barrier()
            check(bits(full_rm), want, "fused peer store")
            assert bq.device_status() == 0
            # fused through the switch: one multimem.st per tile to the multicast address of the buffers
            mc_rm, mc_ptrs, mc = par.alloc_peer_buffers_multicast((m, n))
            if mc:
                mc_rm.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                plan = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind=kind, gather=par.GATHER_FUSED_MULTICAST)
                for _ in range(2):
                    plan.forward(None, dev(aq), dev(sa), w_local, sb_local, y_local, peer_ptrs=mc_ptrs, ldd_full=n,
                                 multicast_ptr=mc)
                    ctx.stream_barrier(scratch)
                torch.cuda.synchronize()
                dist.barrier()
                check(bits(mc_rm), want, "fused multicast store")
                assert bq.device_status() == 0
            # the same weight stored row-major [K, N]: rank r's shard is a column range (strided view), fused gather
            if n_local % 16 == 0 and m >= 256:
                w_kn = torch.from_numpy(np.ascontiguousarray(wq.T)).cuda()
                full_rm.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                plan = par.ColumnParallelQGemmPlan(ctx, m, n, k, kind=kind, gather=par.GATHER_FUSED_PEER_STORE,
                                                   layout=bq.LayoutSku.Rrr)
                plan.forward(None, dev(aq), dev(sa), w_kn[:, lo:lo + n_local], sb_local, y_local, peer_ptrs=ptrs, ldd_full=n)
                ctx.stream_barrier(scratch)
                torch.cuda.synchronize()
                dist.barrier()
                check(bits(full_rm), want, "fused peer store, row-major weight")
                assert bq.device_status() == 0
        # K-sharded (row-parallel) forward: raw accumulators all-reduced, one dequant pass, bias added once
        for kind, (m, n, k) in (("w8a8", (300, 1040, 1024)), ("fp8", (512, 1024, 2048)), ("w8a8", (1024, 2048, 4096))):
            if k % (128 * world) != 0:
                continue
            rng = np.random.default_rng(11)
            a = rng.standard_normal((m, k)).astype(np.float32)
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            bias = rng.standard_normal(n).astype(np.float32)
            if kind == "w8a8":
                aq, sa = orc.quantize_rows_s8(a)      # one per-token scale over the whole K, shared by the ranks
                wq, sb = orc.quantize_rows_s8(w)
                y = orc.dequant_s32_f32(orc.gemm_s8_s32(aq, wq, orc.RCR, m, n, k), sa, sb)
            else:
                aq, sa = orc.quantize_rows_e4m3(a)
                wq, sb = orc.quantize_rows_e4m3(w)
                acc = orc.gemm_e4m3_f32(aq, wq, orc.RCR, m, n, k)
                y = ((sa[:, None] * sb[None, :]).astype(np.float32) * acc).astype(np.float32)
            want = orc.f32_to_bf16_bits((y + bias[None, :]).astype(np.float32))
            want_f = orc.bf16_bits_to_f32(want)
            plan = par.RowParallelQGemmPlan(ctx, m, n, k, kind=kind)
            ws = torch.empty(plan.workspace_size(), dtype=torch.uint8, device="cuda")
            y_d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
            plan.forward(None, par.shard_cols(torch.from_numpy(aq), world, rank).cuda(), dev(sa),
                         par.shard_cols(torch.from_numpy(wq), world, rank).cuda(), dev(sb), y_d, ws, bias=dev(bias))
            torch.cuda.synchronize()
            def check_rp(t, what):
                if kind == "w8a8":
                    assert np.array_equal(bits(t), want), f"{what} w8a8 rank {rank}"
                else:
                    g_f = orc.bf16_bits_to_f32(bits(t))
                    assert orc.compare_tolerant(want_f, g_f, 1e-2, 1e-4 * float(np.abs(want_f).max())) == -1, f"{what} fp8"

            check_rp(y_d, "row-parallel (nccl)")
            assert bq.device_status() == 0
            # fused: GEMM epilogue scatters raw partial sums to the owners, owners reduce + dequant + store to every rank
            if m % world == 0:
                y_sym, y_ptrs = par.alloc_peer_buffers((m, n))
                st_sym, st_ptrs = par.alloc_peer_buffers((world, m // world, n), dtype=torch.int32)
                y_sym.zero_()
                st_sym.fill_(0x7F7F7F7F)  # stale contents must not matter
                torch.cuda.synchronize()
                dist.barrier()
                fplan = par.RowParallelQGemmPlan(ctx, m, n, k, kind=kind, reduce=par.REDUCE_FUSED_PEER)
                scratch = torch.zeros(1, device="cuda")
                a_l = par.shard_cols(torch.from_numpy(aq), world, rank).cuda()
                w_l = par.shard_cols(torch.from_numpy(wq), world, rank).cuda()
                for _ in range(2):  # twice: the staging buffers are reused
                    fplan.forward_fused(None, a_l, dev(sa), w_l, dev(sb), y_ptrs, st_ptrs, scratch, bias=dev(bias))
                torch.cuda.synchronize()
                dist.barrier()
                check_rp(y_sym, "row-parallel (fused)")
                assert bq.device_status() == 0
                # the same with the flag barrier over peer memory instead of the one-float all-reduces: three calls on
                # stale staging contents, results cleared in between, no communicator involved in the exchange
                flag_buf, flag_ptrs = par.alloc_peer_flags()
                for rep in range(3):
                    y_sym.zero_()
                    torch.cuda.synchronize()
                    dist.barrier()
                    fplan.forward_fused(None, a_l, dev(sa), w_l, dev(sb), y_ptrs, st_ptrs, bias=dev(bias), peer_flags=flag_ptrs)
                    torch.cuda.synchronize()
                    check_rp(y_sym, f"row-parallel (fused, flag barrier, call {rep})")
                assert bq.device_status() == 0
                assert int(flag_buf[16].item()) == 6  # two barriers per call, epochs kept in the buffer
                ctx.flag_barrier(flag_ptrs)
                torch.cuda.synchronize()
                assert int(flag_buf[16].item()) == 7 and bq.device_status() == 0
                dist.barrier()
        ctx.destroy()
        with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def _worlds():
    """2, and the largest power of two the box offers (4 or 8) when that is more."""
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    top = 8 if n >= 8 else (4 if n >= 4 else (2 if n >= 2 else 0))
    return sorted({w for w in (2, top) if 2 <= w <= n})


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_and_row_parallel_parity(tmp_path, world):
    if world not in _worlds():
        pytest.skip(f"runs at world sizes {_worlds()} on this box")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
