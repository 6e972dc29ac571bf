"""Column-parallel (N-sharded) quantized linear inside one NVLink box.

Host-side mirror of the forward half of the reference's tensor-parallel layer
(`TensorParallelContext` and `ColumnParallelLinearPlan::{new, forward}`,
crates/baracuda-megatron/src/lib.rs:153-240, 729-905): rank r owns rows
[r*N/G, (r+1)*N/G) of the [N,K] weight and the matching weight scales, the
activations are replicated, every rank computes its output slice with the
tcgen05 GEMM, and the output is left sharded, NCCL all-gathered (rank-major
[G, M, N/G], the reference's contract) or written straight into every rank's
row-major [M, N] buffer by the GEMM epilogue over NVLink (fused mode).

One process per GPU.  torch.distributed is only used to hand the NCCL unique
id around; the collective itself is issued by the C library on the caller's
stream.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .plans import SCALE_PER_ROW_COL, _need_typed, _ptr, _stream_ptr
from .vocab import BaracudaError, InvalidProblem, LayoutSku, status_to_result

GATHER_NONE = 0
GATHER_NCCL = 1
GATHER_FUSED_PEER_STORE = 2
GATHER_FUSED_MULTICAST = 3


class CommUnavailable(BaracudaError):
    """libnccl.so.2 could not be loaded (status 6)."""


class CommFailure(BaracudaError):
    """An NCCL call returned an error (status 7)."""


def _check(status: int, what: str) -> None:
    if status == 6:
        raise CommUnavailable(f"{what}: NCCL is not loadable in this process")
    if status == 7:
        raise CommFailure(f"{what}: NCCL call failed")
    status_to_result(status, what)


def shard_range(out_features: int, world: int, rank: int) -> tuple[int, int]:
    """Rows of the [N,K] weight that `rank` owns.  N must divide evenly (lib.rs:781-785)."""
    if world < 1 or not (0 <= rank < world):
        raise InvalidProblem(f"rank {rank} outside world {world}")
    if out_features % world != 0:
        raise InvalidProblem(f"out_features {out_features} is not divisible by the world size {world}")
    per = out_features // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's contiguous row slice of a weight ([N,K]) or of a per-channel vector ([N])."""
    lo, hi = shard_range(t.shape[0], world, rank)
    return t[lo:hi].contiguous()


def shard_cols(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's contiguous K slice (columns) of a weight ([N,K]) or of the activations ([M,K]); K must divide
    evenly (RowParallelLinearPlan::new, lib.rs:1080-1110)."""
    lo, hi = shard_range(t.shape[1], world, rank)
    return t[:, lo:hi].contiguous()


def gathered_to_row_major(y_full: torch.Tensor) -> torch.Tensor:
    """[G, M, N/G] (what the all-gather produces, lib.rs:824-836) -> row-major [M, N]."""
    g, m, n_local = y_full.shape
    return y_full.permute(1, 0, 2).reshape(m, g * n_local)


class TensorParallelContext:
    """Rank, world size and this rank's NCCL communicator (lib.rs:153-240)."""

    def __init__(self, rank: int, world: int, comm: Optional[int] = None):
        if world < 1 or not (0 <= rank < world):
            raise InvalidProblem(f"rank {rank} outside world {world}")
        self.rank, self.world, self.comm = rank, world, comm

    @classmethod
    def from_torch_distributed(cls, group=None) -> "TensorParallelContext":
        """Rank 0 creates the NCCL unique id, torch.distributed broadcasts its 128 bytes, every rank joins."""
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if world == 1:
            return cls(0, 1, None)
        lib = _lib.load()
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            _check(lib.baracuda_q_nccl_unique_id(buf), "nccl_unique_id")
        backend = dist.get_backend(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        t = torch.tensor(list(buf), dtype=torch.uint8, device=dev)
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        id_bytes = (C.c_uint8 * 128)(*t.cpu().tolist())
        comm = C.c_void_p()
        _check(lib.baracuda_q_nccl_comm_init_rank(C.byref(comm), world, id_bytes, rank), "nccl_comm_init_rank")
        return cls(rank, world, comm.value)

    def stream_barrier(self, scratch: torch.Tensor, stream=None) -> None:
        """Orders the ranks on their streams (one-float all-reduce); used after the fused peer-store mode."""
        if self.world == 1:
            return
        _check(_lib.load().baracuda_q_nccl_stream_barrier(self.comm, scratch.data_ptr(), _stream_ptr(stream)),
               "nccl_stream_barrier")

    def flag_barrier(self, peer_flags: Sequence[int], stream=None, limit_cycles: int = 0) -> None:
        """Orders the ranks on their streams with the one-block flag-barrier kernel over peer memory (`peer_flags`: one
        pointer per rank from alloc_peer_flags) instead of an all-reduce: about 5 us instead of about 20 at eight GPUs.
        A wait that runs out (about a second by default) shows up as device_status() == 301."""
        if self.world == 1:
            return
        if len(peer_flags) != self.world:
            raise InvalidProblem("one flag buffer per rank is needed")
        flags = (C.c_void_p * self.world)(*peer_flags)
        _check(_lib.load().baracuda_q_peer_barrier_run(flags, self.rank, self.world, limit_cycles, _stream_ptr(stream)),
               "peer_barrier")

    def destroy(self) -> None:
        if self.comm:
            _check(_lib.load().baracuda_q_nccl_comm_destroy(self.comm), "nccl_comm_destroy")
            self.comm = None


class ColumnParallelQGemmPlan:
    """N-sharded FP8 or W8A8 GEMM with an optional replicated output."""

    def __init__(self, ctx: TensorParallelContext, m: int, out_features: int, k: int, kind: str = "fp8",
                 scale_mode: int = SCALE_PER_ROW_COL, gather: int = GATHER_NONE, layout: LayoutSku = LayoutSku.Rcr):
        """`layout` Rcr: the shard is rows [lo, hi) of the [N, K] weight (contiguous).  Rrr: the weight is row-major
        [K, N] and the shard is its column range [lo, hi) -- pass the strided view `w[:, lo:hi]` as `w_local`."""
        if kind not in ("fp8", "w8a8"):
            raise InvalidProblem("kind must be 'fp8' or 'w8a8'")
        if gather not in (GATHER_NONE, GATHER_NCCL, GATHER_FUSED_PEER_STORE, GATHER_FUSED_MULTICAST):
            raise InvalidProblem("unknown gather mode")
        if layout not in (LayoutSku.Rcr, LayoutSku.Rrr):
            raise InvalidProblem("unknown layout")
        self.layout = layout
        if min(m, out_features, k) < 0:
            raise InvalidProblem("negative dimension")
        lo, hi = shard_range(out_features, ctx.world, ctx.rank)
        self.ctx, self.m, self.n, self.k = ctx, m, out_features, k
        self.n_local, self.col0 = hi - lo, lo
        self.kind, self.scale_mode, self.gather = kind, scale_mode, gather

    def _operand_dtypes(self):
        return (torch.int8,) if self.kind == "w8a8" else (torch.uint8, torch.float8_e4m3fn)

    def replicate_activations(self, stream, a_rows: torch.Tensor, scale_a_rows: torch.Tensor, a_full: torch.Tensor,
                              scale_a_full: torch.Tensor) -> None:
        """Each rank holds rows [rank*M/G, (rank+1)*M/G) of the activations (and of scale_a), e.g. freshly uploaded
        from the host; all-gathers them over NVLink into the replicated [M, K] / [M] buffers the forward reads, so a
        step moves M*K/G bytes over each GPU's host link instead of M*K.  M must divide by the world size."""
        g = self.ctx.world
        if self.m % g != 0:
            raise InvalidProblem(f"M = {self.m} is not divisible by the world size {g}")
        rows = self.m // g
        _need_typed(a_rows, self._operand_dtypes(), rows * self.k, "a_rows")
        _need_typed(a_full, self._operand_dtypes(), self.m * self.k, "a_full")
        _need_typed(scale_a_rows, torch.float32, rows, "scale_a_rows")
        _need_typed(scale_a_full, torch.float32, self.m, "scale_a_full")
        lib = _lib.load()
        s = _stream_ptr(stream)
        _check(lib.baracuda_q_nccl_all_gather_bytes(self.ctx.comm, g, _ptr(a_rows), _ptr(a_full), rows * self.k, s),
               "replicate_activations")
        _check(lib.baracuda_q_nccl_all_gather_bytes(self.ctx.comm, g, _ptr(scale_a_rows), _ptr(scale_a_full), rows * 4, s),
               "replicate_activations")

    def forward(self, stream, a: torch.Tensor, scale_a: torch.Tensor, w_local: torch.Tensor,
                scale_b_local: torch.Tensor, y_local: torch.Tensor, y_full: Optional[torch.Tensor] = None,
                peer_ptrs: Optional[Sequence[int]] = None, ldd_full: int = 0, alpha: float = 1.0,
                multicast_ptr: int = 0) -> None:
        """Y_local[M, N/G] = dequant(A x W_local^T); then the selected gather.  Asynchronous on `stream`.
        GATHER_FUSED_MULTICAST also needs `multicast_ptr`, the multicast address of the peer buffers."""
        per_vec = self.kind == "w8a8" or self.scale_mode == SCALE_PER_ROW_COL
        _need_typed(a, self._operand_dtypes(), self.m * self.k, "a")
        _need_typed(w_local, self._operand_dtypes(), self.n_local * self.k, "w_local")
        _need_typed(scale_a, torch.float32, self.m if per_vec else 1, "scale_a")
        _need_typed(scale_b_local, torch.float32, self.n_local if per_vec else 1, "scale_b_local")
        _need_typed(y_local, torch.bfloat16, self.m * self.n_local, "y_local")
        if self.gather == GATHER_NCCL:
            _need_typed(y_full, torch.bfloat16, self.m * self.n, "y_full")
        peers = None
        if self.gather in (GATHER_FUSED_PEER_STORE, GATHER_FUSED_MULTICAST):
            if peer_ptrs is None or len(peer_ptrs) != self.ctx.world:
                raise InvalidProblem("fused mode needs one peer buffer pointer per rank")
            if self.gather == GATHER_FUSED_MULTICAST:
                if not multicast_ptr:
                    raise InvalidProblem("the multicast mode needs the buffers' multicast address")
                peers = (C.c_void_p * (self.ctx.world + 1))(*peer_ptrs, multicast_ptr)
            else:
                peers = (C.c_void_p * self.ctx.world)(*peer_ptrs)
            ldd_full = ldd_full or self.n
        lib = _lib.load()
        if self.layout is LayoutSku.Rrr:
            if w_local.dim() != 2 or w_local.stride(1) != 1 or w_local.stride(0) < self.n_local:
                raise InvalidProblem("Rrr: w_local must be the [K, N/G] column view of a row-major [K, N] weight")
            ldb = max(int(w_local.stride(0)), 1)
        else:
            ldb = max(self.k, 1)
        common = (self.ctx.rank, self.ctx.world, self.ctx.comm, self.gather, self.m, self.n_local, self.k,
                  _ptr(a), max(self.k, 1), _ptr(w_local), ldb, _ptr(y_local), max(self.n_local, 1),
                  _ptr(scale_a), _ptr(scale_b_local))
        tail = (_ptr(y_full), peers, ldd_full, None, 0, _stream_ptr(stream))
        lay = self.layout.value
        if self.kind == "fp8":
            st = getattr(lib, f"baracuda_kernels_gemm_fp8_e4m3_{lay}_bf16_sm100a_nshard_run")(*common, self.scale_mode, alpha, *tail)
        else:
            st = getattr(lib, f"baracuda_kernels_gemm_w8a8_s8_{lay}_bf16_sm100a_nshard_run")(*common, alpha, *tail)
        _check(st, "ColumnParallelQGemmPlan.forward")


REDUCE_NONE, REDUCE_NCCL, REDUCE_FUSED_PEER = 0, 1, 2


class RowParallelQGemmPlan:
    """K-sharded FP8 or W8A8 GEMM: every rank multiplies its K slice, the raw accumulators are all-reduced
    (ncclAllReduce, sum) and dequantised once -- the forward of the reference's RowParallelLinearPlan
    (crates/baracuda-megatron/src/lib.rs:1002-1200), for 8-bit operands.  `scale_a` is one per-token scale
    taken over the whole K, the same on every rank."""

    def __init__(self, ctx: TensorParallelContext, m: int, out_features: int, in_features: int, kind: str = "w8a8",
                 scale_mode: int = SCALE_PER_ROW_COL, reduce: int = REDUCE_NCCL):
        if kind not in ("fp8", "w8a8"):
            raise InvalidProblem("kind must be 'fp8' or 'w8a8'")
        if reduce not in (REDUCE_NONE, REDUCE_NCCL, REDUCE_FUSED_PEER):
            raise InvalidProblem("unknown reduce mode")
        if reduce == REDUCE_FUSED_PEER and (ctx.world < 2 or m % ctx.world != 0):
            raise InvalidProblem("the fused mode needs two or more ranks and M divisible by the world size")
        if min(m, out_features, in_features) < 0:
            raise InvalidProblem("negative dimension")
        lo, hi = shard_range(in_features, ctx.world, ctx.rank)
        self.ctx, self.m, self.n, self.k = ctx, m, out_features, in_features
        self.k_local, self.k0 = hi - lo, lo
        self.kind, self.scale_mode, self.reduce = kind, scale_mode, reduce

    def workspace_size(self) -> int:
        return int(_lib.load().baracuda_kernels_gemm_q8_kshard_workspace_size(self.m, self.n))

    def _check_operands(self, a_local, scale_a, w_local, scale_b, bias) -> None:
        ops = (torch.int8,) if self.kind == "w8a8" else (torch.uint8, torch.float8_e4m3fn)
        per_vec = self.kind == "w8a8" or self.scale_mode == SCALE_PER_ROW_COL
        _need_typed(a_local, ops, self.m * self.k_local, "a_local")
        _need_typed(w_local, ops, self.n * self.k_local, "w_local")
        _need_typed(scale_a, torch.float32, self.m if per_vec else 1, "scale_a")
        _need_typed(scale_b, torch.float32, self.n if per_vec else 1, "scale_b")
        if bias is not None:
            _need_typed(bias, torch.float32, self.n, "bias")

    def forward(self, stream, a_local: torch.Tensor, scale_a: torch.Tensor, w_local: torch.Tensor,
                scale_b: torch.Tensor, y: torch.Tensor, workspace: torch.Tensor,
                bias: Optional[torch.Tensor] = None, alpha: float = 1.0) -> None:
        """Y[M, N] = bf16((scale_a x scale_b) * sum_ranks(A_local x W_local^T) * alpha + bias) on every rank."""
        self._check_operands(a_local, scale_a, w_local, scale_b, bias)
        _need_typed(y, torch.bfloat16, self.m * self.n, "y")
        ws_bytes = workspace.numel() * workspace.element_size()
        lib = _lib.load()
        common = (self.ctx.rank, self.ctx.world, self.ctx.comm, self.reduce, self.m, self.n, self.k_local,
                  _ptr(a_local), max(self.k_local, 1), _ptr(w_local), max(self.k_local, 1), _ptr(y), max(self.n, 1),
                  _ptr(scale_a), _ptr(scale_b))
        tail = (_ptr(bias), alpha, _ptr(workspace), ws_bytes, _stream_ptr(stream))
        if self.kind == "fp8":
            st = lib.baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run(*common, self.scale_mode, *tail)
        else:
            st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(*common, *tail)
        _check(st, "RowParallelQGemmPlan.forward")

    def forward_fused(self, stream, a_local: torch.Tensor, scale_a: torch.Tensor, w_local: torch.Tensor,
                      scale_b: torch.Tensor, peer_y: Sequence[int], peer_staging: Sequence[int],
                      barrier_scratch: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, alpha: float = 1.0,
                      ldy: int = 0, peer_flags: Optional[Sequence[int]] = None) -> None:
        """REDUCE_FUSED_PEER: the GEMM epilogue scatters the partial sums into the owners' staging buffers, each owner
        adds, dequantises and stores its rows into every rank's result.  `peer_y` / `peer_staging`: one device pointer per
        rank (see alloc_peer_buffers): [M, N] bf16 and [world, M/world, N] int32.  The ranks meet twice per call: through a
        one-float all-reduce on `barrier_scratch`, or, when `peer_flags` (alloc_peer_flags) is given, through the flag
        barrier over peer memory -- no communicator involved."""
        if self.reduce != REDUCE_FUSED_PEER:
            raise InvalidProblem("plan was not built for the fused mode")
        if len(peer_y) != self.ctx.world or len(peer_staging) != self.ctx.world:
            raise InvalidProblem("one pointer per rank is needed")
        self._check_operands(a_local, scale_a, w_local, scale_b, bias)
        ys = (C.c_void_p * self.ctx.world)(*peer_y)
        st_ptrs = (C.c_void_p * self.ctx.world)(*peer_staging)
        lib = _lib.load()
        if peer_flags is not None:
            if len(peer_flags) != self.ctx.world:
                raise InvalidProblem("one flag buffer per rank is needed")
            flags = (C.c_void_p * self.ctx.world)(*peer_flags)
            head = (self.ctx.rank, self.ctx.world, self.m, self.n, self.k_local, _ptr(a_local), max(self.k_local, 1),
                    _ptr(w_local), max(self.k_local, 1), ys, ldy or max(self.n, 1), _ptr(scale_a), _ptr(scale_b))
            rest = (_ptr(bias), alpha, st_ptrs, flags, _stream_ptr(stream))
            if self.kind == "fp8":
                st = lib.baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run(*head, self.scale_mode, *rest)
            else:
                st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run(*head, *rest)
            _check(st, "RowParallelQGemmPlan.forward_fused")
            return
        if barrier_scratch is None:
            raise InvalidProblem("barrier_scratch or peer_flags is needed")
        _need_typed(barrier_scratch, torch.float32, 1, "barrier_scratch")
        common = (self.ctx.rank, self.ctx.world, self.ctx.comm, self.m, self.n, self.k_local, _ptr(a_local),
                  max(self.k_local, 1), _ptr(w_local), max(self.k_local, 1), ys, ldy or max(self.n, 1), _ptr(scale_a),
                  _ptr(scale_b))
        tail = (_ptr(bias), alpha, st_ptrs, _ptr(barrier_scratch), _stream_ptr(stream))
        if self.kind == "fp8":
            st = lib.baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run(*common, self.scale_mode, *tail)
        else:
            st = lib.baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run(*common, *tail)
        _check(st, "RowParallelQGemmPlan.forward_fused")


def alloc_peer_buffers(shape, dtype=torch.bfloat16, group=None):
    """One buffer of `shape` per rank, each mapped into every rank's address space (NVLink peer
    memory), for the fused peer-store mode.  Returns (this rank's tensor, [device pointer per rank]).
    Uses torch's symmetric-memory allocator as plumbing; the stores themselves are issued by the
    GEMM epilogue."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    local = symm_mem.empty(*shape, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
    handle = symm_mem.rendezvous(local, group=group)
    return local, [int(p) for p in handle.buffer_ptrs]


def alloc_peer_flags(group=None):
    """The flag buffers of the peer barrier: one zero-filled buffer per rank, each mapped into every rank's address space.
    Returns (this rank's tensor, [device pointer per rank]); every rank has zeroed its buffer and all ranks have met
    before this returns, so the first barrier finds clean flags."""
    import torch.distributed as dist

    words = int(_lib.load().baracuda_q_peer_barrier_flag_bytes()) // 4
    local, ptrs = alloc_peer_buffers((words,), dtype=torch.int32, group=group)
    local.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    return local, ptrs


def alloc_peer_buffers_multicast(shape, dtype=torch.bfloat16, group=None):
    """As alloc_peer_buffers, plus the buffers' multicast address (0 when the fabric or the allocator offers none):
    a store to it lands at the same offset of every rank's buffer (GATHER_FUSED_MULTICAST)."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    local = symm_mem.empty(*shape, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
    handle = symm_mem.rendezvous(local, group=group)
    mc = int(getattr(handle, "multicast_ptr", 0) or 0)
    return local, [int(p) for p in handle.buffer_ptrs], mc
