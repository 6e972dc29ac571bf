// Column-parallel (N-sharded) entry points: each rank runs the tcgen05 GEMM on
// its slice of the weight rows and, when the caller wants the output
// replicated, either NCCL all-gathers the bf16 slices (rank-major
// [world, M, N/world], the reference's contract) or — fused — lets the GEMM
// epilogue store every tile straight into each peer's row-major [M, N] buffer
// over NVLink while the tensor cores work on the next tile.
//
// Follows the forward of the reference's ColumnParallelLinearPlan
//   crates/baracuda-megatron/src/lib.rs:729-905 (local GEMM, then all_gather)
// and the communicator calls of
//   crates/baracuda-nccl/src/lib.rs:243-261, 468-489 (init by unique id, all_gather).
// NCCL is resolved at run time (dlopen of libnccl.so.2, as the reference's
// baracuda-nccl-sys does, crates/baracuda-nccl-sys/src/lib.rs:347-431); a
// library that is already loaded in the process is reused.

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "../../include/baracuda_kernels_q.h"
#include "launch.h"

namespace {

// The few NCCL declarations used here (stable across NCCL 2.x).
struct NcclUniqueId {
    char internal[128];
};
using NcclComm = void*;
constexpr int kNcclInt8 = 0, kNcclInt32 = 2, kNcclFloat32 = 7, kNcclBfloat16 = 9;
constexpr int kNcclSum = 0;

struct NcclApi {
    int (*GetVersion)(int*) = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // reuse a copy the process already has
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) return a;
        a.GetVersion = reinterpret_cast<decltype(a.GetVersion)>(dlsym(h, "ncclGetVersion"));
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
        a.ok = a.GetVersion && a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather && a.AllReduce;
        return a;
    }();
    return api;
}

int32_t nshard_run(int32_t layout, int32_t kind, int32_t rank, int32_t world, void* comm, int32_t gather, int32_t m, int32_t n_local,
                   int32_t k, const void* a, int64_t lda, const void* b_local, int64_t ldb, void* d_local, int64_t ldd,
                   const void* scale_a, const void* scale_b_local, int32_t scale_mode, float alpha, void* d_full,
                   void* const* peer_d, int64_t ldd_full, void* stream) {
    if (world < 1 || rank < 0 || rank >= world) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (gather < BARACUDA_Q_GATHER_NONE || gather > BARACUDA_Q_GATHER_FUSED_MULTICAST)
        return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (m < 0 || n_local < 0 || k < 0) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const bool fused = gather == BARACUDA_Q_GATHER_FUSED_PEER_STORE || gather == BARACUDA_Q_GATHER_FUSED_MULTICAST;
    void* mc_d = nullptr;
    if (fused) {
        if (world > BARACUDA_Q_MAX_PEERS || !peer_d) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
        if (ldd_full < static_cast<int64_t>(n_local) * world) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
        for (int r = 0; r < world; ++r) {
            if (!peer_d[r]) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
        }
        if (gather == BARACUDA_Q_GATHER_FUSED_MULTICAST) {
            mc_d = peer_d[world];  // one more entry: the multicast address of the same buffers
            if (!mc_d) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
        }
    }
    if (gather == BARACUDA_Q_GATHER_NCCL) {
        if (!d_full || (world > 1 && !comm)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
        // ncclAllGather sends one contiguous block per rank
        if (ldd != (n_local > 0 ? n_local : 1)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    }

    int32_t st;
    if (kind == bq::BQ_KIND_S8) {
        st = bq::launch_gemm_bf16_checked(layout, kind, m, n_local, k, a, lda, b_local, ldb, d_local, ldd, scale_a, scale_b_local,
                                         BARACUDA_Q_SCALE_PER_ROW_COL, alpha, fused ? peer_d : nullptr, world, rank, ldd_full, s,
                                         mc_d);
    } else {
        st = bq::launch_gemm_bf16_checked(layout, kind, m, n_local, k, a, lda, b_local, ldb, d_local, ldd, scale_a, scale_b_local,
                                         scale_mode, alpha, fused ? peer_d : nullptr, world, rank, ldd_full, s, mc_d);
    }
    if (st != BARACUDA_Q_STATUS_OK) return st;
    if (gather != BARACUDA_Q_GATHER_NCCL) return BARACUDA_Q_STATUS_OK;

    const size_t count = static_cast<size_t>(m) * static_cast<size_t>(n_local);
    if (count == 0) return BARACUDA_Q_STATUS_OK;
    if (world == 1) {
        // degenerate world: the collective is a device-to-device copy (the reference does the same,
        // crates/baracuda-megatron/src/lib.rs:53-57)
        if (d_full != d_local &&
            cudaMemcpyAsync(d_full, d_local, count * 2, cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return BARACUDA_Q_STATUS_LAUNCH_FAILURE;
        }
        return BARACUDA_Q_STATUS_OK;
    }
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    if (nccl().AllGather(d_local, d_full, count, kNcclBfloat16, comm, s) != 0) return BARACUDA_Q_STATUS_COMM_FAILURE;
    return BARACUDA_Q_STATUS_OK;
}

// K-sharded ("row-parallel") forward: Y_partial = X_local x W_local^T on this rank's K slice, all-reduce of the raw
// accumulators, then one dequant pass (crates/baracuda-megatron/src/lib.rs:1002-1200: local GEMM, all_reduce(Sum),
// bias after the reduction).  Adding int32 sums is exact, so the W8A8 result has the bits of the unsharded GEMM.
int32_t kshard_run(int32_t kind, int32_t rank, int32_t world, void* comm, int32_t reduce, int32_t m, int32_t n,
                   int32_t k_local, const void* a_local, int64_t lda, const void* b_local, int64_t ldb, void* d,
                   int64_t ldd, const void* scale_a, const void* scale_b, int32_t scale_mode, const void* bias, float alpha,
                   void* workspace, size_t workspace_bytes, void* stream) {
    if (world < 1 || rank < 0 || rank >= world) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (reduce != BARACUDA_Q_REDUCE_NONE && reduce != BARACUDA_Q_REDUCE_NCCL) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (m < 0 || n < 0 || k_local < 0) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (ldd < (n > 0 ? n : 1)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (m == 0 || n == 0) return BARACUDA_Q_STATUS_OK;
    if (!d || !scale_a || !scale_b) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (scale_mode != BARACUDA_Q_SCALE_PER_TENSOR && scale_mode != BARACUDA_Q_SCALE_PER_ROW_COL)
        return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (reduce == BARACUDA_Q_REDUCE_NCCL && world > 1 && !comm) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    const size_t count = static_cast<size_t>(m) * static_cast<size_t>(n);
    if (!workspace || workspace_bytes < count * 4) return BARACUDA_Q_STATUS_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return BARACUDA_Q_STATUS_MISALIGNED;
    // int32 partial sums are added across ranks: the whole K (k_local * world) must keep them inside 32 bits
    if (kind == bq::BQ_KIND_S8 && static_cast<int64_t>(k_local) * world > 131071) return BARACUDA_Q_STATUS_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const int32_t st = kind == bq::BQ_KIND_S8
                           ? baracuda_kernels_gemm_s8_rcr_s32_sm100a_run(m, n, k_local, a_local, lda, b_local, ldb, nullptr, 0,
                                                                         workspace, n, 1.0f, 0.0f, nullptr, 0, stream)
                           : baracuda_kernels_gemm_fp8_e4m3_rcr_f32_sm100a_run(m, n, k_local, a_local, lda, b_local, ldb,
                                                                               nullptr, 0, workspace, n, 1.0f, 0.0f, nullptr,
                                                                               0, stream);
    if (st != BARACUDA_Q_STATUS_OK) return st;
    if (reduce == BARACUDA_Q_REDUCE_NCCL && world > 1) {
        if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
        if (nccl().AllReduce(workspace, workspace, count, kind == bq::BQ_KIND_S8 ? kNcclInt32 : kNcclFloat32, kNcclSum, comm,
                             s) != 0) {
            return BARACUDA_Q_STATUS_COMM_FAILURE;
        }
    }
    return bq::launch_dequant_rows(kind, m, n, workspace, n, static_cast<const float*>(scale_a),
                                   static_cast<const float*>(scale_b), scale_mode, alpha, static_cast<const float*>(bias), d,
                                   ldd, s);
}

// The same forward with both exchanges done by the kernels themselves over peer memory: the GEMM epilogue scatters its raw
// partial sums by row block into the owners' staging buffers while the tensor cores work on the next tile
// (GEMM -> reduce-scatter in one kernel), each owner adds its `world` slots, dequantises, and stores the bf16 rows into
// every rank's output (reduce -> all-gather in one kernel).  Two one-float all-reduces order the ranks in between.
int32_t kshard_fused_run(int32_t kind, int32_t rank, int32_t world, void* comm, int32_t m, int32_t n, int32_t k_local,
                         const void* a_local, int64_t lda, const void* b_local, int64_t ldb, void* const* peer_y, int64_t ldy,
                         const void* scale_a, const void* scale_b, int32_t scale_mode, const void* bias, float alpha,
                         void* const* peer_staging, void* barrier_scratch, void* stream, void* const* peer_flags = nullptr) {
    if (world < 2 || world > BARACUDA_Q_MAX_PEERS || rank < 0 || rank >= world) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (m < 0 || n < 0 || k_local < 0 || (m % world) != 0) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (ldy < (n > 0 ? n : 1)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (m == 0 || n == 0) return BARACUDA_Q_STATUS_OK;
    if (!peer_y || !peer_staging || !scale_a || !scale_b) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (!peer_flags && (!comm || !barrier_scratch)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (scale_mode != BARACUDA_Q_SCALE_PER_TENSOR && scale_mode != BARACUDA_Q_SCALE_PER_ROW_COL)
        return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (k_local == 0) return BARACUDA_Q_STATUS_UNSUPPORTED;
    if (!peer_flags && !nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the two points where the ranks must meet: a one-float all-reduce, or the flag barrier over peer memory
    auto meet = [&]() -> int32_t {
        if (peer_flags) return bq::launch_peer_flag_barrier(peer_flags, rank, world, 0, s);
        return nccl().AllReduce(barrier_scratch, barrier_scratch, 1, kNcclFloat32, kNcclSum, comm, s) == 0
                   ? BARACUDA_Q_STATUS_OK
                   : BARACUDA_Q_STATUS_COMM_FAILURE;
    };
    int32_t st = bq::launch_gemm_raw_reduce_scatter_checked(kind, m, n, k_local, a_local, lda, b_local, ldb, peer_staging, world,
                                                            rank, s);
    if (st != BARACUDA_Q_STATUS_OK) return st;
    // every rank's partial sums have landed in the owners' staging buffers
    if (const int32_t b = meet(); b != BARACUDA_Q_STATUS_OK) return b;
    st = bq::launch_reduce_dequant_broadcast(kind, rank, world, m / world, n, peer_staging[rank],
                                             static_cast<const float*>(scale_a), static_cast<const float*>(scale_b), scale_mode,
                                             alpha, static_cast<const float*>(bias), peer_y, ldy, s);
    if (st != BARACUDA_Q_STATUS_OK) return st;
    // every owner's rows have landed in every rank's output, and the staging buffers may be written again
    return meet();
}

}  // namespace

extern "C" {

int32_t baracuda_q_nccl_version(void) {
    if (!nccl().ok) return 0;
    int v = 0;
    return nccl().GetVersion(&v) == 0 ? v : 0;
}

int32_t baracuda_q_nccl_unique_id(void* id_out_128_bytes) {
    if (!id_out_128_bytes) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    NcclUniqueId id;
    if (nccl().GetUniqueId(&id) != 0) return BARACUDA_Q_STATUS_COMM_FAILURE;
    memcpy(id_out_128_bytes, &id, sizeof(id));
    return BARACUDA_Q_STATUS_OK;
}

int32_t baracuda_q_nccl_comm_init_rank(void** comm_out, int32_t world, const void* id_128_bytes, int32_t rank) {
    if (!comm_out || !id_128_bytes || world < 1 || rank < 0 || rank >= world) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    NcclUniqueId id;
    memcpy(&id, id_128_bytes, sizeof(id));
    NcclComm c = nullptr;
    if (nccl().CommInitRank(&c, world, id, rank) != 0) return BARACUDA_Q_STATUS_COMM_FAILURE;
    *comm_out = c;
    return BARACUDA_Q_STATUS_OK;
}

int32_t baracuda_q_nccl_comm_destroy(void* comm) {
    if (!comm) return BARACUDA_Q_STATUS_OK;
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    return nccl().CommDestroy(comm) == 0 ? BARACUDA_Q_STATUS_OK : BARACUDA_Q_STATUS_COMM_FAILURE;
}

int32_t baracuda_q_nccl_stream_barrier(void* comm, void* scratch_one_float, void* stream) {
    if (!comm || !scratch_one_float) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    return nccl().AllReduce(scratch_one_float, scratch_one_float, 1, kNcclFloat32, kNcclSum, comm,
                            static_cast<cudaStream_t>(stream)) == 0
               ? BARACUDA_Q_STATUS_OK
               : BARACUDA_Q_STATUS_COMM_FAILURE;
}

int32_t baracuda_q_nccl_all_gather_bytes(void* comm, int32_t world, const void* send, void* recv, size_t bytes_per_rank,
                                         void* stream) {
    if (world < 1 || (!send && bytes_per_rank) || (!recv && bytes_per_rank)) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (bytes_per_rank == 0) return BARACUDA_Q_STATUS_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (world == 1) {
        if (recv != send && cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return BARACUDA_Q_STATUS_LAUNCH_FAILURE;
        }
        return BARACUDA_Q_STATUS_OK;
    }
    if (!comm) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    if (!nccl().ok) return BARACUDA_Q_STATUS_COMM_UNAVAILABLE;
    return nccl().AllGather(send, recv, bytes_per_rank, kNcclInt8, comm, s) == 0 ? BARACUDA_Q_STATUS_OK
                                                                                 : BARACUDA_Q_STATUS_COMM_FAILURE;
}

int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather, int32_t m, int32_t n_local, int32_t k, const void* a,
    int64_t lda, const void* b_local, int64_t ldb, void* d_local, int64_t ldd, const void* scale_a,
    const void* scale_b_local, int32_t scale_mode, float alpha, void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return nshard_run(bq::BQ_LAYOUT_RCR, bq::BQ_KIND_E4M3, rank, world, comm, gather, m, n_local, k, a, lda, b_local, ldb,
                      d_local, ldd, scale_a, scale_b_local, scale_mode, alpha, d_full, peer_d, ldd_full, stream);
}

int32_t baracuda_kernels_gemm_fp8_e4m3_rrr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather, int32_t m, int32_t n_local, int32_t k, const void* a,
    int64_t lda, const void* b_local, int64_t ldb, void* d_local, int64_t ldd, const void* scale_a,
    const void* scale_b_local, int32_t scale_mode, float alpha, void* d_full, void* const* peer_d, int64_t ldd_full,
    void* workspace, size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return nshard_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_E4M3, rank, world, comm, gather, m, n_local, k, a, lda, b_local, ldb,
                      d_local, ldd, scale_a, scale_b_local, scale_mode, alpha, d_full, peer_d, ldd_full, stream);
}

int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather, int32_t m, int32_t n_local, int32_t k, const void* a,
    int64_t lda, const void* b_local, int64_t ldb, void* d_local, int64_t ldd, const void* scale_a,
    const void* scale_b_local, float alpha, void* d_full, void* const* peer_d, int64_t ldd_full, void* workspace,
    size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return nshard_run(bq::BQ_LAYOUT_RCR, bq::BQ_KIND_S8, rank, world, comm, gather, m, n_local, k, a, lda, b_local, ldb,
                      d_local, ldd, scale_a, scale_b_local, BARACUDA_Q_SCALE_PER_ROW_COL, alpha, d_full, peer_d, ldd_full,
                      stream);
}

int32_t baracuda_kernels_gemm_w8a8_s8_rrr_bf16_sm100a_nshard_run(
    int32_t rank, int32_t world, void* comm, int32_t gather, int32_t m, int32_t n_local, int32_t k, const void* a,
    int64_t lda, const void* b_local, int64_t ldb, void* d_local, int64_t ldd, const void* scale_a,
    const void* scale_b_local, float alpha, void* d_full, void* const* peer_d, int64_t ldd_full, void* workspace,
    size_t workspace_bytes, void* stream) {
    (void)workspace;
    (void)workspace_bytes;
    return nshard_run(bq::BQ_LAYOUT_RRR, bq::BQ_KIND_S8, rank, world, comm, gather, m, n_local, k, a, lda, b_local, ldb,
                      d_local, ldd, scale_a, scale_b_local, BARACUDA_Q_SCALE_PER_ROW_COL, alpha, d_full, peer_d, ldd_full,
                      stream);
}

size_t baracuda_kernels_gemm_q8_kshard_workspace_size(int32_t m, int32_t n) {
    return (m > 0 && n > 0) ? static_cast<size_t>(m) * static_cast<size_t>(n) * 4 : 0;
}

int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_run(
    int32_t rank, int32_t world, void* comm, int32_t reduce, int32_t m, int32_t n, int32_t k_local, const void* a_local,
    int64_t lda, const void* b_local, int64_t ldb, void* d, int64_t ldd, const void* scale_a, const void* scale_b,
    const void* bias, float alpha, void* workspace, size_t workspace_bytes, void* stream) {
    return kshard_run(bq::BQ_KIND_S8, rank, world, comm, reduce, m, n, k_local, a_local, lda, b_local, ldb, d, ldd, scale_a,
                      scale_b, BARACUDA_Q_SCALE_PER_ROW_COL, bias, alpha, workspace, workspace_bytes, stream);
}

int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_run(
    int32_t rank, int32_t world, void* comm, int32_t reduce, int32_t m, int32_t n, int32_t k_local, const void* a_local,
    int64_t lda, const void* b_local, int64_t ldb, void* d, int64_t ldd, const void* scale_a, const void* scale_b,
    int32_t scale_mode, const void* bias, float alpha, void* workspace, size_t workspace_bytes, void* stream) {
    return kshard_run(bq::BQ_KIND_E4M3, rank, world, comm, reduce, m, n, k_local, a_local, lda, b_local, ldb, d, ldd, scale_a,
                      scale_b, scale_mode, bias, alpha, workspace, workspace_bytes, stream);
}

int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_run(
    int32_t rank, int32_t world, void* comm, int32_t m, int32_t n, int32_t k_local, const void* a_local, int64_t lda,
    const void* b_local, int64_t ldb, void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    const void* bias, float alpha, void* const* peer_staging, void* barrier_scratch, void* stream) {
    return kshard_fused_run(bq::BQ_KIND_S8, rank, world, comm, m, n, k_local, a_local, lda, b_local, ldb, peer_y, ldy, scale_a,
                            scale_b, BARACUDA_Q_SCALE_PER_ROW_COL, bias, alpha, peer_staging, barrier_scratch, stream);
}

int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_run(
    int32_t rank, int32_t world, void* comm, int32_t m, int32_t n, int32_t k_local, const void* a_local, int64_t lda,
    const void* b_local, int64_t ldb, void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    int32_t scale_mode, const void* bias, float alpha, void* const* peer_staging, void* barrier_scratch, void* stream) {
    return kshard_fused_run(bq::BQ_KIND_E4M3, rank, world, comm, m, n, k_local, a_local, lda, b_local, ldb, peer_y, ldy,
                            scale_a, scale_b, scale_mode, bias, alpha, peer_staging, barrier_scratch, stream);
}

int32_t baracuda_kernels_gemm_w8a8_s8_rcr_bf16_sm100a_kshard_fused_flags_run(
    int32_t rank, int32_t world, int32_t m, int32_t n, int32_t k_local, const void* a_local, int64_t lda,
    const void* b_local, int64_t ldb, void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    const void* bias, float alpha, void* const* peer_staging, void* const* peer_flags, void* stream) {
    if (!peer_flags) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    return kshard_fused_run(bq::BQ_KIND_S8, rank, world, nullptr, m, n, k_local, a_local, lda, b_local, ldb, peer_y, ldy,
                            scale_a, scale_b, BARACUDA_Q_SCALE_PER_ROW_COL, bias, alpha, peer_staging, nullptr, stream,
                            peer_flags);
}

int32_t baracuda_kernels_gemm_fp8_e4m3_rcr_bf16_sm100a_kshard_fused_flags_run(
    int32_t rank, int32_t world, int32_t m, int32_t n, int32_t k_local, const void* a_local, int64_t lda,
    const void* b_local, int64_t ldb, void* const* peer_y, int64_t ldy, const void* scale_a, const void* scale_b,
    int32_t scale_mode, const void* bias, float alpha, void* const* peer_staging, void* const* peer_flags, void* stream) {
    if (!peer_flags) return BARACUDA_Q_STATUS_INVALID_PROBLEM;
    return kshard_fused_run(bq::BQ_KIND_E4M3, rank, world, nullptr, m, n, k_local, a_local, lda, b_local, ldb, peer_y, ldy,
                            scale_a, scale_b, scale_mode, bias, alpha, peer_staging, nullptr, stream, peer_flags);
}

int32_t baracuda_q_peer_barrier_run(void* const* peer_flags, int32_t rank, int32_t world, int64_t limit_cycles, void* stream) {
    return bq::launch_peer_flag_barrier(peer_flags, rank, world, static_cast<long long>(limit_cycles),
                                        static_cast<cudaStream_t>(stream));
}

size_t baracuda_q_peer_barrier_flag_bytes(void) { return 128; }

}  // extern "C"
