// Internal launch descriptors shared by the kernels and the C-ABI file.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace bq {

// Status codes of the flat C symbols; values follow the reference's contract
// (crates/baracuda-kernels-sys/src/lib.rs:19-27).
enum : int32_t {
    BQ_STATUS_OK = 0,
    BQ_STATUS_MISALIGNED = 1,
    BQ_STATUS_INVALID_PROBLEM = 2,
    BQ_STATUS_UNSUPPORTED = 3,
    BQ_STATUS_WORKSPACE = 4,
    BQ_STATUS_LAUNCH_FAILURE = 5
};

enum : int32_t { BQ_KIND_S8 = 0, BQ_KIND_E4M3 = 1 };
enum : int32_t { BQ_LAYOUT_RRR = 0, BQ_LAYOUT_RCR = 1 };

struct GemmDesc {
    int32_t kind;     // BQ_KIND_*
    int32_t raw_out;  // 1: write the 32-bit accumulators, 0: fused dequant -> bf16
    int32_t b_layout; // BQ_LAYOUT_RCR: weight [N,K]; BQ_LAYOUT_RRR: weight row-major [K,N] (CTA-pair kernel, or the cluster split-K kernel for small batches)
    int32_t q8_out;   // 1 (with raw_out 0): d = sat(alpha*acc + beta*C) in the input type (s8 / e4m3), no scales
    const void* c;    // q8_out only
    int64_t ldc;
    float beta;
    const void* bias;   // per-column bias of the fused epilogue, or null
    int32_t bias_kind;  // 0 none, 1 float[N], 2 int32[N]
    int32_t act;        // 0 none, 1 relu, 2 gelu, 3 silu
    int32_t m, n, k;
    const void* a;
    int64_t lda;
    const void* b;
    int64_t ldb;
    const float* scale_a;
    const float* scale_b;
    int32_t scale_mode;  // 0 per-tensor scalars, 1 per-row / per-column vectors, 2 sa_const by value + per-column vector
    float sa_const;
    float alpha;
    void* d;
    int64_t ldd;
    int32_t force_block_n;  // 0 = choose; 64 / 128 / 256 = 1-CTA kernel with that N-tile; 512 = CTA-pair kernel
    int32_t direct_stores;  // 1: epilogue threads store their own rows directly (no staging); tuning
    int32_t epilogue_warps;  // CTA-pair kernel: 0 = choose, 4 or 8 epilogue warps (tuning and tests)
    int32_t force_pair_tile_n;  // 0 = choose; else 256 / 224 / 192 / 128 (tuning and tests)
    // fused replicated output: the epilogue also stores each tile into these row-major
    // [M, peer_ld] buffers (one per rank, peer-mapped) at column offset peer_col0
    void* peer_d[8];
    void* mc_d;       // multicast address of the peers' buffers, or null (used only when every store can be 16 bytes)
    int32_t n_peers;  // 0 = off
    int64_t peer_ld;
    int32_t peer_col0;
    int32_t peer_rank;
    // raw-accumulator reduce-scatter (raw_out only): row r goes to peer_d[r / rs_rows], slot peer_rank; 0 = off
    int32_t rs_world;
    int32_t rs_rows;
    // gated-MLP epilogue (bf16 output, weights [N,K] only): n = 2F interleaved gate/up rows in blocks of 32, d is [M, F]
    int32_t swiglu;
    int32_t pdl;  // 1: launch with programmatic stream serialization (the caller promises the previous kernel does not write b)
    int32_t cluster_split_k;  // split-K inside a thread-block cluster: 0 = choose, 1 = never, 2 / 4 = that many slices of 128-wide tiles, 256 = two slices of 256-wide tiles
};

// Split-K without scratch: clusters of `slices` CTAs share a 128 x block_n tile and add their partial sums through
// distributed shared memory (gemm_q8_splitk_sm100a.cu); (slices, block_n) is (2, 128), (4, 128) or (2, 256).  bf16 or
// 8-bit output, [N,K] weights, any M and N; every slice needs at least one K block.
int32_t launch_gemm_q8_cluster_split_k(const GemmDesc& g, int32_t slices, int32_t block_n, cudaStream_t stream);
// Clusters of that kernel the current device holds at once (0: cannot run); cached per device.
int gemm_q8_cluster_split_k_max_clusters(int32_t kind, int32_t slices, int32_t block_n);
int32_t read_and_clear_gemm_splitk_device_status();
// True when launch_gemm_q8 would run this problem on the cluster split-K kernel.
bool gemm_q8_takes_cluster_split_k(const GemmDesc& g);

int32_t launch_gemm_q8(const GemmDesc& g, cudaStream_t stream);
// Raw-accumulator GEMM of a K shard whose epilogue scatters the [m, n] partial sums by row block: rows
// [j * m / world, (j + 1) * m / world) go to rank j's staging buffer staging[j] ([world][m / world][n] 32-bit words,
// peer-mapped), slot `rank`.  m must divide by world.
int32_t launch_gemm_raw_reduce_scatter_checked(int32_t kind, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                                               const void* b, int64_t ldb, void* const* staging, int32_t world,
                                               int32_t rank, cudaStream_t stream);
// Second half of the fused K-sharded forward on the owner of a row block: adds the `world` slots of `staging_local`,
// applies scales / alpha / bias like launch_dequant_rows and stores the bf16 rows into every rank's y[q] (row pitch ldy).
int32_t launch_reduce_dequant_broadcast(int32_t kind, int32_t rank, int32_t world, int32_t rows, int32_t n,
                                        const void* staging_local, const float* scale_a, const float* scale_b,
                                        int32_t scale_mode, float alpha, const float* bias, void* const* y, int64_t ldy,
                                        cudaStream_t stream);
// Validates like the flat *_run symbols, then launches the bf16-out GEMM; with `peer_d` the epilogue
// additionally stores into the `world` peer buffers at column offset rank * n.
// `layout` is the weight storage (BQ_LAYOUT_RCR: [N,K] rows, BQ_LAYOUT_RRR: row-major [K,N], ldb >= the full N).
int32_t launch_gemm_bf16_checked(int32_t layout, int32_t kind, int32_t m, int32_t n, int32_t k, const void* a, int64_t lda,
                                const void* b, int64_t ldb, void* d, int64_t ldd, const void* scale_a,
                                const void* scale_b, int32_t scale_mode, float alpha, void* const* peer_d,
                                int32_t world, int32_t rank, int64_t peer_ld, cudaStream_t stream, void* mc_d = nullptr);
int32_t read_and_clear_gemm_device_status();
// CTA-pair (cta_group::2) variant: 256 x 256 output tiles shared by two SMs.
int32_t launch_gemm_q8_pair(const GemmDesc& g, cudaStream_t stream);
int32_t read_and_clear_gemm_pair_device_status();
// helpers exported by the 1-CTA GEMM file
bool make_kmajor_tensor_map(void* map_out, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows);
// [k_rows x n_cols] bytes, N contiguous, row pitch ld; box = box_k rows x 128 bytes, 128-byte swizzle
// l2_promotion: CUtensorMapL2promotion value (0 none, 1 64 B, 2 128 B, 3 256 B)
bool make_mnmajor_tensor_map(void* map_out, const void* base, int64_t k_rows, int64_t n_cols, int64_t ld, int box_k,
                             int l2_promotion = 3);
int sm_count_of_current_device();
// D = bf16((sa*sb) * acc * alpha (+ bias)) for an [m, n] matrix of int32 (BQ_KIND_S8) or f32 (BQ_KIND_E4M3) accumulators.
// Interleaves gate and up rows in blocks of 32 (the operand layout of GemmDesc::swiglu): rows of `row_bytes` bytes.
int32_t launch_interleave_gate_up(int64_t f_rows, int64_t row_bytes, const void* gate, int64_t gate_pitch, const void* up,
                                  int64_t up_pitch, void* out, int64_t out_pitch, cudaStream_t stream);
int32_t launch_dequant_rows(int32_t kind, int32_t m, int32_t n, const void* acc, int64_t ld_acc, const float* scale_a,
                            const float* scale_b, int32_t scale_mode, float alpha, const float* bias, void* d, int64_t ldd,
                            cudaStream_t stream);

struct GemvDesc {
    int32_t raw_out;  // 1: int32 accumulators, 0: bf16
    int32_t m, n, k, batch;
    int32_t layout;  // BQ_LAYOUT_*
    float alpha, beta;
    const int8_t* a;
    int64_t lda, stride_a;
    const int8_t* b;
    int64_t ldb, stride_b;
    const float* scale_a;
    int64_t stride_scale_a;
    const float* scale_b;
    int64_t stride_scale_b;
    void* d;
    int64_t ldd, stride_d;
    void* workspace;
    size_t workspace_bytes;
    int32_t variant;  // 0 = choose (tuning and tests)
    int32_t pdl;      // 1: launch the streaming kernel with programmatic stream serialization
};

// One-block barrier kernel between the ranks of a box over peer-mapped flag buffers (32 zero-initialised words per rank).
int32_t launch_peer_flag_barrier(void* const* peer_flags, int32_t rank, int32_t world, long long limit_cycles,
                                 cudaStream_t stream);
int32_t read_and_clear_peer_barrier_device_status();
int32_t launch_gemv_q8(const GemvDesc& g, cudaStream_t stream);
int32_t read_and_clear_gemv_device_status();
// Launches one thread that waits on a barrier nothing completes; the wait gives up after limit_cycles and sets status 299.
int32_t launch_bounded_wait_selftest(long long limit_cycles, cudaStream_t stream);
size_t gemv_q8_workspace_bytes(int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout);
// Decode GEMV with the per-token quantiser inside: bf16 activations in, K-contiguous int8 weights, bf16 out.
bool gemv_q8_quant_bf16_supported(int32_t m, int32_t n, int32_t k);
int32_t launch_gemv_q8_quant_bf16(int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax, float alpha, float beta,
                                  const void* x_bf16, int64_t ldx, const int8_t* b, int64_t ldb, const float* scale_b,
                                  float* scale_a_out, void* d, int64_t ldd, int32_t pdl, cudaStream_t stream);

}  // namespace bq
