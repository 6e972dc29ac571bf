// Split-K form of the 8-bit tensor-core GEMM for problems whose output tiles leave SMs idle (small batches against one
// layer's weight; prefill at M = 512 against 4096 columns): a thread-block cluster of S CTAs shares one 128 x BN output
// tile (S = 2 or 4 with BN = 128 -- either weight layout --, S = 2 with BN = 256), CTA s multiplies K slice s, and the partial sums
// meet through distributed shared memory -- no scratch in global memory, no second launch.
//
// Per CTA (six warps, the roles of gemm_q8_kernel): warp 0 streams its slice's A and B tiles through a ring of
// shared-memory stages by TMA, warp 1 issues tcgen05.mma into one TMEM accumulator, warps 2-5 (thread = output row)
// wait for the accumulator.  Then the exchange: the tile's BN columns are cut into S strips, CTA j owns strip j;
// every CTA stores its partial sums of the strips it does not own into the owners' shared memory (16-byte
// st.shared::cluster, laid out so that a warp writes 512 contiguous bytes), the cluster meets again, and every CTA adds what it received
// to its own strip, still in TMEM (int32 adds; f32 adds in slice order), applies the fused epilogue of the one-pass
// kernel (epilogue_store_32: scales, alpha, beta * C, bias, activation, bf16 or 8-bit output) and stores 128 rows x
// BN / S columns.  (The receive buffer is a region of its own for 128-wide tiles; for 256-wide tiles it reuses the operand
// ring, after one more meeting of the cluster that tells every main loop is over.)  Every mbarrier wait is bounded; a wait that runs out records a status word, and the CTA still
// walks to both cluster barriers so that its partners are released.
//
// Replaces, for these shapes, the same reference kernels as gemm_q8_sm100a.cu
//   crates/baracuda-cutlass-kernels-sys/kernels/gemm_s8_rcr_sm80.cu:48-198
//   crates/baracuda-kernels-sys/kernels/include/baracuda_fp8_rcr_sm89.cuh:102-323

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_q8_common.cuh"
#include "launch.h"
#include "ptx_sm100a.cuh"

namespace bq {

__device__ int g_gemm_splitk_device_status = 0;

namespace {

constexpr int SK_BLOCK_M = 128;
constexpr int SK_BLOCK_K = 128;  // bytes of K per stage == one 128-byte swizzle row
constexpr int SK_UMMA_K = 32;
constexpr int SK_THREADS = 192;
constexpr long long SK_WAIT_LIMIT = 1LL << 31;  // about a second

template <int S, int BN>
struct SkSmem {
    // 128-wide tiles: five stages and a receive buffer of its own, so the exchange needs one meeting after the main
    // loop; 256-wide tiles: four stages fill the shared memory, the receive buffer reuses the ring, which takes a
    // second meeting (every main loop over) before the first remote store
    static constexpr bool RECV_IN_RING = BN != 128;
    static constexpr int STAGES = BN == 128 ? 5 : 4;
    static constexpr int A_BYTES = SK_BLOCK_M * SK_BLOCK_K;
    static constexpr int B_BYTES = BN * SK_BLOCK_K;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int STRIP = BN / S;                         // columns a CTA owns
    static constexpr int SRC_WORDS = SK_BLOCK_M * STRIP;         // one partner's partial sums of that strip
    static constexpr int RECV_BYTES = (S - 1) * SRC_WORDS * 4;
    static constexpr int RECV_OFFSET = RECV_IN_RING ? 0 : TILE_BYTES;
    static constexpr int SB_OFFSET = TILE_BYTES + (RECV_IN_RING ? 0 : RECV_BYTES);
    static constexpr int SB_BYTES = 2 * 4 * BN * 4;              // column scales and bias, one private copy per epilogue warp
    static constexpr int BAR_BYTES = (2 * STAGES + 1) * 8 + 16;
    static constexpr int TOTAL = SB_OFFSET + SB_BYTES + BAR_BYTES + 1024;  // + alignment slack
    static_assert(RECV_BYTES <= TILE_BYTES, "the receive buffer fits the operand ring");
    static_assert(STRIP % 32 == 0, "the epilogue works on 32-column blocks");
};

__device__ __forceinline__ void sk_timeout(volatile uint32_t* abort_word, int code) {
    *abort_word = 1u;
    atomicCAS(&g_gemm_splitk_device_status, 0, code);
}

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

// B_MN: the weight is row-major [K, N] (N contiguous): its tile is loaded as [128 K-rows x 128 N-bytes] and described to
// the MMA as an MN-major operand (128-wide tiles only: one 128-byte swizzle atom of N).
template <uint32_t KIND, int S, int BN, bool B_MN = false>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_q8_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const GemmParams p) {
    using L = SkSmem<S, BN>;
    constexpr int STAGES = L::STAGES;
    static_assert(!B_MN || BN == 128, "row-major weights: one swizzle atom of N per tile");
    extern __shared__ uint8_t sk_smem_raw[];
    // every CTA of the cluster rounds up by the same amount (same kernel, same static layout), so an offset into this
    // CTA's window is the same offset in a partner's
    uint8_t* smem = sk_smem_raw + ((1024u - (smem_u32(sk_smem_raw) & 1023u)) & 1023u);
    uint8_t* tiles = smem;
    uint32_t* recv = reinterpret_cast<uint32_t*>(smem + L::RECV_OFFSET);
    float* sb_s = reinterpret_cast<float*>(smem + L::SB_OFFSET);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::SB_OFFSET + L::SB_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int slice = static_cast<int>(cluster_ctarank());
    const int tile = static_cast<int>(blockIdx.x) / S;  // clusters are consecutive groups of S CTAs along x
    const int m_blk = tile % p.m_tiles;
    const int n_blk = tile / p.m_tiles;
    const int num_kb = (p.k + SK_BLOCK_K - 1) / SK_BLOCK_K;
    const int kb0 = slice * p.kb_per_slice;
    int nk = num_kb - kb0;
    if (nk > p.kb_per_slice) nk = p.kb_per_slice;
    if (nk < 0) nk = 0;  // an empty slice contributes zeros (the host sizes the slices so that none is empty)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_word = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // own receive buffer: every CTA of the cluster is running (its shared memory live) before anyone may store into it
    if constexpr (!L::RECV_IN_RING) cluster_sync_all();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    float sa_row = 1.0f;
    const int q = warp & 3;  // TMEM lane quarter an epilogue warp may read
    const int row_local = q * 32 + lane;
    const int row = m_blk * SK_BLOCK_M + row_local;
    float* sb_tile = sb_s + (warp >= 2 ? warp - 2 : 0) * BN;
    bool have = false;  // epilogue threads: the accumulator is complete

    if (warp == 0) {
        if (lane == 0) {
            int first = 0;
            if (p.pdl) {
                // dependent launch: the first ring of (static) weight tiles is requested while the previous kernel of
                // the stream is still finishing; the activations follow once it has completed
                first = nk < STAGES ? nk : STAGES;
                for (int i = 0; i < first; ++i) {
                    mbar_arrive_expect_tx(&full_bar[i], L::STAGE_BYTES);
                    if constexpr (B_MN) {
                        tma_load_2d(tiles + i * L::STAGE_BYTES + L::A_BYTES, &tmap_b, &full_bar[i], n_blk * BN, (kb0 + i) * SK_BLOCK_K);
                    } else {
                        tma_load_2d(tiles + i * L::STAGE_BYTES + L::A_BYTES, &tmap_b, &full_bar[i], (kb0 + i) * SK_BLOCK_K,
                                    n_blk * BN);
                    }
                }
                asm volatile("griddepcontrol.wait;" ::: "memory");
                for (int i = 0; i < first; ++i) {
                    tma_load_2d(tiles + i * L::STAGE_BYTES, &tmap_a, &full_bar[i], (kb0 + i) * SK_BLOCK_K, m_blk * SK_BLOCK_M);
                }
            }
            for (int i = first; i < nk; ++i) {
                const int stage = i % STAGES;
                const uint32_t phase = static_cast<uint32_t>(i / STAGES) & 1u;
                if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_word, SK_WAIT_LIMIT)) {
                    sk_timeout(abort_word, 121);
                    break;
                }
                uint8_t* st = tiles + stage * L::STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
                tma_load_2d(st, &tmap_a, &full_bar[stage], (kb0 + i) * SK_BLOCK_K, m_blk * SK_BLOCK_M);
                if constexpr (B_MN) {
                    tma_load_2d(st + L::A_BYTES, &tmap_b, &full_bar[stage], n_blk * BN, (kb0 + i) * SK_BLOCK_K);
                } else {
                    tma_load_2d(st + L::A_BYTES, &tmap_b, &full_bar[stage], (kb0 + i) * SK_BLOCK_K, n_blk * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(KIND, SK_BLOCK_M, BN, B_MN);
            bool ok = true;
            for (int i = 0; i < nk; ++i) {
                const int stage = i % STAGES;
                const uint32_t phase = static_cast<uint32_t>(i / STAGES) & 1u;
                if (!mbar_wait_bounded(&full_bar[stage], phase, abort_word, SK_WAIT_LIMIT)) {
                    sk_timeout(abort_word, 122);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_addr = smem_u32(tiles + stage * L::STAGE_BYTES);
                const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
                const uint64_t b_desc = B_MN ? umma_desc_mnmajor_sw128(a_addr + L::A_BYTES, L::B_BYTES, 1024)
                                             : umma_desc_kmajor_sw128(a_addr + L::A_BYTES);
#pragma unroll
                for (int ks = 0; ks < SK_BLOCK_K / SK_UMMA_K; ++ks) {
                    const uint64_t koff = static_cast<uint64_t>((ks * SK_UMMA_K) >> 4);
                    // MN-major: 32 K-rows are four 1024-byte atoms further down the tile
                    const uint64_t boff = B_MN ? static_cast<uint64_t>((ks * SK_UMMA_K * 128) >> 4) : koff;
                    umma_ss<KIND>(tmem_base, a_desc + koff, b_desc + boff, idesc, (i | ks) != 0 ? 1u : 0u);
                }
                umma_commit(&empty_bar[stage]);
            }
            if (ok && nk > 0) umma_commit(tfull_bar);
        }
    } else {
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // scales, C and D belong to the stream's past
        // this warp's private copy of the tile's column scales and bias (no barrier between the epilogue warps)
        if (!p.out_q8 || p.bias_kind != 0) {
            float sv[BN / 32], bv[BN / 32];
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) {
                const int col = n_blk * BN + j * 32 + lane;
                const bool in = col < p.n;
                sv[j] = 0.0f;
                bv[j] = 0.0f;
                if (!p.out_q8) sv[j] = (p.scale_mode != 0) ? (in ? __ldg(p.sb + col) : 0.0f) : __ldg(p.sb);
                if (p.bias_kind == 1) {
                    if (in) bv[j] = __ldg(reinterpret_cast<const float*>(p.bias) + col);
                } else if (p.bias_kind == 2) {
                    if (in) bv[j] = static_cast<float>(__ldg(reinterpret_cast<const int32_t*>(p.bias) + col));
                }
            }
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) {
                if (!p.out_q8) sb_tile[j * 32 + lane] = sv[j];
                if (p.bias_kind != 0) sb_tile[p.bias_off + j * 32 + lane] = bv[j];
            }
            __syncwarp();
        }
        if (!p.out_q8) {
            sa_row = (p.scale_mode == 1) ? (row < p.m ? __ldg(p.sa + row) : 0.0f) : (p.scale_mode == 2 ? p.sa_const : __ldg(p.sa));
        }
        // the accumulator is complete: every MMA of this CTA has read its stages, every copy into the ring has landed
        have = nk > 0;
        if (have && !mbar_wait_bounded(tfull_bar, 0u, abort_word, SK_WAIT_LIMIT)) {
            sk_timeout(abort_word, 123);
            have = false;
        }
        tc_fence_after_sync();
    }

    // Receive buffer in the ring: every CTA of the cluster has finished its main loop (the epilogue threads arrive after
    // the accumulator barrier), so every ring is free to receive.  Every thread of every CTA comes here, also after
    // a time-out.
    if constexpr (L::RECV_IN_RING) {
        __syncwarp();
        cluster_sync_all();
    }

    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (warp >= 2) {
        // the strips of the partners, nearest partner first so that no CTA is everyone's target at once
#pragma unroll 1
        for (int dj = 1; dj < S; ++dj) {
            const int dst = (slice + dj) % S;
            const int slot = slice < dst ? slice : slice - 1;  // a receive buffer holds the S - 1 partners in rank order
            const uint32_t remote = map_to_cta(smem_u32(recv), static_cast<uint32_t>(dst)) +
                                    static_cast<uint32_t>(slot * L::SRC_WORDS * 4);
#pragma unroll 1
            for (int cb = 0; cb < L::STRIP / 32; ++cb) {
                uint32_t r[32];
                if (have) {
                    __syncwarp();
                    tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(dst * L::STRIP + cb * 32), r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = 0u;
                }
                // four columns per store; group g of the strip's 4-column groups sits at [g][row][4]: a warp writes 512
                // contiguous bytes, and reads them back the same way
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                    st_cluster_v4(remote + static_cast<uint32_t>(((cb * 8 + v) * SK_BLOCK_M + row_local) * 16), r[4 * v],
                                  r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                }
            }
        }
    }

    // All partial sums have been stored (release) and are visible after the wait (acquire).  Every thread of every CTA
    // comes here, also after a time-out.
    __syncwarp();
    cluster_sync_all();

    if (warp >= 2) {
#pragma unroll 1
        for (int cb = 0; cb < L::STRIP / 32; ++cb) {
            uint32_t r[32];
            if (have) {
                __syncwarp();
                tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(slice * L::STRIP + cb * 32), r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) r[c] = 0u;
            }
            const uint4* rv = reinterpret_cast<const uint4*>(recv);
            if constexpr (KIND == UMMA_KIND_I8) {
#pragma unroll
                for (int src = 0; src < S - 1; ++src) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const uint4 x = rv[src * (L::SRC_WORDS / 4) + (cb * 8 + v) * SK_BLOCK_M + row_local];
                        r[4 * v] += x.x;
                        r[4 * v + 1] += x.y;
                        r[4 * v + 2] += x.z;
                        r[4 * v + 3] += x.w;
                    }
                }
            } else {
                // f32: slices added in slice order, this CTA's own sum at its place
                float f[32];
#pragma unroll
                for (int s = 0; s < S; ++s) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        uint4 x = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        if (s != slice) x = rv[(s < slice ? s : s - 1) * (L::SRC_WORDS / 4) + (cb * 8 + v) * SK_BLOCK_M + row_local];
                        const uint32_t bits[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            f[4 * v + e] = (s == 0) ? __uint_as_float(bits[e]) : __fadd_rn(f[4 * v + e], __uint_as_float(bits[e]));
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(f[c]);
            }
            const int local_col = slice * L::STRIP + cb * 32;
            const int col0 = n_blk * BN + local_col;
            if (row < p.m && col0 < p.n && *abort_word == 0u) {
                epilogue_store_32<KIND, false, false>(p, row, col0, r, sa_row, sb_tile + local_col);
            }
        }
    }

    // Teardown.  On the error path give copies and MMAs still in flight a bounded time to land before TMEM goes back.
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, BN);
    }
}

template <uint32_t KIND, int S, int BN, bool B_MN>
int32_t launch_splitk(const GemmDesc& g, int kb_per_slice, cudaStream_t stream, int* max_clusters_out) {
    using L = SkSmem<S, BN>;
    auto kern = gemm_q8_splitk_kernel<KIND, S, BN, B_MN>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    const int m_tiles = (g.m + SK_BLOCK_M - 1) / SK_BLOCK_M;
    const int n_tiles = (g.n + BN - 1) / BN;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(m_tiles * n_tiles * S), 1, 1);
    cfg.blockDim = dim3(SK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (max_clusters_out) {  // how many clusters of this kernel the device holds at once (a host query, no launch)
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        *max_clusters_out = n;
        return BQ_STATUS_OK;
    }
    cfg.numAttrs = g.pdl ? 2 : 1;
    CUtensorMap map_a, map_b;
    if (!make_kmajor_tensor_map(&map_a, g.a, g.m, g.k, g.lda, SK_BLOCK_M)) return BQ_STATUS_LAUNCH_FAILURE;
    if constexpr (B_MN) {
        if (!make_mnmajor_tensor_map(&map_b, g.b, g.k, g.n, g.ldb, SK_BLOCK_K)) return BQ_STATUS_LAUNCH_FAILURE;
    } else {
        if (!make_kmajor_tensor_map(&map_b, g.b, g.n, g.k, g.ldb, BN)) return BQ_STATUS_LAUNCH_FAILURE;
    }
    GemmParams p;
    p.d = g.d;
    p.ldd = g.ldd;
    p.sa = g.scale_a;
    p.sb = g.scale_b;
    p.scale_mode = g.scale_mode;
    p.sa_const = g.sa_const;
    p.alpha = g.alpha;
    p.m = g.m;
    p.n = g.n;
    p.k = g.k;
    p.m_tiles = m_tiles;
    p.n_tiles = n_tiles;
    const int64_t elem = g.q8_out ? 1 : 2;
    p.vec_store = ((reinterpret_cast<uintptr_t>(g.d) & 15u) == 0 && ((g.ldd * elem) & 15) == 0) ? 1 : 0;
    for (auto& pd : p.peer_d) pd = nullptr;
    p.mc_d = nullptr;
    p.n_peers = 0;
    p.peer_ld = 0;
    p.peer_col0 = 0;
    p.peer_vec = 0;
    p.peer_rank = 0;
    p.coalesce = 0;
    p.out_q8 = g.q8_out;
    p.c = g.c;
    p.ldc = g.ldc;
    p.beta = g.beta;
    p.bias = g.bias;
    p.bias_kind = g.bias ? g.bias_kind : 0;
    p.act = g.act;
    p.bias_off = 4 * BN;
    p.rs_world = 0;
    p.rs_rows = 0;
    p.swiglu = 0;
    p.mixed = 0;
    p.mixed_full_cols = 0;
    p.raster_gm = 1;
    p.pdl = g.pdl;
    p.kb_per_slice = kb_per_slice;
    if (cudaLaunchKernelEx(&cfg, kern, map_a, map_b, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

template <int S, int BN, bool B_MN>
int32_t launch_splitk_kind(const GemmDesc& g, int kb_per_slice, cudaStream_t stream, int* max_clusters_out) {
    return g.kind == BQ_KIND_S8 ? launch_splitk<UMMA_KIND_I8, S, BN, B_MN>(g, kb_per_slice, stream, max_clusters_out)
                                : launch_splitk<UMMA_KIND_F8, S, BN, B_MN>(g, kb_per_slice, stream, max_clusters_out);
}

int32_t launch_splitk_shape(const GemmDesc& g, int slices, int block_n, int kb_per_slice, cudaStream_t stream,
                            int* max_clusters_out) {
    const bool mn = g.b_layout == BQ_LAYOUT_RRR;
    if (block_n == 256 && slices == 2 && !mn) return launch_splitk_kind<2, 256, false>(g, kb_per_slice, stream, max_clusters_out);
    if (block_n == 128 && slices == 2) {
        return mn ? launch_splitk_kind<2, 128, true>(g, kb_per_slice, stream, max_clusters_out)
                  : launch_splitk_kind<2, 128, false>(g, kb_per_slice, stream, max_clusters_out);
    }
    if (block_n == 128 && slices == 4) {
        return mn ? launch_splitk_kind<4, 128, true>(g, kb_per_slice, stream, max_clusters_out)
                  : launch_splitk_kind<4, 128, false>(g, kb_per_slice, stream, max_clusters_out);
    }
    return BQ_STATUS_INVALID_PROBLEM;
}

}  // namespace

int32_t launch_gemm_q8_cluster_split_k(const GemmDesc& g, int32_t slices, int32_t block_n, cudaStream_t stream) {
    if (g.raw_out || g.swiglu || g.n_peers > 0 || g.rs_world > 0 || g.k <= 0 ||
        (g.b_layout == BQ_LAYOUT_RRR && block_n != 128)) {
        return BQ_STATUS_INVALID_PROBLEM;
    }
    const int num_kb = (g.k + SK_BLOCK_K - 1) / SK_BLOCK_K;
    if (slices < 2 || num_kb < slices) return BQ_STATUS_INVALID_PROBLEM;
    const int kb_per_slice = (num_kb + slices - 1) / slices;
    if ((num_kb + kb_per_slice - 1) / kb_per_slice != slices) return BQ_STATUS_INVALID_PROBLEM;  // an empty slice
    return launch_splitk_shape(g, slices, block_n, kb_per_slice, stream, nullptr);
}

int gemm_q8_cluster_split_k_max_clusters(int32_t kind, int32_t slices, int32_t block_n) {
    const int shape = (block_n == 128 && slices == 2) ? 0 : (block_n == 128 && slices == 4) ? 1 : (block_n == 256 && slices == 2) ? 2 : -1;
    if (shape < 0) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    static int cache[64][2][3];  // [device][kind][shape]; 0 = not asked yet, -1 = none
    int& c = cache[dev][kind == BQ_KIND_S8 ? 0 : 1][shape];
    if (c == 0) {
        GemmDesc g = {};
        g.kind = kind;
        g.m = SK_BLOCK_M;
        g.n = block_n;
        g.k = SK_BLOCK_K;
        int n = 0;
        (void)launch_splitk_shape(g, slices, block_n, 1, nullptr, &n);
        c = n > 0 ? n : -1;
    }
    return c > 0 ? c : 0;
}

int32_t read_and_clear_gemm_splitk_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_splitk_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_gemm_splitk_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
