// 8-bit tensor-core GEMM on CTA pairs with a 256 x 512 output tile per pair.
//
// The CTA-pair kernel of gemm_q8_pair_sm100a.cu is fed through L2: per K step of 128 bytes each CTA
// loads 128 rows of A plus half of the tile's weight rows, i.e. 1/128 byte per MAC at a 256-wide
// tile.  Doubling the tile width to 512 columns cuts that to 1/171 byte per MAC.  The price is TMEM:
// a CTA's 128 x 512 accumulator fills all 512 columns, so there is no second accumulator to overlap
// the epilogue with.  Instead the tile is treated as two 256-column halves with their own
// "accumulator ready" / "accumulator drained" barriers; the epilogue drains half 0 then half 1, and
// the MMA thread starts the next tile on half 0 (for as many K steps as the ring holds) while half 1
// is still being drained.
//
// Per K step the leader issues, for each 32-byte K slice, two tcgen05.mma.cta_group::2 of 256 x 256:
// half h reads weight rows [h*128, h*128+128) of both CTAs' stage, so CTA c loads the global weight
// rows n0 + h*256 + c*128 + [0,128) into that region.  Roles, bounded waits, status word and the
// C symbols served are those of the other two GEMM kernels.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_q8_common.cuh"
#include "launch.h"
#include "ptx_sm100a.cuh"

namespace bq {

__device__ int g_gemm_wide_device_status = 0;

namespace {

constexpr int W_TILE_M = 256;
constexpr int W_TILE_N = 512;
constexpr int W_HALF_N = 256;
constexpr int W_CTA_ROWS = 128;
constexpr int W_BLOCK_K = 128;
constexpr int W_UMMA_K = 32;
constexpr int W_STAGES = 4;
constexpr int W_THREADS = 192;
constexpr int W_A_BYTES = W_CTA_ROWS * W_BLOCK_K;        // 16 KiB
constexpr int W_BH_BYTES = W_CTA_ROWS * W_BLOCK_K;       // one half's weight rows held by this CTA, 16 KiB
constexpr int W_STAGE_BYTES = W_A_BYTES + 2 * W_BH_BYTES;  // 48 KiB
constexpr int W_TILE_BYTES = W_STAGES * W_STAGE_BYTES;
constexpr int W_STG_BYTES = 4 * 4096;  // per epilogue warp: 32 rows x 128 bytes of output staging
constexpr int W_SB_BYTES = W_STG_BYTES + 2 * 4 * W_TILE_N * 4;  // column scales and bias, one private copy per epilogue warp
constexpr int W_BAR_BYTES = (2 * W_STAGES + 4) * 8 + 16;
constexpr int W_SMEM_TOTAL = W_TILE_BYTES + W_SB_BYTES + W_BAR_BYTES + 1024;
constexpr int W_TMEM_COLS = 512;
constexpr int W_SKEW = W_STAGES - 1;  // K steps of half 0 issued ahead of half 1 at the start of a tile
constexpr long long W_WAIT_LIMIT = 1LL << 31;

__device__ __forceinline__ void wide_timeout(volatile uint32_t* abort_word, int code) {
    *abort_word = 1u;
    atomicCAS(&g_gemm_wide_device_status, 0, code);
}

template <uint32_t KIND, bool RAW, bool FUSED>
__global__ void __launch_bounds__(W_THREADS, 1)
gemm_q8_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // round up inside the shared window (an offset added to the shared array keeps shared-memory addressing)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* tiles = smem;
    uint4* stage_all = reinterpret_cast<uint4*>(smem + W_TILE_BYTES);
    float* sb_s = reinterpret_cast<float*>(smem + W_TILE_BYTES + W_STG_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + W_TILE_BYTES + W_SB_BYTES);
    uint64_t* empty_bar = full_bar + W_STAGES;
    uint64_t* tfull_bar = empty_bar + W_STAGES;  // [half]
    uint64_t* tempty_bar = tfull_bar + 2;        // [half], the leader's copies are used
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < W_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(&tfull_bar[h], 1);
            mbar_init(&tempty_bar[h], 8);  // one arrival per epilogue warp of both CTAs
        }
        *abort_word = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, W_TMEM_COLS);
        tmem_relinquish_alloc_permit_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = (p.k + W_BLOCK_K - 1) / W_BLOCK_K;
    const int total_tiles = p.m_tiles * p.n_tiles;  // 256 x 512 tiles

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs) {
                const int m_blk = tile % p.m_tiles;
                const int n_blk = tile / p.m_tiles;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_word, W_WAIT_LIMIT)) {
                        wide_timeout(abort_word, 121);
                        ok = false;
                        break;
                    }
                    uint8_t* a_tile = tiles + stage * W_STAGE_BYTES;
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * W_STAGE_BYTES);
                    const uint32_t full_on_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
                    const int r = static_cast<int>(rank);
                    tma_load_2d_pair(a_tile, &tmap_a, full_on_leader, kb * W_BLOCK_K, m_blk * W_TILE_M + r * W_CTA_ROWS);
                    tma_load_2d_pair(a_tile + W_A_BYTES, &tmap_b, full_on_leader, kb * W_BLOCK_K,
                                     n_blk * W_TILE_N + r * W_CTA_ROWS);
                    tma_load_2d_pair(a_tile + W_A_BYTES + W_BH_BYTES, &tmap_b, full_on_leader, kb * W_BLOCK_K,
                                     n_blk * W_TILE_N + W_HALF_N + r * W_CTA_ROWS);
                    if (++stage == W_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc(KIND, W_TILE_M, W_HALF_N);
            // global K-step counter -> ring slot and phase
            long long step_base = 0;  // K steps issued by earlier tiles
            bool ok = true;
            int it = 0;
            auto wait_full = [&](long long gstep) -> bool {
                const int stage = static_cast<int>(gstep % W_STAGES);
                const uint32_t phase = static_cast<uint32_t>((gstep / W_STAGES) & 1);
                if (!mbar_wait_bounded(&full_bar[stage], phase, abort_word, W_WAIT_LIMIT)) {
                    wide_timeout(abort_word, 123);
                    return false;
                }
                tc_fence_after_sync();
                return true;
            };
            auto issue_half = [&](long long gstep, int kb, int h) {
                const int stage = static_cast<int>(gstep % W_STAGES);
                const uint32_t a_addr = smem_u32(tiles + stage * W_STAGE_BYTES);
                const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
                const uint64_t b_desc = umma_desc_kmajor_sw128(a_addr + W_A_BYTES + h * W_BH_BYTES);
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(h * W_HALF_N);
#pragma unroll
                for (int ks = 0; ks < W_BLOCK_K / W_UMMA_K; ++ks) {
                    const uint64_t koff = static_cast<uint64_t>((ks * W_UMMA_K) >> 4);
                    umma_ss_pair<KIND>(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | ks) != 0 ? 1u : 0u);
                }
            };
            for (int tile = pair_id; ok && tile < total_tiles; tile += num_pairs, ++it) {
                const uint32_t acc_phase = it & 1;  // each half is used once per tile
                const int skew = num_kb < W_SKEW ? num_kb : W_SKEW;
                // half 0 runs ahead while the epilogue still drains half 1 of the previous tile
                if (!mbar_wait_bounded(&tempty_bar[0], acc_phase ^ 1u, abort_word, W_WAIT_LIMIT)) {
                    wide_timeout(abort_word, 122);
                    break;
                }
                tc_fence_after_sync();
                for (int kb = 0; kb < skew && ok; ++kb) {
                    ok = wait_full(step_base + kb);
                    if (ok) issue_half(step_base + kb, kb, 0);
                }
                if (!ok) break;
                if (!mbar_wait_bounded(&tempty_bar[1], acc_phase ^ 1u, abort_word, W_WAIT_LIMIT)) {
                    wide_timeout(abort_word, 124);
                    break;
                }
                tc_fence_after_sync();
                for (int kb = 0; kb < skew; ++kb) {
                    issue_half(step_base + kb, kb, 1);
                    umma_commit_pair(&empty_bar[(step_base + kb) % W_STAGES], 0x3);  // both halves have read it
                }
                for (int kb = skew; kb < num_kb && ok; ++kb) {
                    ok = wait_full(step_base + kb);
                    if (!ok) break;
                    issue_half(step_base + kb, kb, 0);
                    if (kb == num_kb - 1) umma_commit_pair(&tfull_bar[0], 0x3);  // half 0 complete
                    issue_half(step_base + kb, kb, 1);
                    umma_commit_pair(&empty_bar[(step_base + kb) % W_STAGES], 0x3);
                }
                if (!ok) break;
                if (num_kb <= skew) umma_commit_pair(&tfull_bar[0], 0x3);
                umma_commit_pair(&tfull_bar[1], 0x3);
                step_base += num_kb;
            }
        }
    } else {
        const int q = warp & 3;
        uint4* stage_buf = stage_all + (warp - 2) * 256;
        int it = 0;
        for (int tile = pair_id; tile < total_tiles; tile += num_pairs, ++it) {
            const uint32_t acc_phase = it & 1;
            const int m_blk = tile % p.m_tiles;
            const int n_blk = tile / p.m_tiles;
            float* sb_tile = sb_s + (warp - 2) * W_TILE_N;
            if (!RAW && (!p.out_q8 || p.bias_kind != 0)) {
                __syncwarp();
                for (int i = lane; i < W_TILE_N; i += 32) {
                    const int col = n_blk * W_TILE_N + i;
                    if (!p.out_q8) sb_tile[i] = (p.scale_mode == 1) ? (col < p.n ? __ldg(p.sb + col) : 0.0f) : __ldg(p.sb);
                    if (p.bias_kind == 1) {
                        sb_tile[p.bias_off + i] = col < p.n ? __ldg(reinterpret_cast<const float*>(p.bias) + col) : 0.0f;
                    } else if (p.bias_kind == 2) {
                        sb_tile[p.bias_off + i] =
                            col < p.n ? static_cast<float>(__ldg(reinterpret_cast<const int32_t*>(p.bias) + col)) : 0.0f;
                    }
                }
                __syncwarp();
            }
            const int row = m_blk * W_TILE_M + static_cast<int>(rank) * W_CTA_ROWS + q * 32 + lane;
            const bool row_ok = row < p.m;
            float sa_row = 1.0f;
            if (!RAW && !p.out_q8) {
                sa_row = (p.scale_mode == 1) ? (row_ok ? __ldg(p.sa + row) : 0.0f) : __ldg(p.sa);
            }
            bool ok = true;
            for (int h = 0; h < 2; ++h) {
                if (!mbar_wait_bounded(&tfull_bar[h], acc_phase, abort_word, W_WAIT_LIMIT)) {
                    wide_timeout(abort_word, 125);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                       static_cast<uint32_t>(h * W_HALF_N);
                {
                    int c = 0;
                    if constexpr (!RAW) {
                        for (; c + 2 <= W_HALF_N / 32; c += 2) {
                            const int col0 = n_blk * W_TILE_N + h * W_HALF_N + c * 32;
                            if (col0 >= p.n) break;  // warp-uniform
                            if (!block_64_ok<FUSED>(p, col0)) break;
                            epilogue_block_64<KIND, FUSED>(p, t_row + static_cast<uint32_t>(c * 32),
                                                           m_blk * W_TILE_M + static_cast<int>(rank) * W_CTA_ROWS + q * 32, lane,
                                                           col0, sa_row, sb_tile + h * W_HALF_N + c * 32, stage_buf);
                        }
                    }
#pragma unroll 1
                    for (; c < W_HALF_N / 32; ++c) {
                        const int col0 = n_blk * W_TILE_N + h * W_HALF_N + c * 32;
                        if (col0 >= p.n) break;  // warp-uniform
                        uint32_t r[32];
                        __syncwarp();
                        tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c * 32), r);
                        tmem_ld_wait();
                        if (row_ok) {
                            epilogue_store_32<KIND, RAW, FUSED>(p, row, col0, r, sa_row, sb_tile + h * W_HALF_N + c * 32);
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[h]), 0));
            }
            if (!ok) break;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, W_TMEM_COLS);
    }
}

template <uint32_t KIND, bool RAW, bool FUSED>
int32_t launch_wide(const GemmDesc& g, cudaStream_t stream) {
    const int sms = sm_count_of_current_device();
    if (sms < 2) return BQ_STATUS_LAUNCH_FAILURE;
    CUtensorMap map_a, map_b;
    if (!make_kmajor_tensor_map(&map_a, g.a, g.m, g.k, g.lda, W_CTA_ROWS)) return BQ_STATUS_LAUNCH_FAILURE;
    if (!make_kmajor_tensor_map(&map_b, g.b, g.n, g.k, g.ldb, W_CTA_ROWS)) return BQ_STATUS_LAUNCH_FAILURE;
    GemmParams p;
    p.d = g.d;
    p.ldd = g.ldd;
    p.sa = g.scale_a;
    p.sb = g.scale_b;
    p.scale_mode = g.scale_mode;
    p.alpha = g.alpha;
    p.m = g.m;
    p.n = g.n;
    p.k = g.k;
    p.m_tiles = (g.m + W_TILE_M - 1) / W_TILE_M;
    p.n_tiles = (g.n + W_TILE_N - 1) / W_TILE_N;
    const int64_t elem = RAW ? 4 : (g.q8_out ? 1 : 2);
    p.out_q8 = RAW ? 0 : g.q8_out;
    p.c = g.c;
    p.ldc = g.ldc;
    p.beta = g.beta;
    p.bias = g.bias;
    p.bias_kind = g.bias ? g.bias_kind : 0;
    p.act = g.act;
    p.bias_off = 4 * W_TILE_N;
    p.vec_store = ((reinterpret_cast<uintptr_t>(g.d) & 15u) == 0 && ((g.ldd * elem) & 15) == 0) ? 1 : 0;
    p.n_peers = FUSED ? g.n_peers : 0;
    p.peer_ld = g.peer_ld;
    p.peer_col0 = g.peer_col0;
    p.peer_rank = g.peer_rank;
    p.rs_world = RAW ? g.rs_world : 0;
    p.swiglu = 0;
    p.rs_rows = g.rs_rows;
    p.peer_vec = ((g.peer_ld * 2) & 15) == 0 && ((static_cast<int64_t>(g.peer_col0) * 2) & 15) == 0;
    for (int r = 0; r < 8; ++r) {
        p.peer_d[r] = g.peer_d[r];
        if (r < p.n_peers && (reinterpret_cast<uintptr_t>(g.peer_d[r]) & 15u) != 0) p.peer_vec = 0;
    }
    auto kern = gemm_q8_wide_kernel<KIND, RAW, FUSED>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_TOTAL) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    p.coalesce = g.direct_stores == 1 ? 0 : 1;  // the epilogue of this kernel is partly exposed: staged stores win
    if (p.out_q8) p.coalesce = 0;  // the staging path is bf16-only
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    cfg.blockDim = dim3(W_THREADS, 1, 1);
    cfg.dynamicSmemBytes = W_SMEM_TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, map_a, map_b, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

}  // namespace

int32_t launch_gemm_q8_wide(const GemmDesc& g, cudaStream_t stream) {
    const bool fused = g.n_peers > 0 && !g.raw_out;
    if (g.kind == BQ_KIND_S8) {
        if (g.raw_out) return launch_wide<UMMA_KIND_I8, true, false>(g, stream);
        return fused ? launch_wide<UMMA_KIND_I8, false, true>(g, stream) : launch_wide<UMMA_KIND_I8, false, false>(g, stream);
    }
    if (g.raw_out) return launch_wide<UMMA_KIND_F8, true, false>(g, stream);
    return fused ? launch_wide<UMMA_KIND_F8, false, true>(g, stream) : launch_wide<UMMA_KIND_F8, false, false>(g, stream);
}

int32_t read_and_clear_gemm_wide_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_wide_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_gemm_wide_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
