// 8-bit tensor-core GEMM on CTA pairs (tcgen05 cta_group::2): two SMs of a
// 2-CTA cluster share every MMA and together own a 256 x 256 output tile.
// Each CTA streams its own 128 rows of A and its own 128 rows of the weight
// tile (no operand is loaded twice, no multicast is involved), the leader CTA
// issues 256 x 256 x 32 MMAs that read both CTAs' shared memory, and each CTA
// keeps its 128 accumulator rows in its own TMEM.  Compared with the 1-CTA
// kernel this halves the shared-memory and L2 traffic of the weight operand
// per MAC and leaves room for a deeper TMA ring (6 stages of 32 KiB per CTA).
//
// Same roles per CTA as the 1-CTA kernel (warp 0 TMA producer, warp 1 TMEM
// owner / MMA issuer on the leader, warps 2-5 epilogue), same double-buffered
// accumulator, same bounded waits.  Serves the same C symbols; replaces the
// same reference kernels as gemm_q8_sm100a.cu.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_q8_common.cuh"
#include "launch.h"
#include "ptx_sm100a.cuh"

namespace bq {

__device__ int g_gemm_pair_device_status = 0;

namespace {

constexpr int PAIR_TILE_M = 256;   // rows per CTA pair
// columns per CTA pair: template parameter TN (256, 224, 192 or 128; any multiple of 32 works for the MMA)
constexpr int CTA_ROWS = 128;      // A rows and weight rows each CTA loads
constexpr int PAIR_BLOCK_K = 128;  // bytes of K per stage
constexpr int PAIR_UMMA_K = 32;
constexpr int PAIR_THREADS = 192;
constexpr int PAIR_A_BYTES = CTA_ROWS * PAIR_BLOCK_K;
constexpr long long PAIR_WAIT_LIMIT = 1LL << 31;

template <int TN>
struct PairCfg {
    static constexpr int B_ROWS = TN / 2;  // weight rows each CTA loads
    static constexpr int B_BYTES = B_ROWS * PAIR_BLOCK_K;
    static constexpr int STAGE_BYTES = PAIR_A_BYTES + B_BYTES;  // a multiple of 1024 for TN % 16 == 0
    static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int STG_BYTES = 4 * 4096;  // per epilogue warp: 32 rows x 128 bytes of output staging
    // Staged column scales, then staged bias: a private slice per epilogue warp.  Four warps hold TN floats each; eight
    // warps hold half of the tile's 32-column blocks each, rounded up (TN = 224: 4 + 3 blocks, 128 floats per slice).
    static constexpr int SB_HALF = ((TN / 32 + 1) / 2) * 32;
    static constexpr int SB_FLOATS = 8 * SB_HALF;  // >= 4 * TN
    static constexpr int SB_BYTES = STG_BYTES + 2 * SB_FLOATS * 4;
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int SMEM_TOTAL = TILE_BYTES + SB_BYTES + BAR_BYTES + 1024;
    static constexpr int TMEM_COLS = (2 * TN <= 256) ? 256 : 512;
};

__device__ __forceinline__ void pair_timeout(volatile uint32_t* abort_word, int code) {
    *abort_word = 1u;
    atomicCAS(&g_gemm_pair_device_status, 0, code);
}

// B_MN: the weight is row-major [K, N] (N contiguous): its tile is loaded as [128 K-rows x 128 N-bytes] and
// described to the MMA as an MN-major operand.  Needs TN == 256 (one 128-byte atom of N per CTA).
// MIXED (TN == 256, K-contiguous weights): the launch follows GemmParams' mixed-width schedule; a 128-wide tile uses
// half of the stage's weight area, the weight map's box is 64 rows (two loads per stage for a wide tile).
// EW8: eight epilogue warps instead of four -- two per tensor-memory lane quadrant, each taking half of the tile's
// column blocks (32 columns at a time through a 2 KiB staging area) -- for epilogue chains whose arithmetic (bias + gelu /
// silu: about 26 instructions per element) four warps cannot hide behind the next tile's MMAs at short K.
template <uint32_t KIND, bool RAW, bool FUSED, int TN, bool B_MN = false, bool MIXED = false, bool EW8 = false>
__global__ void __launch_bounds__(EW8 ? PAIR_THREADS + 128 : PAIR_THREADS, 1)
gemm_q8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
    using C = PairCfg<TN>;
    constexpr int PAIR_TILE_N = TN;
    constexpr int PAIR_STAGES = C::STAGES;
    constexpr int PAIR_STAGE_BYTES = C::STAGE_BYTES;
    constexpr int PAIR_TILE_BYTES = C::TILE_BYTES;
    constexpr int PAIR_SB_BYTES = C::SB_BYTES;
    constexpr int PAIR_TMEM_COLS = C::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    // round up inside the shared window (an offset added to the shared array keeps shared-memory addressing)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* tiles = smem;
    uint4* stage_all = reinterpret_cast<uint4*>(smem + PAIR_TILE_BYTES);
    float* sb_s = reinterpret_cast<float*>(smem + PAIR_TILE_BYTES + C::STG_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + PAIR_TILE_BYTES + PAIR_SB_BYTES);
    uint64_t* empty_bar = full_bar + PAIR_STAGES;
    uint64_t* tfull_bar = empty_bar + PAIR_STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader (issues the MMAs), 1 = partner
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader producer's arrive + both CTAs' TMA bytes
            mbar_init(&empty_bar[s], 1);  // one commit arrival from the leader's MMA thread
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);   // one commit arrival
            mbar_init(&tempty_bar[b], EW8 ? 16 : 8);  // one arrival per epilogue warp of both CTAs (leader's copy is used)
        }
        *abort_word = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, PAIR_TMEM_COLS);
        tmem_relinquish_alloc_permit_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = (p.k + PAIR_BLOCK_K - 1) / PAIR_BLOCK_K;
    const int total_tiles = p.m_tiles * p.n_tiles;  // counted in 256 x TN pair tiles
    // Every role walks the same tile list: body(m_blk, col0, tn, it) returns false to stop.
    auto for_each_tile = [&](auto&& body) {
        int it = 0;
        if constexpr (MIXED) {
            for (int phase = 0; phase < 2; ++phase) {
                const int lo = phase ? p.half_begin[pair_id] : p.full_begin[pair_id];
                const int hi = phase ? p.half_begin[pair_id + 1] : p.full_begin[pair_id + 1];
                for (int tile = lo; tile < hi; ++tile, ++it) {
                    const int nb = tile / p.m_tiles;
                    const int col0 = phase ? p.mixed_full_cols * 256 + nb * 128 : nb * 256;
                    if (!body(tile - nb * p.m_tiles, col0, phase ? 128 : 256, it)) return;
                }
            }
        } else {
            const int group_tiles = p.raster_gm * p.n_tiles;
            for (int tile = pair_id; tile < total_tiles; tile += num_pairs, ++it) {
                const int grp = tile / group_tiles;
                const int within = tile - grp * group_tiles;
                const int m0 = grp * p.raster_gm;
                const int rows = p.m_tiles - m0 < p.raster_gm ? p.m_tiles - m0 : p.raster_gm;
                const int nb = within / rows;
                if (!body(m0 + within - nb * rows, nb * PAIR_TILE_N, PAIR_TILE_N, it)) return;
            }
        }
    };

    // All roles: let the next kernel of the stream be scheduled as soon as SMs free up (it only matters to a kernel
    // that was itself launched as a programmatic dependent).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            // The producer numbers its (tile, K block) steps 0, 1, 2, ...; step i uses ring stage i % STAGES in phase
            // (i / STAGES) & 1.  what: 0 = arm the barrier and load both operands, 1 = arm and load the weights only,
            // 2 = load the activations only (barrier already armed, stage known to be free).
            auto walk = [&](int first, int last, int what) {
                int idx = 0;
                for_each_tile([&](int m_blk, int col0, int tn, int) {
                    for (int kb = 0; kb < num_kb; ++kb, ++idx) {
                        if (idx < first) continue;
                        if (idx >= last) return false;
                        const int stage = idx % PAIR_STAGES;
                        const uint32_t phase = static_cast<uint32_t>(idx / PAIR_STAGES) & 1u;
                        if (what == 0 && !mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_word, PAIR_WAIT_LIMIT)) {
                            pair_timeout(abort_word, 111);
                            return false;
                        }
                        uint8_t* a_tile = tiles + stage * PAIR_STAGE_BYTES;
                        if (rank == 0 && what != 2) {
                            mbar_arrive_expect_tx(&full_bar[stage], 2 * (PAIR_A_BYTES + (tn / 2) * PAIR_BLOCK_K));
                        }
                        // completion bytes of both CTAs' loads are counted on the leader's barrier
                        const uint32_t full_on_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
                        if (what != 1) {
                            tma_load_2d_pair(a_tile, &tmap_a, full_on_leader, kb * PAIR_BLOCK_K,
                                             m_blk * PAIR_TILE_M + static_cast<int>(rank) * CTA_ROWS);
                        }
                        if (what != 2) {
                            if constexpr (B_MN) {
                                tma_load_2d_pair(a_tile + PAIR_A_BYTES, &tmap_b, full_on_leader,
                                                 col0 + static_cast<int>(rank) * C::B_ROWS, kb * PAIR_BLOCK_K);
                            } else if constexpr (MIXED) {
                                const int row0 = col0 + static_cast<int>(rank) * (tn / 2);
                                tma_load_2d_pair(a_tile + PAIR_A_BYTES, &tmap_b, full_on_leader, kb * PAIR_BLOCK_K, row0);
                                if (tn == 256) {
                                    tma_load_2d_pair(a_tile + PAIR_A_BYTES + 64 * PAIR_BLOCK_K, &tmap_b, full_on_leader,
                                                     kb * PAIR_BLOCK_K, row0 + 64);
                                }
                            } else {
                                tma_load_2d_pair(a_tile + PAIR_A_BYTES, &tmap_b, full_on_leader, kb * PAIR_BLOCK_K,
                                                 col0 + static_cast<int>(rank) * C::B_ROWS);
                            }
                        }
                    }
                    return true;
                });
            };
            int done = 0;
            if (p.pdl) {
                // Dependent launch: the weights are static, so the first ring of weight tiles is requested while the
                // previous kernel of the stream is still finishing; the activations follow once it has completed.
                walk(0, PAIR_STAGES, 1);
                asm volatile("griddepcontrol.wait;" ::: "memory");
                walk(0, PAIR_STAGES, 2);
                done = PAIR_STAGES;
            }
            walk(done, 0x7fffffff, 0);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc_full = umma_idesc(KIND, PAIR_TILE_M, PAIR_TILE_N, B_MN);
            constexpr uint32_t idesc_half = umma_idesc(KIND, PAIR_TILE_M, 128, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            for_each_tile([&](int, int, int tn, int it) {
                const uint32_t idesc = (MIXED && tn == 128) ? idesc_half : idesc_full;
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait_bounded(&tempty_bar[buf], acc_phase ^ 1u, abort_word, PAIR_WAIT_LIMIT)) {
                    pair_timeout(abort_word, 112);
                    return false;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * (PAIR_TMEM_COLS / 2));
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, abort_word, PAIR_WAIT_LIMIT)) {
                        pair_timeout(abort_word, 113);
                        return false;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + stage * PAIR_STAGE_BYTES);
                    const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
                    const uint64_t b_desc = B_MN ? umma_desc_mnmajor_sw128(a_addr + PAIR_A_BYTES, C::B_BYTES, 1024)
                                                 : umma_desc_kmajor_sw128(a_addr + PAIR_A_BYTES);
#pragma unroll
                    for (int ks = 0; ks < PAIR_BLOCK_K / PAIR_UMMA_K; ++ks) {
                        const uint64_t koff = static_cast<uint64_t>((ks * PAIR_UMMA_K) >> 4);
                        // MN-major: 32 K-rows are four 1024-byte atoms further down the tile
                        const uint64_t boff = B_MN ? static_cast<uint64_t>((ks * PAIR_UMMA_K * 128) >> 4) : koff;
                        umma_ss_pair<KIND>(d_tmem, a_desc + koff, b_desc + boff, idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[stage], 0x3);  // frees this stage in both CTAs
                    if (++stage == PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                umma_commit_pair(&tfull_bar[buf], 0x3);  // accumulator ready, both CTAs' epilogues
                return true;
            });
        }
    } else {
        const int q = warp & 3;
        const int half = EW8 ? (warp - 2) >> 2 : 0;  // EW8: which half of the tile's column blocks this warp takes
        uint4* stage_buf = stage_all + (warp - 2) * (EW8 ? 128 : 256);
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // scales, C and D belong to the stream's past
        for_each_tile([&](int m_blk, int tile_col0, int tn, int it) {
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int blocks = tn / 32;
            const int c_begin = EW8 ? (half ? (blocks + 1) / 2 : 0) : 0;
            const int c_end = EW8 ? (half ? blocks : (blocks + 1) / 2) : blocks;
            float* sb_tile = sb_s + (warp - 2) * (EW8 ? C::SB_HALF : PAIR_TILE_N) - c_begin * 32;  // indexed by column of the tile
            if (!RAW && (!p.out_q8 || p.bias_kind != 0)) {
                __syncwarp();
                // all loads of the tile's scales and bias in flight together, then the shared-memory writes
                constexpr int MAX_BLK = EW8 ? (TN / 32 + 1) / 2 : TN / 32;
                float sv[MAX_BLK], bv[MAX_BLK];
#pragma unroll
                for (int j = 0; j < MAX_BLK; ++j) {
                    const int i = (c_begin + j) * 32 + lane;
                    const int col = tile_col0 + i;
                    const bool in = (c_begin + j) < c_end && col < p.n;
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
                for (int j = 0; j < MAX_BLK; ++j) {
                    const int i = (c_begin + j) * 32 + lane;
                    if (c_begin + j < c_end) {
                        if (!p.out_q8) sb_tile[i] = sv[j];
                        if (p.bias_kind != 0) sb_tile[p.bias_off + i] = bv[j];
                    }
                }
                __syncwarp();
            }
            // the row scale is requested before the wait for the accumulator, not after it
            const int row_base = m_blk * PAIR_TILE_M + static_cast<int>(rank) * CTA_ROWS + q * 32;
            const int row = row_base + lane;
            const bool row_ok = row < p.m;
            float sa_row = 1.0f;
            if (!RAW && !p.out_q8) {
                sa_row = (p.scale_mode == 1) ? (row_ok ? __ldg(p.sa + row) : 0.0f) : (p.scale_mode == 2 ? p.sa_const : __ldg(p.sa));
            }
            if (!mbar_wait_bounded(&tfull_bar[buf], acc_phase, abort_word, PAIR_WAIT_LIMIT)) {
                pair_timeout(abort_word, 114);
                return false;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                   static_cast<uint32_t>(buf * (PAIR_TMEM_COLS / 2));
            {
                int c = c_begin;
                if constexpr (!RAW && !EW8) {
                    // 64 columns at a time through the warp's staging buffer (coalesced 128-byte row segments)
                    for (; c + 2 <= c_end; c += 2) {
                        const int col0 = tile_col0 + c * 32;
                        if (col0 >= p.n) break;  // warp-uniform
                        if (p.swiglu) {  // launch-uniform; the host guarantees whole 64-column blocks and aligned rows
                            epilogue_block_64_swiglu<KIND>(p, t_row + static_cast<uint32_t>(c * 32), row_base, lane, col0, sa_row,
                                                           sb_tile + c * 32, stage_buf);
                            continue;
                        }
                        if (!block_64_ok<FUSED>(p, col0)) break;
                        epilogue_block_64<KIND, FUSED>(p, t_row + static_cast<uint32_t>(c * 32), row_base, lane, col0, sa_row,
                                                       sb_tile + c * 32, stage_buf);
                    }
                }
#pragma unroll 1
                for (; c < c_end; ++c) {
                    const int col0 = tile_col0 + c * 32;
                    if (col0 >= p.n) break;  // warp-uniform
                    if constexpr (!RAW) {
                        if (block_32_ok<FUSED>(p, col0)) {
                            epilogue_block_32<KIND, FUSED>(p, t_row + static_cast<uint32_t>(c * 32), row_base, lane, col0, sa_row,
                                                           sb_tile + c * 32, stage_buf);
                            continue;
                        }
                    }
                    if constexpr (RAW) {
                        if ((p.rs_world > 1 || p.coalesce) && p.vec_store && col0 + 32 <= p.n) {  // warp-uniform
                            epilogue_block_raw32_scatter(p, t_row + static_cast<uint32_t>(c * 32), row_base, lane, col0, stage_buf);
                            continue;
                        }
                    }
                    uint32_t r[32];
                    __syncwarp();
                    tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(c * 32), r);
                    tmem_ld_wait();
                    if (row_ok) epilogue_store_32<KIND, RAW, FUSED>(p, row, col0, r, sa_row, sb_tile + c * 32);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
            return true;
        });
    }

    // Teardown: nobody leaves (or frees TMEM) while the partner may still signal or read.
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
    }
}

// Relative cost of a 256 x 128 tile against a 256 x 256 one (1.0).  Between the operand-feed model (each CTA loads
// 128 + 64 rows instead of 128 + 128 per K step: 0.75) and the MMA count (0.5); measured on 4096^3 and the prefill set.
constexpr double MIXED_HALF_COST = 0.72;
constexpr int MIXED_MAX_PAIRS = 96;

struct MixedSchedule {
    bool ok = false;
    int full_cols = 0, pairs = 0;
    double makespan = 0.0;
    uint16_t full_begin[98] = {0};
    uint16_t half_begin[98] = {0};
};

// 256-wide tiles for the first `full_cols` tile columns, 128-wide tiles for the rest of N.  The wide tiles are dealt
// out evenly (contiguous runs, so a pair keeps its weight columns), then the narrow ones level the pairs: the smallest
// finishing time T with sum_q floor((T - load_q) / c) >= number of narrow tiles.
MixedSchedule build_mixed_schedule(int m_tiles, int n, int sm_pairs, int full_cols) {
    MixedSchedule sc;
    const int64_t f_tiles = static_cast<int64_t>(full_cols) * m_tiles;
    const int rest = n - full_cols * 256;
    const int half_cols = rest > 0 ? (rest + 127) / 128 : 0;
    const int64_t h_tiles = static_cast<int64_t>(half_cols) * m_tiles;
    if (f_tiles > 60000 || h_tiles > 60000 || f_tiles + h_tiles == 0) return sc;
    int pairs = sm_pairs < MIXED_MAX_PAIRS ? sm_pairs : MIXED_MAX_PAIRS;
    if (f_tiles + h_tiles < pairs) pairs = static_cast<int>(f_tiles + h_tiles);
    const int base = static_cast<int>(f_tiles / pairs), extra = static_cast<int>(f_tiles % pairs);
    const double c = MIXED_HALF_COST;
    auto cap = [&](double t, int load) { return t > load ? static_cast<int64_t>((t - load) / c + 1e-9) : 0; };
    double lo = base, hi = base + 1 + (h_tiles / pairs + 2) * c;
    for (int i = 0; i < 40; ++i) {
        const double mid = 0.5 * (lo + hi);
        const int64_t can = (pairs - extra) * cap(mid, base) + extra * cap(mid, base + 1);
        if (can >= h_tiles) hi = mid; else lo = mid;
    }
    int64_t left = h_tiles;
    int fpos = 0, hpos = 0;
    double worst = 0.0;
    for (int q = 0; q < pairs; ++q) {
        const int load = base + (q < extra ? 1 : 0);
        int64_t take = cap(hi, load);
        if (take > left) take = left;
        if (q == pairs - 1) take = left;  // rounding slack, if any, ends on the last pair
        sc.full_begin[q] = static_cast<uint16_t>(fpos);
        sc.half_begin[q] = static_cast<uint16_t>(hpos);
        fpos += load;
        hpos += static_cast<int>(take);
        left -= take;
        const double t = load + c * take;
        if (t > worst) worst = t;
    }
    sc.full_begin[pairs] = static_cast<uint16_t>(fpos);
    sc.half_begin[pairs] = static_cast<uint16_t>(hpos);
    sc.ok = (fpos == f_tiles && hpos == h_tiles);
    sc.full_cols = full_cols;
    sc.pairs = pairs;
    sc.makespan = worst;
    return sc;
}

template <uint32_t KIND, bool RAW, bool FUSED, int TN, bool B_MN = false, bool MIXED = false, bool EW8 = false>
int32_t launch_pair_tn(const GemmDesc& g, cudaStream_t stream, const MixedSchedule* mixed = nullptr) {
    using C = PairCfg<TN>;
    constexpr int PAIR_TILE_N = TN;
    constexpr int PAIR_SMEM_TOTAL = C::SMEM_TOTAL;
    const int sms = sm_count_of_current_device();
    if (sms < 2) return BQ_STATUS_LAUNCH_FAILURE;
    CUtensorMap map_a, map_b;
    if (!make_kmajor_tensor_map(&map_a, g.a, g.m, g.k, g.lda, CTA_ROWS)) return BQ_STATUS_LAUNCH_FAILURE;
    if constexpr (B_MN) {
        if (!make_mnmajor_tensor_map(&map_b, g.b, g.k, g.n, g.ldb, PAIR_BLOCK_K)) return BQ_STATUS_LAUNCH_FAILURE;
    } else {
        if (!make_kmajor_tensor_map(&map_b, g.b, g.n, g.k, g.ldb, MIXED ? 64 : C::B_ROWS)) return BQ_STATUS_LAUNCH_FAILURE;
    }
    GemmParams p;
    p.mixed = 0;
    p.mixed_full_cols = 0;
    p.pdl = g.pdl;
    {
        // row blocks of A per group: as many as keep the group's A rows (256 x K bytes each) within about 36 MB, the
        // share of the L2 that stays resident beside the weight and output streams; groups of equal height
        const int m_tiles = (g.m + PAIR_TILE_M - 1) / PAIR_TILE_M;
        const int64_t row_block_bytes = static_cast<int64_t>(PAIR_TILE_M) * (g.k > 0 ? g.k : 1);
        int64_t gm_max = (36LL << 20) / row_block_bytes;
        if (gm_max < 2) gm_max = 2;
        const int groups = static_cast<int>((m_tiles + gm_max - 1) / gm_max);
        p.raster_gm = (m_tiles + groups - 1) / (groups > 0 ? groups : 1);
        if (p.raster_gm < 1) p.raster_gm = 1;
    }
    if constexpr (MIXED) {
        if (!mixed || !mixed->ok) return BQ_STATUS_LAUNCH_FAILURE;
        p.mixed = 1;
        p.mixed_full_cols = mixed->full_cols;
        for (int i = 0; i < 98; ++i) {
            p.full_begin[i] = mixed->full_begin[i];
            p.half_begin[i] = mixed->half_begin[i];
        }
    }
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
    p.m_tiles = (g.m + PAIR_TILE_M - 1) / PAIR_TILE_M;
    p.n_tiles = (g.n + PAIR_TILE_N - 1) / PAIR_TILE_N;
    const int64_t elem = RAW ? 4 : (g.q8_out ? 1 : 2);
    p.out_q8 = RAW ? 0 : g.q8_out;
    p.c = g.c;
    p.ldc = g.ldc;
    p.beta = g.beta;
    p.bias = g.bias;
    p.bias_kind = g.bias ? g.bias_kind : 0;
    p.act = g.act;
    p.bias_off = PairCfg<TN>::SB_FLOATS;
    p.vec_store = ((reinterpret_cast<uintptr_t>(g.d) & 15u) == 0 && ((g.ldd * elem) & 15) == 0) ? 1 : 0;
    p.n_peers = FUSED ? g.n_peers : 0;
    p.peer_ld = g.peer_ld;
    p.peer_col0 = g.peer_col0;
    p.peer_rank = g.peer_rank;
    p.rs_world = RAW ? g.rs_world : 0;
    p.swiglu = (!RAW && !FUSED && !g.q8_out) ? g.swiglu : 0;
    p.rs_rows = g.rs_rows;
    p.peer_vec = ((g.peer_ld * 2) & 15) == 0 && ((static_cast<int64_t>(g.peer_col0) * 2) & 15) == 0;
    for (int r = 0; r < 8; ++r) {
        p.peer_d[r] = g.peer_d[r];
        if (r < p.n_peers && (reinterpret_cast<uintptr_t>(g.peer_d[r]) & 15u) != 0) p.peer_vec = 0;
    }
    // the multicast store is 16 bytes wide: used only where every tile takes the staged path, else the unicast stores run
    p.mc_d = (FUSED && p.peer_vec && p.vec_store && (g.n % 32) == 0 && (reinterpret_cast<uintptr_t>(g.mc_d) & 15u) == 0) ? g.mc_d
                                                                                                                  : nullptr;
    auto kern = gemm_q8_pair_kernel<KIND, RAW, FUSED, TN, B_MN, MIXED, EW8>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_TOTAL) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
    const int64_t pairs = MIXED ? mixed->pairs : (tiles < sms / 2 ? tiles : sms / 2);
    // Output rows go through the shared-memory staging (full 128-byte row segments per store) when the
    // stores cross NVLink (fused mode) or when there are so few waves of tiles that the last epilogue is
    // exposed; in long steady-state runs the direct per-thread stores leave more shared-memory bandwidth
    // to the tensor cores and measure 2-5 % faster.  direct_stores: 1 forces direct, 2 forces staged.
    const int64_t waves = (tiles + pairs - 1) / pairs;
    p.coalesce = (g.direct_stores == 2) || (g.direct_stores == 0 && (FUSED || waves <= 6));
    if (p.out_q8) p.coalesce = 0;  // the staging path is bf16-only
    // raw 32-bit output: 128 bytes per row and block, always worth staging (8192 x 28672 x 4096: 704 -> 624 us)
    if (RAW) p.coalesce = g.direct_stores != 1 ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    cfg.blockDim = dim3(EW8 ? PAIR_THREADS + 128 : PAIR_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PAIR_SMEM_TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g.pdl ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, kern, map_a, map_b, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

// Tile width: the kernel is fed through L2, so a tile costs what each CTA loads per K step
// (128 rows of A plus TN/2 rows of the weight); pick the width that minimises
// (waves of pair tiles) x (that cost).  Narrow tiles only win when they remove a whole wave.
int pick_tile_n(const GemmDesc& g) {
    if (g.force_pair_tile_n != 0 && g.force_pair_tile_n != 2) return g.force_pair_tile_n;
    const int sms = sm_count_of_current_device();
    const int64_t pairs = sms / 2 > 0 ? sms / 2 : 1;
    const int64_t m_tiles = (g.m + PAIR_TILE_M - 1) / PAIR_TILE_M;
    const int cand[4] = {256, 224, 192, 128};
    int best = 256;
    int64_t best_cost = INT64_MAX;
    for (int i = 0; i < 4; ++i) {
        if (g.swiglu && cand[i] % 64 != 0) continue;  // gate/up blocks of 64 columns must not straddle tiles
        const int64_t tiles = m_tiles * ((g.n + cand[i] - 1) / cand[i]);
        const int64_t waves = (tiles + pairs - 1) / pairs;
        const int64_t cost = waves * (CTA_ROWS + cand[i] / 2);
        if (cost < best_cost) {
            best_cost = cost;
            best = cand[i];
        }
    }
    return best;
}

// Cost of the best single-width schedule, in 256 x 256 tile times.
double single_width_cost(const GemmDesc& g, int tn) {
    const int sms = sm_count_of_current_device();
    const int64_t pairs = sms / 2 > 0 ? sms / 2 : 1;
    const int64_t tiles = static_cast<int64_t>((g.m + PAIR_TILE_M - 1) / PAIR_TILE_M) * ((g.n + tn - 1) / tn);
    return static_cast<double>((tiles + pairs - 1) / pairs) * (CTA_ROWS + tn / 2) / 256.0;
}

template <uint32_t KIND, bool RAW, bool FUSED>
int32_t launch_pair(const GemmDesc& g, cudaStream_t stream) {
    if (g.b_layout == BQ_LAYOUT_RRR) return launch_pair_tn<KIND, RAW, FUSED, 256, true>(g, stream);
    const int tn = pick_tile_n(g);
    // Mixed widths: when the wide tiles do not fill their last wave, the columns of that wave are cut into 128-wide
    // tiles spread over all pairs (force_pair_tile_n 2 forces the mixed schedule, any other forced width keeps it off).
    // Every pair walks its own contiguous run of tiles, so the pairs are spread over the whole matrix at any moment:
    // fine while both operands fit in L2 (64 MB), which is also where partly filled waves matter.
    const int64_t operand_bytes = (static_cast<int64_t>(g.m) + g.n) * g.k;
    if (g.force_pair_tile_n == 2 || (g.force_pair_tile_n == 0 && operand_bytes <= (64LL << 20))) {
        const int sm_pairs = sm_count_of_current_device() / 2;
        const int m_tiles = (g.m + PAIR_TILE_M - 1) / PAIR_TILE_M;
        const int nc = g.n / 256;
        MixedSchedule best;
        for (int x = nc; x >= 0 && x >= nc - 3; --x) {
            const MixedSchedule sc = build_mixed_schedule(m_tiles, g.n, sm_pairs, x);
            if (sc.ok && (!best.ok || sc.makespan < best.makespan - 1e-9)) best = sc;
        }
        if (best.ok && (g.force_pair_tile_n == 2 || best.makespan < 0.98 * single_width_cost(g, tn))) {
            return launch_pair_tn<KIND, RAW, FUSED, 256, false, true>(g, stream, &best);
        }
    }
    if constexpr (!RAW && !FUSED) {
        // bias + gelu / silu with at most two waves of tiles: eight epilogue warps, because the last tile's epilogue is
        // exposed (512 x 14336 x 4096 gelu 44 -> 42 us).  In longer runs four warps hide the chain behind the next
        // tile's MMAs just as well since it shrank to fifteen instructions per element (8192 x 28672 x 4096: 660 us
        // either way), and at K = 8192 the extra warps slow the main loop.
        const int64_t ew_tiles = static_cast<int64_t>((g.m + PAIR_TILE_M - 1) / PAIR_TILE_M) * ((g.n + tn - 1) / tn);
        const bool ew8 = g.epilogue_warps == 8 ||
                         (g.epilogue_warps == 0 && g.act >= 2 && ew_tiles <= 2 * (sm_count_of_current_device() / 2));
        if (ew8 && !g.swiglu) {
            switch (tn) {
                case 256: return launch_pair_tn<KIND, false, false, 256, false, false, true>(g, stream);
                case 224: return launch_pair_tn<KIND, false, false, 224, false, false, true>(g, stream);
                case 192: return launch_pair_tn<KIND, false, false, 192, false, false, true>(g, stream);
                case 128: return launch_pair_tn<KIND, false, false, 128, false, false, true>(g, stream);
                default: return BQ_STATUS_INVALID_PROBLEM;
            }
        }
    }
    switch (tn == 2 ? 256 : tn) {
        case 256: return launch_pair_tn<KIND, RAW, FUSED, 256>(g, stream);
        case 224: return launch_pair_tn<KIND, RAW, FUSED, 224>(g, stream);
        case 192: return launch_pair_tn<KIND, RAW, FUSED, 192>(g, stream);
        case 128: return launch_pair_tn<KIND, RAW, FUSED, 128>(g, stream);
        default: return BQ_STATUS_INVALID_PROBLEM;
    }
}

}  // namespace

int32_t launch_gemm_q8_pair(const GemmDesc& g, cudaStream_t stream) {
    const bool fused = g.n_peers > 0 && !g.raw_out;
    if (g.kind == BQ_KIND_S8) {
        if (g.raw_out) return launch_pair<UMMA_KIND_I8, true, false>(g, stream);
        return fused ? launch_pair<UMMA_KIND_I8, false, true>(g, stream) : launch_pair<UMMA_KIND_I8, false, false>(g, stream);
    }
    if (g.raw_out) return launch_pair<UMMA_KIND_F8, true, false>(g, stream);
    return fused ? launch_pair<UMMA_KIND_F8, false, true>(g, stream) : launch_pair<UMMA_KIND_F8, false, false>(g, stream);
}

int32_t read_and_clear_gemm_pair_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_pair_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_gemm_pair_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
