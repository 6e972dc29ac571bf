// 8-bit tensor-core GEMM for sm_100a: D[M,N] = epilogue(A[M,K] x B[K,N]) with
// A row-major and B column-major ("RCR": both operands K-contiguous).
//
// One persistent CTA per SM, six warps with fixed roles:
//   warp 0    TMA producer: streams 128-byte-swizzled A and B tiles through a
//             ring of shared-memory stages, one mbarrier pair per stage;
//   warp 1    owns TMEM and issues tcgen05.mma (s8 x s8 -> s32 or
//             e4m3 x e4m3 -> f32), 128 x BLOCK_N x 32 per instruction;
//   warps 2-5 epilogue: tcgen05.ld the accumulator, apply the fused
//             per-row x per-column dequant scale, write bf16 (or the raw
//             32-bit accumulators).
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps
// the main loop of tile i+1.  Every barrier wait is bounded; a wait that runs
// out records a status word and all roles leave.
//
// Replaces, for the bf16-out W8A8 / FP8 use, the reference's
//   crates/baracuda-cutlass-kernels-sys/kernels/gemm_s8_rcr_sm80.cu:48-198 (s8 RCR tensor-core GEMM)
//   crates/baracuda-kernels-sys/kernels/include/baracuda_fp8_rcr_sm89.cuh:102-323 (e4m3 RCR GEMM)
//   crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:245-301 (W8A8 dequant math)

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "gemm_q8_common.cuh"
#include "launch.h"
#include "ptx_sm100a.cuh"

namespace bq {

__device__ int g_gemm_device_status = 0;

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;  // bytes of K per stage == one 128-byte swizzle row
constexpr int UMMA_K = 32;    // K per tcgen05.mma for 8-bit operands
constexpr int GEMM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr long long WAIT_LIMIT_CYCLES = 1LL << 31;  // about a second


template <int BLOCK_N, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BLOCK_M * BLOCK_K;
    static constexpr int B_BYTES = BLOCK_N * BLOCK_K;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int STG_BYTES = 4 * 4096;        // per epilogue warp: 32 rows x 128 bytes of output staging
    static constexpr int SB_BYTES = STG_BYTES + 2 * 4 * BLOCK_N * 4;  // + private copies of the column scales and of the bias per epilogue warp
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int TOTAL = TILE_BYTES + SB_BYTES + BAR_BYTES + 1024;  // + alignment slack
    static constexpr int TMEM_COLS = (2 * BLOCK_N <= 32) ? 32 : (2 * BLOCK_N <= 64) ? 64
                                     : (2 * BLOCK_N <= 128) ? 128 : (2 * BLOCK_N <= 256) ? 256 : 512;
};

__device__ __forceinline__ void record_timeout(volatile uint32_t* abort_word, int code) {
    *abort_word = 1u;
    atomicCAS(&g_gemm_device_status, 0, code);
}

template <uint32_t KIND, bool RAW, int BLOCK_N, int STAGES, bool FUSED = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_q8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmParams p) {
    using L = Smem<BLOCK_N, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    // round up inside the shared window (an offset added to the shared array keeps shared-memory addressing)
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* tiles = smem;
    uint4* stage_all = reinterpret_cast<uint4*>(smem + L::TILE_BYTES);
    float* sb_s = reinterpret_cast<float*>(smem + L::TILE_BYTES + L::STG_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::TILE_BYTES + L::SB_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);
            mbar_init(&tempty_bar[b], EPI_THREADS);
        }
        *abort_word = 0u;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, L::TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = (p.k + BLOCK_K - 1) / BLOCK_K;
    const int total_tiles = p.m_tiles * p.n_tiles;

    // let the next kernel of the stream be scheduled as SMs free up (matters only to a programmatic dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            // step i of this CTA's (tile, K block) sequence uses ring stage i % STAGES in phase (i / STAGES) & 1.
            // what: 0 = arm the barrier and load both operands, 1 = arm and load the weights only, 2 = activations only
            auto walk = [&](int first, int last, int what) {
                int idx = 0;
                for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                    const int m_blk = tile % p.m_tiles;
                    const int n_blk = tile / p.m_tiles;
                    for (int kb = 0; kb < num_kb; ++kb, ++idx) {
                        if (idx < first) continue;
                        if (idx >= last) return;
                        const int stage = idx % STAGES;
                        const uint32_t phase = static_cast<uint32_t>(idx / STAGES) & 1u;
                        if (what == 0 && !mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_word, WAIT_LIMIT_CYCLES)) {
                            record_timeout(abort_word, 101);
                            return;
                        }
                        uint8_t* sa_tile = tiles + stage * L::STAGE_BYTES;
                        if (what != 2) mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
                        if (what != 1) tma_load_2d(sa_tile, &tmap_a, &full_bar[stage], kb * BLOCK_K, m_blk * BLOCK_M);
                        if (what != 2) tma_load_2d(sa_tile + L::A_BYTES, &tmap_b, &full_bar[stage], kb * BLOCK_K, n_blk * BLOCK_N);
                    }
                }
            };
            int done = 0;
            if (p.pdl) {
                // dependent launch: the first ring of (static) weight tiles is requested while the previous kernel of
                // the stream is still finishing; the activations follow once it has completed
                walk(0, STAGES, 1);
                asm volatile("griddepcontrol.wait;" ::: "memory");
                walk(0, STAGES, 2);
                done = STAGES;
            }
            walk(done, 0x7fffffff, 0);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(KIND, BLOCK_M, BLOCK_N);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait_bounded(&tempty_bar[buf], acc_phase ^ 1u, abort_word, WAIT_LIMIT_CYCLES)) {
                    record_timeout(abort_word, 102);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BLOCK_N);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, abort_word, WAIT_LIMIT_CYCLES)) {
                        record_timeout(abort_word, 103);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + stage * L::STAGE_BYTES);
                    const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_kmajor_sw128(a_addr + L::A_BYTES);
#pragma unroll
                    for (int ks = 0; ks < BLOCK_K / UMMA_K; ++ks) {
                        // advancing K inside the swizzle row = adding the byte offset (in 16-byte units)
                        const uint64_t koff = static_cast<uint64_t>((ks * UMMA_K) >> 4);
                        umma_ss<KIND>(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(&tfull_bar[buf]);
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        uint4* stage_buf = stage_all + (warp - 2) * 256;
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // scales, C and D belong to the stream's past
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int m_blk = tile % p.m_tiles;
            const int n_blk = tile / p.m_tiles;
            // each warp stages its own copy of this tile's column scales, so the
            // epilogue warps never have to meet at a barrier
            float* sb_tile = sb_s + (warp - 2) * BLOCK_N;
            if (!RAW && (!p.out_q8 || p.bias_kind != 0)) {
                __syncwarp();
                // all loads of the tile's scales and bias in flight together, then the shared-memory writes
                float sv[BLOCK_N / 32], bv[BLOCK_N / 32];
#pragma unroll
                for (int j = 0; j < BLOCK_N / 32; ++j) {
                    const int col = n_blk * BLOCK_N + j * 32 + lane;
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
                for (int j = 0; j < BLOCK_N / 32; ++j) {
                    if (!p.out_q8) sb_tile[j * 32 + lane] = sv[j];
                    if (p.bias_kind != 0) sb_tile[p.bias_off + j * 32 + lane] = bv[j];
                }
                __syncwarp();
            }
            // the row scale is requested before the wait for the accumulator, not after it
            const int row = m_blk * BLOCK_M + q * 32 + lane;
            const bool row_ok = row < p.m;
            float sa_row = 1.0f;
            if (!RAW && !p.out_q8) {
                sa_row = (p.scale_mode == 1) ? (row_ok ? __ldg(p.sa + row) : 0.0f) : (p.scale_mode == 2 ? p.sa_const : __ldg(p.sa));
            }
            if (!mbar_wait_bounded(&tfull_bar[buf], acc_phase, abort_word, WAIT_LIMIT_CYCLES)) {
                record_timeout(abort_word, 104);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                   static_cast<uint32_t>(buf * BLOCK_N);
            {
                int c = 0;
                if constexpr (!RAW) {
                    // 64 columns at a time through the warp's staging buffer (coalesced 128-byte row segments)
                    for (; c + 2 <= BLOCK_N / 32; c += 2) {
                        const int col0 = n_blk * BLOCK_N + c * 32;
                        if (col0 >= p.n) break;  // warp-uniform
                        if (p.swiglu) {  // launch-uniform; the host guarantees whole 64-column blocks and aligned rows
                            epilogue_block_64_swiglu<KIND>(p, t_row + static_cast<uint32_t>(c * 32), m_blk * BLOCK_M + q * 32, lane, col0, sa_row,
                                                           sb_tile + c * 32, stage_buf);
                            continue;
                        }
                        if (!block_64_ok<FUSED>(p, col0)) break;
                        epilogue_block_64<KIND, FUSED>(p, t_row + static_cast<uint32_t>(c * 32), m_blk * BLOCK_M + q * 32, lane, col0, sa_row,
                                                       sb_tile + c * 32, stage_buf);
                    }
                }
#pragma unroll 1
                for (; c < BLOCK_N / 32; ++c) {
                    const int col0 = n_blk * BLOCK_N + c * 32;
                    if (col0 >= p.n) break;  // warp-uniform
                    if constexpr (!RAW) {
                        if (block_32_ok<FUSED>(p, col0)) {
                            epilogue_block_32<KIND, FUSED>(p, t_row + static_cast<uint32_t>(c * 32), m_blk * BLOCK_M + q * 32, lane, col0, sa_row,
                                                           sb_tile + c * 32, stage_buf);
                            continue;
                        }
                    }
                    if constexpr (RAW) {
                        if ((p.rs_world > 1 || p.coalesce) && p.vec_store && col0 + 32 <= p.n) {  // warp-uniform
                            epilogue_block_raw32_scatter(p, t_row + static_cast<uint32_t>(c * 32), m_blk * BLOCK_M + q * 32, lane, col0, stage_buf);
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
            mbar_arrive(&tempty_bar[buf]);
        }
    }

    // Teardown.  On the error path give copies and MMAs still in flight a
    // bounded time to land before TMEM goes back.
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// K == 0: the contraction is empty, every output is the scaled zero.
template <typename T>
__global__ void fill_zero_kernel(T* d, int64_t ldd, int m, int n) {
    const int64_t total = static_cast<int64_t>(m) * n;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / n, c = i % n;
        d[r * ldd + c] = T(0);
    }
}

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

// rows x k bytes, K contiguous, row pitch ld bytes; box = box_rows x 128 bytes, 128-byte swizzle.
bool make_kmajor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
    auto enc = tensor_map_encoder();
    if (!enc) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    // a single row never uses its pitch; any 16-byte multiple satisfies the encoder
    cuuint64_t pitch = static_cast<cuuint64_t>(rows > 1 ? ld : ((k + 15) / 16) * 16);
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(BLOCK_K), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

int sm_count_impl() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    static std::mutex mu;
    static int cache[64] = {0};
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && cache[dev] > 0) return cache[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) cache[dev] = n;
    return n;
}

template <uint32_t KIND, bool RAW, int BLOCK_N, int STAGES, bool FUSED = false>
int32_t launch_config(const GemmDesc& g, int sms, cudaStream_t stream) {
    using L = Smem<BLOCK_N, STAGES>;
    CUtensorMap map_a, map_b;
    if (!make_kmajor_map(&map_a, g.a, g.m, g.k, g.lda, BLOCK_M)) return BQ_STATUS_LAUNCH_FAILURE;
    if (!make_kmajor_map(&map_b, g.b, g.n, g.k, g.ldb, BLOCK_N)) return BQ_STATUS_LAUNCH_FAILURE;
    GemmParams p;
    p.d = g.d;
    p.ldd = g.ldd;
    p.sa = g.scale_a;
    p.sb = g.scale_b;
    p.scale_mode = g.scale_mode;
    p.sa_const = g.sa_const;
    p.pdl = g.pdl;
    p.mixed = 0;
    p.mixed_full_cols = 0;
    p.raster_gm = 1;
    p.alpha = g.alpha;
    p.m = g.m;
    p.n = g.n;
    p.k = g.k;
    p.m_tiles = (g.m + BLOCK_M - 1) / BLOCK_M;
    p.n_tiles = (g.n + BLOCK_N - 1) / BLOCK_N;
    p.kb_per_slice = 0;
    const int64_t elem = RAW ? 4 : (g.q8_out ? 1 : 2);
    p.out_q8 = RAW ? 0 : g.q8_out;
    p.c = g.c;
    p.ldc = g.ldc;
    p.beta = g.beta;
    p.bias = g.bias;
    p.bias_kind = g.bias ? g.bias_kind : 0;
    p.act = g.act;
    p.bias_off = 4 * BLOCK_N;
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
    auto kern = gemm_q8_kernel<KIND, RAW, BLOCK_N, STAGES, FUSED>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
    const int grid = static_cast<int>(tiles < sms ? tiles : sms);
    p.coalesce = (g.direct_stores == 2) || (g.direct_stores == 0 && (FUSED || (tiles + grid - 1) / grid <= 6));
    if (p.out_q8) p.coalesce = 0;  // the staging path is bf16-only
    // raw 32-bit output: 128 bytes per row and block, always worth staging (8192 x 28672 x 4096: 704 -> 624 us)
    if (RAW) p.coalesce = g.direct_stores != 1 ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, map_a, map_b, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

// Cost model of the small problems (fewer than one wave of wide tiles), fitted to measurements at M = 32..384 against
// one layer's weights coming from HBM: a wave of tiles walks one 128-byte K block in about COST_KB microseconds (narrow
// tiles are cheaper per block but not in proportion -- an SM ingests operands at a bounded rate), every further
// wave costs the same again, and a launch cannot beat the weight bytes over the HBM rate.
constexpr float COST_KB_64 = 0.22f, COST_KB_128 = 0.25f, COST_KB_256 = 0.40f, COST_KB_PAIR = 0.33f;
constexpr float PAIR_FIXED_US = 2.0f;      // cluster launch and pair hand-shakes
constexpr float HBM_BYTES_PER_US = 6.5e6f;

float wave_cost(int64_t tiles, int sms, float cost_kb, int64_t num_kb) {
    return static_cast<float>((tiles + sms - 1) / sms) * cost_kb * static_cast<float>(num_kb);
}

// Estimated time of the best one-pass launch; *bn_out: 64 / 128 / 256, or 512 for the CTA-pair kernel.
float one_pass_cost(int64_t m, int64_t n, int64_t k, int sms, bool allow_pair, int* bn_out) {
    const int64_t m_tiles = (m + BLOCK_M - 1) / BLOCK_M;
    const int64_t num_kb = (k + BLOCK_K - 1) / BLOCK_K;
    const int widths[3] = {64, 128, 256};
    const float costs[3] = {COST_KB_64, COST_KB_128, COST_KB_256};
    float best = 0.0f;
    int bn = 0;
    for (int i = 0; i < 3; ++i) {
        const float c = wave_cost(m_tiles * ((n + widths[i] - 1) / widths[i]), sms, costs[i], num_kb);
        if (bn == 0 || c < best) {
            best = c;
            bn = widths[i];
        }
    }
    if (allow_pair && m > BLOCK_M && n >= 512 && (m % 256 == 0 || m % 256 >= BLOCK_M)) {  // no mostly empty row block
        const int64_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
        const float c = wave_cost(pair_tiles, sms / 2, COST_KB_PAIR, num_kb) + PAIR_FIXED_US;
        if (c < best) {
            best = c;
            bn = 512;
        }
    }
    if (bn_out) *bn_out = bn;
    const float hbm = static_cast<float>(n) * static_cast<float>(k) / HBM_BYTES_PER_US;
    return best > hbm ? best : hbm;
}

// Split-K inside a thread-block cluster (gemm_q8_splitk_sm100a.cu), slices of this launch (0 = none).  A problem whose
// 128 x 128 tiles cover at most half of the SMs walks its whole K on a few SMs while the others idle; clusters of 2 or 4
// CTAs per tile cut that walk, at the price of the exchange through distributed shared memory (about a microsecond).
// Slices of at least four K blocks, every cluster resident at once; taken when the model gains at least a microsecond
// (CUDA-graph timing over rotating weights, M <= 128: 4096 x 4096 12.5 -> 8.5 us, K = 14336 against 4096 columns
// 32 -> 16 us, K = 8192 20.3 -> 12.2 us, 8192 x 8192 20.8 -> 17.5 us with two slices).
constexpr int SPLIT_MIN_KB = 16;  // K >= 2048 bytes
constexpr float CLUSTER_SPLIT_FIXED_US = 1.0f;
constexpr float COST_KB_WIDE_SPLIT = 0.39f;   // 128 x 256 tiles, every SM busy
constexpr float WIDE_SPLIT_FIXED_US = 2.3f;   // two meetings of the cluster, 64 KB exchanged per CTA, 128 columns of epilogue

struct SplitChoice {
    int slices = 0;  // 0 = none
    int bn = 128;
};

SplitChoice cluster_split_choice(const GemmDesc& g, int sms) {
    SplitChoice none, pick;
    if (g.cluster_split_k == 1 || g.raw_out || g.swiglu || g.n_peers > 0 || g.rs_world > 0 || g.force_block_n != 0) return none;
    const bool rrr = g.b_layout == BQ_LAYOUT_RRR;  // row-major weights: the 128-wide shapes only
    const int64_t num_kb = (static_cast<int64_t>(g.k) + BLOCK_K - 1) / BLOCK_K;
    const int64_t m_tiles = (static_cast<int64_t>(g.m) + BLOCK_M - 1) / BLOCK_M;
    if (g.cluster_split_k != 0) {  // forced: 2 / 4 slices of 128-wide tiles, 256 = two slices of 256-wide tiles
        pick.slices = g.cluster_split_k == 256 ? 2 : g.cluster_split_k;
        pick.bn = g.cluster_split_k == 256 ? 256 : 128;
        const int64_t kbps = (num_kb + pick.slices - 1) / pick.slices;
        const bool ok = num_kb >= pick.slices && (num_kb + kbps - 1) / kbps == pick.slices && !(rrr && pick.bn != 128) &&
                        gemm_q8_cluster_split_k_max_clusters(g.kind, pick.slices, pick.bn) > 0;
        return ok ? pick : none;
    }
    if (num_kb < SPLIT_MIN_KB) return none;
    const float hbm = static_cast<float>(g.n) * static_cast<float>(g.k) / HBM_BYTES_PER_US;
    float best = one_pass_cost(g.m, g.n, g.k, sms, true, nullptr) - 1.0f;
    if (rrr) {  // the one-pass form of this layout is the CTA-pair kernel, whatever the shape
        const int64_t pair_tiles = ((static_cast<int64_t>(g.m) + 255) / 256) * ((static_cast<int64_t>(g.n) + 255) / 256);
        const float c = wave_cost(pair_tiles, sms / 2 > 0 ? sms / 2 : 1, COST_KB_PAIR, num_kb) + PAIR_FIXED_US;
        best = (c > hbm ? c : hbm) - 1.0f;
    }
    // small batches: 128 x 128 tiles on at most half of the SMs, two or four slices
    const int64_t tiles = m_tiles * ((static_cast<int64_t>(g.n) + 127) / 128);
    if (2 * tiles <= sms) {
        for (int s = 2; s <= 4; s += 2) {
            const int64_t kbps = (num_kb + s - 1) / s;
            if (s * tiles > sms || kbps < 4 || (num_kb + kbps - 1) / kbps != s) continue;
            if (tiles > gemm_q8_cluster_split_k_max_clusters(g.kind, s, 128)) continue;
            const float walk = static_cast<float>(kbps) * COST_KB_128;
            const float c = (walk > hbm ? walk : hbm) + CLUSTER_SPLIT_FIXED_US;
            if (c < best) {
                best = c;
                pick.slices = s;
                pick.bn = 128;
            }
        }
    }
    // three or more row blocks against few columns and a long K (prefill at M = 512 against the down projection): the
    // 128 x 128 tiles already fill the SMs, but each SM ingests 32 KB per K block for a 128 x 128 tile; two CTAs per
    // 128 x 256 tile, half of K each, ingest 48 KB per K block for twice the tile.  Fitted to CUDA-graph timing at
    // M = 384..1024 (512 x 4096 x 14336 33.7 -> 29.6 us, 512 x 4096 x 8192 22.2 -> 20.2, 1024 x 2048 x 8192 21.8 -> 19.4;
    // at K = 4096 the exchange costs what the walk saves).
    const int64_t tiles256 = m_tiles * ((static_cast<int64_t>(g.n) + 255) / 256);
    if (!rrr && g.m > 256 && num_kb >= 60 && 2 * tiles256 <= sms && tiles256 <= gemm_q8_cluster_split_k_max_clusters(g.kind, 2, 256)) {
        const float walk = static_cast<float>((num_kb + 1) / 2) * COST_KB_WIDE_SPLIT;
        const float c = (walk > hbm ? walk : hbm) + WIDE_SPLIT_FIXED_US;
        if (c < best) {
            best = c;
            pick.slices = 2;
            pick.bn = 256;
        }
    }
    return pick;
}

template <uint32_t KIND, bool RAW>
int32_t launch_kind(const GemmDesc& g, cudaStream_t stream) {
    const int sms = sm_count_impl();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    if constexpr (!RAW) {
        const SplitChoice cs = cluster_split_choice(g, sms);
        if (cs.slices > 1) return launch_gemm_q8_cluster_split_k(g, cs.slices, cs.bn, stream);
    }
    const int64_t m_tiles = (g.m + BLOCK_M - 1) / BLOCK_M;
    auto tiles_at = [&](int bn) { return m_tiles * ((g.n + bn - 1) / bn); };
    if (g.b_layout == BQ_LAYOUT_RRR) return launch_gemm_q8_pair(g, stream);  // row-major weights: CTA-pair kernel only
    // 256 x 256 tiles on CTA pairs (force_block_n 512 forces it, 256/128/64 forces it off) from 24 such tiles up:
    // measured at M = 512, K = 4096..14336 (32 to 48 tiles) the pair kernel is 1.4-1.7x faster than 128 x 64 tiles
    // on every SM, whose operand traffic per MAC is three times higher; at 16 tiles the narrow tiles still win.
    const int64_t pair_tiles = ((g.m + 255) / 256) * static_cast<int64_t>((g.n + 255) / 256);
    const int64_t pairs = sms / 2;
    bool use_pair = g.force_block_n == 512 || (g.force_block_n == 0 && g.m >= 512 && g.n >= 512 && pair_tiles >= 24);
    int bn = g.force_block_n;
    if (g.force_block_n == 0) {
        // One or two row blocks of 256 rows with at least a wave and a half of pair tiles also go to the pair kernel
        // (256 x 28672 x 4096: 31.0 us against 35.6 us on 128 x 256 tiles).
        if (!use_pair && g.m >= 256 && g.n >= 512 && (g.m % 256 == 0 || g.m % 256 > 128) && 2 * pair_tiles >= 3 * pairs) {
            use_pair = true;
        }
        // A single, partly filled wave of pair tiles: if 128 x 256 or 128 x 128 tiles fill at least 80 % of the SMs in
        // ONE wave, they win -- the 1-CTA kernel starts and ends about 2 us sooner (no cluster launch, no pair
        // hand-shakes): 512 x 4096 x 4096 13.1 against 15.4 us, 1024 x 4096 x 4096 16.5 against 18.7 us,
        // 512 x 4096 x 14336 33.5 against 38.0 us (CUDA-graph timing).  With less fill the pair kernel's lower operand
        // traffic wins again (512 x 6144 x 4096: 96 tiles of 128 x 256, 18.3 against 16.7 us).
        if (use_pair && pair_tiles <= pairs) {
            const int cand[2] = {256, 128};
            for (int i = 0; i < 2; ++i) {
                const int64_t t = tiles_at(cand[i]);
                if (t <= sms && 5 * t >= 4 * static_cast<int64_t>(sms)) {
                    use_pair = false;
                    bn = cand[i];
                    break;
                }
            }
        }
    }
    if (use_pair) return launch_gemm_q8_pair(g, stream);
    if (bn == 0) {
        // small problems: the tile width (or the pair kernel) with the cheapest waves.  The old rule -- the widest tile
        // that still gives every SM a tile -- spilled many shapes into a second wave of narrow tiles
        // (384 x 4096 x 14336: 192 tiles of 128 x 64 took 65.6 us, 96 tiles of 128 x 128 take 40.4 us;
        // 256 x 8192 x 8192 43.0 -> 30.7 us; 32 x 14336 x 4096 26.6 -> 23.0 us)
        (void)one_pass_cost(g.m, g.n, g.k, sms, true, &bn);
        if (bn == 512) return launch_gemm_q8_pair(g, stream);
    }
    if constexpr (!RAW) {
        if (g.n_peers > 0) {
            switch (bn) {
                case 256: return launch_config<KIND, RAW, 256, 4, true>(g, sms, stream);
                case 128: return launch_config<KIND, RAW, 128, 6, true>(g, sms, stream);
                case 64: return launch_config<KIND, RAW, 64, 8, true>(g, sms, stream);
                default: return BQ_STATUS_INVALID_PROBLEM;
            }
        }
    }
    switch (bn) {
        case 256: return launch_config<KIND, RAW, 256, 4>(g, sms, stream);
        case 128: return launch_config<KIND, RAW, 128, 6>(g, sms, stream);
        case 64: return launch_config<KIND, RAW, 64, 8>(g, sms, stream);
        default: return BQ_STATUS_INVALID_PROBLEM;
    }
}

}  // namespace

int32_t launch_gemm_q8(const GemmDesc& g, cudaStream_t stream) {
    if (g.k == 0) {
        const int n_out = (g.swiglu && !g.raw_out) ? g.n / 2 : g.n;  // silu(0) * 0 = 0
        const int64_t total = static_cast<int64_t>(g.m) * n_out;
        const int blocks = static_cast<int>((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        if (g.raw_out) {
            fill_zero_kernel<uint32_t><<<blocks, 256, 0, stream>>>(static_cast<uint32_t*>(g.d), g.ldd, g.m, g.n);
        } else {
            fill_zero_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(g.d), g.ldd,
                                                                        g.m, n_out);
        }
        return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
    }
    if (g.kind == BQ_KIND_S8) {
        return g.raw_out ? launch_kind<UMMA_KIND_I8, true>(g, stream) : launch_kind<UMMA_KIND_I8, false>(g, stream);
    }
    return g.raw_out ? launch_kind<UMMA_KIND_F8, true>(g, stream) : launch_kind<UMMA_KIND_F8, false>(g, stream);
}

int sm_count_of_current_device() { return sm_count_impl(); }

bool gemm_q8_takes_cluster_split_k(const GemmDesc& g) {
    const int sms = sm_count_impl();
    return sms > 0 && g.k > 0 && !g.raw_out && cluster_split_choice(g, sms).slices > 1;
}

bool make_mnmajor_tensor_map(void* map_out, const void* base, int64_t k_rows, int64_t n_cols, int64_t ld, int box_k,
                             int l2_promotion) {
    auto enc = tensor_map_encoder();
    if (!enc) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(n_cols), static_cast<cuuint64_t>(k_rows)};
    cuuint64_t pitch = static_cast<cuuint64_t>(k_rows > 1 ? ld : ((n_cols + 15) / 16) * 16);
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_k)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(static_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     static_cast<CUtensorMapL2promotion>(l2_promotion), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_kmajor_tensor_map(void* map_out, const void* base, int64_t rows, int64_t k, int64_t ld, int box_rows) {
    return make_kmajor_map(static_cast<CUtensorMap*>(map_out), base, rows, k, ld, box_rows);
}

int32_t read_and_clear_gemm_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_gemm_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
