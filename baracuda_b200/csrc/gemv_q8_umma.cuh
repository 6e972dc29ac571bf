// Decode GEMV for row-major weights [K, N] (N contiguous, the layout of the reference's GEMV:
// crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:101-343) on the 5th-generation tensor cores.
//
// A weight tile [128 K-rows x 128 N-bytes] lands in shared memory by one tensor copy with the 128-byte swizzle and is
// consumed *as it lies* by tcgen05.mma as an MN-major B operand: no transposition in registers, which is what kept the
// mma.sync streaming kernel at 40 % of the memory rate.  The m <= 8 activation rows are the first eight rows of a
// 64-row K-major A tile whose other rows stay zero; the 64 x 128 accumulator lives in tensor memory (two buffers).
//
// CTAs work in teams of `gu_team` neighbours: a team streams a strip of gu_team adjacent column tiles, member j its
// own [128 K-rows x 128 columns] tile of the strip, all members walking the same K blocks at the same time so that the
// team's concurrent copies cover long contiguous runs of each weight row (isolated 128-byte runs stream from DRAM at
// two thirds of the rate).  Work is cut into units of one [128 K-rows x strip] slab, numbered strip major; team g of
// G owns units [g * U / G, (g + 1) * U / G): every SM streams the same number of bytes, whatever N and K are.  A run
// crosses at most a few strips; for each (a "segment") a member accumulates over its K blocks and writes the m partial
// rows to its own slot of a workspace; a second kernel, chained with programmatic dependent launch, adds the slots of
// a column tile, applies scales / alpha / beta and stores.  Roles: warp 0 epilogue (tensor-memory lanes 0..31 hold
// accumulator rows 0..15), warp 1 owns tensor memory and issues the MMAs, warp 2 is the copy producer.
// Included by gemv_q8_sm100a.cu inside its anonymous namespace.

constexpr int GU_TN = 128;                     // columns per unit
constexpr int GU_BK = 128;                     // K rows per unit
constexpr int GU_M = 64;                       // MMA rows; rows m..63 of the A tile are zero
constexpr int GU_A_BYTES = GU_M * 128;         // 8 KiB, of which the first 1 KiB (rows 0..7) is rewritten per unit
constexpr int GU_X_BYTES = 8 * 128;
constexpr int GU_B_BYTES = GU_BK * GU_TN;      // 16 KiB
constexpr int GU_STAGE_BYTES = GU_A_BYTES + GU_B_BYTES;
constexpr int GU_STAGES = 4;                   // 64 KiB of weights in flight per CTA, two CTAs per SM
constexpr int GU_THREADS = 96;
constexpr int GU_TMEM_COLS = 256;              // two accumulators of 128 columns
constexpr int GU_SMEM = GU_STAGES * GU_STAGE_BYTES + (2 * GU_STAGES + 4) * 8 + 16 + 1024;
constexpr long long GU_WAIT_LIMIT = 1LL << 31;

__device__ __forceinline__ void gu_timeout(volatile uint32_t* abort_word, int code) {
    *abort_word = 1u;
    atomicCAS(&g_gemv_device_status, 0, code);
}

__global__ void __launch_bounds__(GU_THREADS, 2)
gemv_q8_rrr_umma_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_b,
                        const GemvParams p) {
    extern __shared__ uint8_t gu_smem_raw[];
    uint8_t* smem = gu_smem_raw + ((1024u - (smem_u32(gu_smem_raw) & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + GU_STAGES * GU_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + GU_STAGES;
    uint64_t* tfull_bar = empty_bar + GU_STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.gu_kblocks;
    const int64_t units = p.gu_units;
    const int team_size = p.gu_team;
    const int team = blockIdx.x / team_size;
    const int member = blockIdx.x - team * team_size;
    const int teams = gridDim.x / team_size;
    const int64_t u0 = static_cast<int64_t>(team) * units / teams;
    const int64_t u1 = static_cast<int64_t>(team + 1) * units / teams;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GU_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);
            mbar_init(&tempty_bar[b], 1);
        }
        *abort_word = 0u;
        fence_barrier_init();
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_b);
    }
    // rows 8..63 of every stage's A tile are zero for the whole launch
    for (int i = threadIdx.x; i < GU_STAGES * ((GU_A_BYTES - GU_X_BYTES) / 16); i += GU_THREADS) {
        const int s = i / ((GU_A_BYTES - GU_X_BYTES) / 16);
        const int o = i - s * ((GU_A_BYTES - GU_X_BYTES) / 16);
        reinterpret_cast<uint4*>(smem + s * GU_STAGE_BYTES + GU_X_BYTES)[o] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
    if (warp == 1) {
        tmem_alloc(tmem_slot, GU_TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 2) {
        if (lane == 0) {
            // the weights do not depend on the previous kernel of the stream: request them before the dependency wait
            const int64_t run = u1 - u0;
            const int pre = run < GU_STAGES ? static_cast<int>(run) : GU_STAGES;
            for (int s = 0; s < pre; ++s) {
                const int64_t u = u0 + s;
                const int strip = static_cast<int>(u / kblocks), kb = static_cast<int>(u - static_cast<int64_t>(strip) * kblocks);
                const int t = strip * team_size + member;  // beyond the last column tile the copy reads zeros
                mbar_arrive_expect_tx(&full_bar[s], GU_X_BYTES + GU_B_BYTES);
                tma_load_2d(smem + s * GU_STAGE_BYTES + GU_A_BYTES, &tmap_b, &full_bar[s], t * GU_TN, kb * GU_BK);
            }
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int s = 0; s < pre; ++s) {
                const int64_t u = u0 + s;
                const int kb = static_cast<int>(u % kblocks);
                tma_load_2d(smem + s * GU_STAGE_BYTES, &tmap_x, &full_bar[s], kb * GU_BK, 0);
            }
            int stage = pre == GU_STAGES ? 0 : pre;
            uint32_t phase = pre == GU_STAGES ? 1u : 0u;
            for (int64_t u = u0 + pre; u < u1; ++u) {
                if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_word, GU_WAIT_LIMIT)) {
                    gu_timeout(abort_word, 131);
                    break;
                }
                const int strip = static_cast<int>(u / kblocks), kb = static_cast<int>(u - static_cast<int64_t>(strip) * kblocks);
                const int t = strip * team_size + member;
                mbar_arrive_expect_tx(&full_bar[stage], GU_X_BYTES + GU_B_BYTES);
                tma_load_2d(smem + stage * GU_STAGE_BYTES + GU_A_BYTES, &tmap_b, &full_bar[stage], t * GU_TN, kb * GU_BK);
                tma_load_2d(smem + stage * GU_STAGE_BYTES, &tmap_x, &full_bar[stage], kb * GU_BK, 0);
                if (++stage == GU_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(UMMA_KIND_I8, GU_M, GU_TN, true);
            int stage = 0;
            uint32_t phase = 0;
            int seg = 0;
            bool ok = true;
            for (int64_t u = u0; ok && u < u1; ++seg) {
                const int kb0 = static_cast<int>(u % kblocks);
                const int64_t left = u1 - u;
                const int cnt = left < kblocks - kb0 ? static_cast<int>(left) : kblocks - kb0;
                const int buf = seg & 1;
                if (!mbar_wait_bounded(&tempty_bar[buf], ((seg >> 1) & 1) ^ 1u, abort_word, GU_WAIT_LIMIT)) {
                    gu_timeout(abort_word, 132);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * GU_TN);
                for (int i = 0; i < cnt; ++i) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, abort_word, GU_WAIT_LIMIT)) {
                        gu_timeout(abort_word, 133);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + stage * GU_STAGE_BYTES);
                    const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_mnmajor_sw128(a_addr + GU_A_BYTES, GU_B_BYTES, 1024);
#pragma unroll
                    for (int ks = 0; ks < GU_BK / 32; ++ks) {
                        const uint64_t koff = static_cast<uint64_t>((ks * 32) >> 4);
                        const uint64_t boff = static_cast<uint64_t>((ks * 32 * 128) >> 4);  // four 1024-byte atoms down
                        umma_ss<UMMA_KIND_I8>(d_tmem, a_desc + koff, b_desc + boff, idesc, (i | ks) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == GU_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(&tfull_bar[buf]);
                u += cnt;
            }
        }
    } else {
        // warp 0: accumulator rows 0..15 sit in tensor-memory lanes 0..15; lane r < m writes partial row r
        int seg = 0;
        for (int64_t u = u0; u < u1; ++seg) {
            const int kb0 = static_cast<int>(u % kblocks);
            const int64_t left = u1 - u;
            const int cnt = left < kblocks - kb0 ? static_cast<int>(left) : kblocks - kb0;
            const int buf = seg & 1;
            if (!mbar_wait_bounded(&tfull_bar[buf], (seg >> 1) & 1, abort_word, GU_WAIT_LIMIT)) {
                gu_timeout(abort_word, 134);
                break;
            }
            tc_fence_after_sync();
            int32_t* dst = p.gu_partials +
                           ((static_cast<int64_t>(blockIdx.x) * p.gu_smax + seg) * p.m + lane) * GU_TN;
#pragma unroll
            for (int c = 0; c < GU_TN / 32; ++c) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld_32x32b_x32(tmem_base + static_cast<uint32_t>(buf * GU_TN + c * 32), r);
                tmem_ld_wait();
                if (lane < p.m) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        reinterpret_cast<uint4*>(dst + c * 32)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[buf]);
            u += cnt;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_word != 0u) {  // a wait ran out: give copies and MMAs in flight time to land before the CTA leaves
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, GU_TMEM_COLS);
    }
}

// Start of CTA c's run of units, and the CTA that owns unit u (the largest c with start(c) <= u).
__device__ __forceinline__ int64_t gu_start(int c, int64_t units, int ctas) { return static_cast<int64_t>(c) * units / ctas; }
__device__ __forceinline__ int gu_owner(int64_t u, int64_t units, int ctas) {
    int c = static_cast<int>((u * ctas) / units);
    while (c + 1 < ctas && gu_start(c + 1, units, ctas) <= u) ++c;
    while (c > 0 && gu_start(c, units, ctas) > u) --c;
    return c;
}

// Adds the partial rows of the CTAs that shared a column tile and stores the result: one block per column tile and
// activation row, one thread per column.
template <bool RAW>
__global__ void __launch_bounds__(GU_TN)
gemv_q8_rrr_umma_reduce_kernel(const GemvParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the partial rows are complete and visible
    const int t = blockIdx.x;
    const int r = blockIdx.y;
    const int col = t * GU_TN + threadIdx.x;
    const int kblocks = p.gu_kblocks;
    const int64_t units = p.gu_units;
    const int teams = p.gu_ctas / p.gu_team;
    const int strip = t / p.gu_team;
    const int member = t - strip * p.gu_team;
    const int64_t first = static_cast<int64_t>(strip) * kblocks;
    const int c_lo = gu_owner(first, units, teams);
    const int c_hi = gu_owner(first + kblocks - 1, units, teams);
    if (col >= p.n) return;
    int sum = 0;
    for (int c = c_lo; c <= c_hi; ++c) {
        // a team's segments are numbered from the strip its run starts in; empty runs own nothing
        const int64_t s0 = gu_start(c, units, teams);
        if (gu_start(c + 1, units, teams) == s0) continue;
        const int seg = strip - static_cast<int>(s0 / kblocks);
        const int64_t cta = static_cast<int64_t>(c) * p.gu_team + member;
        sum += __ldcg(p.gu_partials + ((cta * p.gu_smax + seg) * p.m + r) * GU_TN + threadIdx.x);
    }
    store_result<RAW>(p, 0, r, col, sum);
}

struct GuPlan {
    bool ok = false;
    int ctas = 0, kblocks = 0, smax = 0, team = 0;
    int64_t units = 0;
    size_t ws_bytes = 0;
};

// Served: one batch slot, m <= 8, 16-byte aligned operands and pitches (the tensor copies), enough units to give
// every SM work.  The workspace holds ctas x smax partial tiles of m x 128 sums.
GuPlan plan_rrr_umma(int m, int n, int k, int sms, int team) {
    GuPlan pl;
    if (m < 1 || m > 8 || n < 1 || k < 1 || sms < 1) return pl;
    pl.kblocks = (k + GU_BK - 1) / GU_BK;
    const int64_t tiles = (n + GU_TN - 1) / GU_TN;
    while (team > 1 && (team > tiles || team > sms)) team >>= 1;
    pl.team = team;
    const int64_t strips = (tiles + team - 1) / team;
    pl.units = strips * pl.kblocks;
    int64_t teams = sms / team;
    if (pl.units < teams) teams = pl.units;
    pl.ctas = static_cast<int>(teams) * team;
    const int64_t run_max = (pl.units + teams - 1) / teams;
    pl.smax = static_cast<int>((run_max + pl.kblocks - 1) / pl.kblocks) + 1;
    pl.ws_bytes = static_cast<size_t>(pl.ctas) * pl.smax * m * GU_TN * sizeof(int32_t);
    pl.ok = true;
    return pl;
}

template <bool RAW>
int32_t launch_rrr_umma(GemvParams p, const GuPlan& pl, const GemvDesc& gd, cudaStream_t stream) {
    CUtensorMap map_x, map_b;
    if (!make_kmajor_tensor_map(&map_x, p.a, p.m, p.k, p.m > 1 ? p.lda : ((p.k + 15) / 16) * 16, 8))
        return BQ_STATUS_LAUNCH_FAILURE;
    // weights are read once: 128-byte L2 promotion measures 1-3 % faster than the 256-byte setting the GEMMs use
    if (!make_mnmajor_tensor_map(&map_b, p.b, p.k, p.n, p.ldb, GU_BK, 2)) return BQ_STATUS_LAUNCH_FAILURE;
    p.gu_kblocks = pl.kblocks;
    p.gu_units = pl.units;
    p.gu_smax = pl.smax;
    p.gu_ctas = pl.ctas;
    p.gu_team = pl.team;
    p.gu_partials = static_cast<int32_t*>(gd.workspace);
    auto kern = gemv_q8_rrr_umma_kernel;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GU_SMEM) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.ctas, 1, 1);
    cfg.blockDim = dim3(GU_THREADS, 1, 1);
    cfg.dynamicSmemBytes = GU_SMEM;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, map_x, map_b, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    cudaLaunchConfig_t rcfg = {};
    rcfg.gridDim = dim3((p.n + GU_TN - 1) / GU_TN, p.m, 1);
    rcfg.blockDim = dim3(GU_TN, 1, 1);
    rcfg.stream = stream;
    rcfg.attrs = attr;
    rcfg.numAttrs = 1;  // may be scheduled while the streaming kernel runs; it waits for it on the device
    if (cudaLaunchKernelEx(&rcfg, gemv_q8_rrr_umma_reduce_kernel<RAW>, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}
