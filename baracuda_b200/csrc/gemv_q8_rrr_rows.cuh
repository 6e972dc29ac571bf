// Decode GEMV for row-major weights [K, N] (N contiguous, the layout of the reference's GEMV:
// crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:101-343), fed by 1-D bulk copies of long row runs.
//
// Every weight row is contiguous along N, so the cheapest way to bring the matrix in is the way the K-contiguous
// kernels do it: cp.async.bulk of whole 1 KiB runs of one row, which stream from HBM at the copy rate (tiled tensor
// copies of 128-byte-wide boxes reach less than half of it on this layout).  A run of one row holds ONE K value of
// 1024 columns, though, while the integer tensor-core instruction wants four consecutive K values of one column per
// register.  ldmatrix .m16n16 .trans .b8 does exactly that transposition on the way from shared memory to registers:
// a 16 (K) x 16 (N) byte block read with .trans arrives as B fragments of mma.sync m16n8k16/k32 (lane (g, t) gets K
// 4t..4t+3 of columns g and g + 8), so no byte permutes are spent.
//
// The matrix is seen as a list of 1 KiB row pieces, strip major (a strip = 1024 columns, all K); CTA c of G owns pieces
// [c * R / G, (c + 1) * R / G): every SM streams the same bytes to within one piece.  A CTA walks its pieces in stages
// of up to 32 K-rows of one strip.  Two producer warps keep six stages in flight (lane i copies row i of a stage,
// completion counted in bytes on the stage's barrier; a single issuing warp was the bottleneck: 22.5 us against
// 15.4 us), sixteen consumer warps each own 64 columns of the strip: wait for the stage, four ldmatrix, hand the stage
// back, eight MMAs against the activation fragments (rows m..7 of the 8-row A tile and K rows the stage does not have
// are zero).  Sums stay in registers until the strip changes or the run ends, then go to the CTA's partial rows in
// the caller's scratch (slot = cta + strip: no atomics, nothing to clear); a second small kernel, chained with
// programmatic dependent launch, adds the partial rows of every strip and applies scales / alpha / beta.  Every wait
// is bounded (status 206 / 207).
// Included by gemv_q8_sm100a.cu inside its anonymous namespace.

constexpr int RR_COLS = 1024;                 // columns per strip = bytes per bulk copy
constexpr int RR_UK = 32;                     // K rows per stage = K of one mma.sync
constexpr int RR_WARP_COLS = 64;              // columns per consumer warp
constexpr int RR_WARPS = RR_COLS / RR_WARP_COLS;  // 16 consumer warps
constexpr int RR_PRODUCERS = 2;               // copy-issuing warps: one warp issuing every copy measured 22.5 us, two 15.4 us, four 15.3 us
constexpr int RR_THREADS = (RR_WARPS + RR_PRODUCERS) * 32;
constexpr int RR_PITCH = RR_COLS + 16;        // row pitch in shared memory: the 16 rows of an ldmatrix hit the 8 16-byte bank groups twice
constexpr int RR_STAGE_BYTES = RR_UK * RR_PITCH;
constexpr int RR_STAGES = (200 * 1024) / RR_STAGE_BYTES;  // 6 stages: 192 KiB of weights in flight per SM
constexpr int RR_MAX_CTAS = 160;              // sizes the scratch without asking the device
constexpr int RR_MAX_RUN = 96;                // stages per CTA the activation staging holds (24 KiB)
constexpr long long RR_WAIT_LIMIT = 1LL << 31;

__device__ __forceinline__ void ldmatrix_b8_16x16_x2_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// Upper bound of the scratch over every device this library meets: RR_MAX_CTAS CTAs, or, for matrices that need
// several waves of CTAs, one CTA per (RR_MAX_RUN - 3) * 32 row pieces plus two waves of slack.
size_t rrr_rows_workspace_bytes(int m, int n, int k, int batch) {
    const int64_t strips = (n + RR_COLS - 1) / RR_COLS;
    const int64_t rows_total = strips * k;
    const int64_t by_length = rows_total / ((RR_MAX_RUN - 3) * RR_UK) + 2 * RR_MAX_CTAS;
    const int64_t ctas = rows_total <= static_cast<int64_t>(128) * (RR_MAX_RUN - 3) * RR_UK ? RR_MAX_CTAS : by_length;
    return static_cast<size_t>(batch) * static_cast<size_t>(ctas + strips) * m * RR_COLS * sizeof(int32_t);
}

struct RrPlan {
    bool ok = false;
    int strips = 0, ctas = 0, run_max = 0, slots_total = 0;
    int64_t rows_total = 0;
    size_t smem = 0, ws_bytes = 0;
};

// Shape of the run for the current device.  Served: any m <= 8, N a multiple of 16, 16-byte aligned rows.
RrPlan plan_rrr_rows(int m, int n, int k, int batch, int sms) {
    RrPlan pl;
    if (sms <= 0 || m <= 0 || n <= 0 || k <= 0 || batch <= 0) return pl;
    pl.strips = (n + RR_COLS - 1) / RR_COLS;
    pl.rows_total = static_cast<int64_t>(pl.strips) * k;  // rows of RR_COLS bytes, strip major
    // one CTA per SM; matrices too long for one CTA's activation staging take whole further waves of CTAs
    const int per_wave = sms < RR_MAX_CTAS ? sms : RR_MAX_CTAS;
    int64_t ctas = pl.rows_total < per_wave ? pl.rows_total : per_wave;
    int64_t run_max = 0;
    for (int wave = 1; wave <= 64; ++wave) {
        if (wave > 1) ctas = static_cast<int64_t>(wave) * per_wave;
        const int64_t rows_per_cta = (pl.rows_total + ctas - 1) / ctas;
        // stages of up to 32 rows that never straddle a strip: full stages, one tail, one more per strip boundary crossed
        run_max = (rows_per_cta + RR_UK - 1) / RR_UK + (rows_per_cta + k - 1) / k + 1;
        if (run_max <= RR_MAX_RUN) break;
    }
    if (run_max > RR_MAX_RUN) return pl;
    pl.ctas = static_cast<int>(ctas);
    pl.run_max = static_cast<int>(run_max);
    pl.slots_total = pl.ctas + pl.strips;
    pl.smem = 128 + static_cast<size_t>(RR_STAGES) * RR_STAGE_BYTES + static_cast<size_t>(run_max) * (8 * RR_UK + 16) +
              2 * RR_STAGES * 8 + 64;
    pl.ws_bytes = static_cast<size_t>(batch) * pl.slots_total * m * RR_COLS * sizeof(int32_t);
    pl.ok = pl.ws_bytes <= rrr_rows_workspace_bytes(m, n, k, batch);  // what *_workspace_size promised the caller
    return pl;
}

// CTA c of G owns rows [c * R / G, (c + 1) * R / G) of the strip-major row list (R = strips x K): every SM streams the
// same number of bytes to within one row.
__device__ __forceinline__ int64_t rr_begin(int c, int64_t rows_total, int ctas) {
    return (static_cast<int64_t>(c) * rows_total) / ctas;
}

__global__ void __launch_bounds__(RR_THREADS, 1)
gemv_q8_rrr_rows_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t rr_smem_raw[];
    uint8_t* smem = rr_smem_raw + ((128u - (smem_u32(rr_smem_raw) & 127u)) & 127u);
    uint8_t* ring = smem;
    uint8_t* xs = smem + RR_STAGES * RR_STAGE_BYTES;                                    // [stage of the run][8 rows][32 bytes]
    int4* sched = reinterpret_cast<int4*>(xs + static_cast<size_t>(p.rr_run_max) * 8 * RR_UK);  // (strip, k0, rows, -) per stage
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sched + p.rr_run_max);
    uint64_t* empty_bar = full_bar + RR_STAGES;
    volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(empty_bar + RR_STAGES);
    volatile int* run_len = reinterpret_cast<volatile int*>(abort_word + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t g = blockIdx.y;
    const int64_t row_begin = rr_begin(blockIdx.x, p.rr_rows_total, gridDim.x);
    const int64_t row_end = rr_begin(blockIdx.x + 1, p.rr_rows_total, gridDim.x);
    const int8_t* b = p.b + g * p.stride_b;

    if (threadIdx.x == 0) {
        *abort_word = 0u;
        for (int s = 0; s < RR_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], RR_WARPS);
        }
        fence_barrier_init();
        fence_proxy_async_smem();
        // this CTA's stages: up to 32 rows of one strip each
        int t = 0;
        for (int64_t pos = row_begin; pos < row_end && t < p.rr_run_max; ++t) {
            const int strip = static_cast<int>(pos / p.k);
            const int k0 = static_cast<int>(pos - static_cast<int64_t>(strip) * p.k);
            int rows = p.k - k0 < RR_UK ? p.k - k0 : RR_UK;
            if (row_end - pos < rows) rows = static_cast<int>(row_end - pos);
            sched[t] = make_int4(strip, k0, rows, 0);
            pos += rows;
        }
        *run_len = t;
    }
    __syncthreads();
    const int run = *run_len;

    if (warp >= RR_WARPS) {
        // ---- producers: warp pi issues the stages t = pi, pi + 2, ...; lane i copies row i of the stage
        const int pi = warp - RR_WARPS;
        auto issue = [&](int t) {
            const int4 sc = sched[t];
            const int slot = t % RR_STAGES;
            const int col0 = sc.x * RR_COLS;
            const uint32_t bytes = static_cast<uint32_t>((p.n - col0 < RR_COLS) ? (p.n - col0) : RR_COLS);
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[slot], bytes * static_cast<uint32_t>(sc.z));
            __syncwarp();
            if (lane < sc.z) {  // rows the stage does not have meet zero activations
                bulk_load_1d(ring + slot * RR_STAGE_BYTES + lane * RR_PITCH, b + static_cast<int64_t>(sc.y + lane) * p.ldb + col0, bytes,
                             &full_bar[slot]);
            }
        };
        // the weights do not depend on the previous kernel of the stream: request them before anything else
        const int pre = run < RR_STAGES ? run : RR_STAGES;
        for (int t = pi; t < pre; t += RR_PRODUCERS) issue(t);
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        bool ok = true;
        int t0 = pre;
        while (t0 % RR_PRODUCERS != pi) ++t0;
        for (int t = t0; ok && t < run; t += RR_PRODUCERS) {
            const int slot = t % RR_STAGES;
            const uint32_t parity = static_cast<uint32_t>((t / RR_STAGES) - 1) & 1u;
            if (lane == 0 && !mbar_wait_bounded(&empty_bar[slot], parity, abort_word, RR_WAIT_LIMIT)) {
                *abort_word = 1u;
                atomicCAS(&g_gemv_device_status, 0, 206);
                ok = false;
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (ok) issue(t);
        }
    } else {
        // ---- consumers: warp w owns columns [64 w, 64 w + 64) of the current strip
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
        // this run's activations: stage t holds x[r][k0 .. k0 + 32) for r < 8, zero beyond m and beyond the stage's rows
        {
            const int8_t* a = p.a + g * p.stride_a;
            for (int i = threadIdx.x; i < run * 64; i += RR_WARPS * 32) {
                const int t = i >> 6, r = (i >> 3) & 7, w = i & 7;
                const int4 sc = sched[t];
                uint32_t word = 0;
                if (r < p.m) {
                    const int8_t* src = a + static_cast<int64_t>(r) * p.lda + sc.y + 4 * w;
                    if (4 * w + 4 <= sc.z && (reinterpret_cast<uintptr_t>(src) & 3u) == 0) {
                        word = __ldg(reinterpret_cast<const uint32_t*>(src));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (4 * w + j < sc.z) word |= static_cast<uint32_t>(static_cast<uint8_t>(__ldg(src + j))) << (8 * j);
                        }
                    }
                }
                reinterpret_cast<uint32_t*>(xs)[i] = word;
            }
        }
        named_bar_sync(1, RR_WARPS * 32);

        const int g8 = lane >> 2, t4 = lane & 3;
        int acc[8][2];  // n-group j: columns 8 j + 2 t4, 8 j + 2 t4 + 1 of this warp's 64, activation row g8
        auto clear = [&]() {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = 0;
        };
        int cur_strip = -1;
        auto finish_strip = [&]() {
            if (g8 < p.m) {
                int32_t* dst = p.rr_partials +
                               ((g * p.rr_slots_total + blockIdx.x + cur_strip) * static_cast<int64_t>(p.m) + g8) * RR_COLS +
                               warp * RR_WARP_COLS + 2 * t4;
#pragma unroll
                for (int j = 0; j < 8; ++j) __stcg(reinterpret_cast<int2*>(dst + 8 * j), make_int2(acc[j][0], acc[j][1]));
            }
        };
        // lane L addresses row L of the stage: rows 0..15 feed the first 16 x 16 matrix of an ldmatrix.x2, 16..31 the second
        const uint32_t lane_off = static_cast<uint32_t>(lane * RR_PITCH + warp * RR_WARP_COLS);
        const uint32_t ring_addr = smem_u32(ring);
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs);
        bool ok = true;
        for (int t = 0; t < run; ++t) {
            const int strip = sched[t].x;
            if (strip != cur_strip) {
                if (cur_strip >= 0) finish_strip();
                cur_strip = strip;
                clear();
            }
            const int slot = t % RR_STAGES;
            if (!mbar_wait_bounded(&full_bar[slot], static_cast<uint32_t>((t / RR_STAGES) & 1), abort_word, RR_WAIT_LIMIT)) {
                *abort_word = 1u;
                atomicCAS(&g_gemv_device_status, 0, 207);
                ok = false;
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const uint32_t base = ring_addr + static_cast<uint32_t>(slot * RR_STAGE_BYTES) + lane_off;
            uint32_t f[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) ldmatrix_b8_16x16_x2_trans(f[c], base + 16u * c);
            const uint32_t a0 = xw[(t * 8 + g8) * 8 + t4];
            const uint32_t a2 = xw[(t * 8 + g8) * 8 + 4 + t4];
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot]);  // the stage now lives in registers
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                mma_s8_16x8x32_top(acc[2 * c][0], acc[2 * c][1], a0, a2, f[c][0], f[c][2]);
                mma_s8_16x8x32_top(acc[2 * c + 1][0], acc[2 * c + 1][1], a0, a2, f[c][1], f[c][3]);
            }
        }
        if (ok && cur_strip >= 0) finish_strip();
    }
    // on the error path give copies still in flight a bounded time to land before the CTA's shared memory goes away
    __syncthreads();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
}

// Adds the partial rows of the CTAs that shared a strip and stores the result (scales, alpha, beta applied): one thread
// per column, every activation row, all loads of a column requested before the first is used.  128 columns per block
// and a grid no larger than the SM count, so that with programmatic dependent launch every block is already resident
// beside a streaming CTA when the streaming kernel ends (a grid of one block per column tile AND row cost 3 us more at
// m >= 4, where its second wave had to wait for the first).
constexpr int RR_REDUCE_THREADS = 128;

// MR: activation rows rounded up to 1, 2, 4 or 8; a thread keeps 16 (MR <= 2) or 32 loads in flight, so a strip shared
// by a dozen CTAs costs one round trip to L2 and one shared by forty (few strips, long K) three.
template <bool RAW, int MR>
__global__ void __launch_bounds__(RR_REDUCE_THREADS)
gemv_q8_rrr_rows_reduce_kernel(const GemvParams p) {
    constexpr int U = MR <= 2 ? 16 / MR * (MR == 2 ? 2 : 1) : 32 / MR;  // 16, 16, 8, 4 partial rows per round
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t g = blockIdx.y;
    const int ctas = p.rr_ctas;
    const int64_t total = p.rr_rows_total;
    const int64_t step = static_cast<int64_t>(p.m) * RR_COLS;
    bool waited = false;
    for (int col = blockIdx.x * RR_REDUCE_THREADS + threadIdx.x; col < p.n; col += gridDim.x * RR_REDUCE_THREADS) {
        const int strip = col / RR_COLS;
        const int in_strip = col - strip * RR_COLS;
        // the CTA that owns piece q of the strip-major list is the largest c with c * total < (q + 1) * ctas
        const int c_lo = static_cast<int>(((static_cast<int64_t>(strip) * p.k + 1) * ctas - 1) / total);
        const int c_hi = static_cast<int>(((static_cast<int64_t>(strip + 1) * p.k) * ctas - 1) / total);
        const int32_t* base = p.rr_partials + (g * p.rr_slots_total + strip) * step + in_strip;
        if (!waited) {  // the index arithmetic above runs while the streaming kernel is still at work
            asm volatile("griddepcontrol.wait;" ::: "memory");  // its partial rows are complete and visible
            waited = true;
        }
        int sum[MR];
#pragma unroll
        for (int r = 0; r < MR; ++r) sum[r] = 0;
        for (int c = c_lo; c <= c_hi; c += U) {
            int v[U][MR];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < MR; ++r)
                    v[u][r] = (c + u <= c_hi && r < p.m) ? __ldcg(base + (c + u) * step + r * RR_COLS) : 0;
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < MR; ++r) sum[r] += v[u][r];
        }
#pragma unroll
        for (int r = 0; r < MR; ++r)
            if (r < p.m) store_result<RAW>(p, g, r, col, sum[r]);
    }
}

template <bool RAW>
int32_t launch_rrr_rows(GemvParams p, int batch, const RrPlan& pl, void* workspace, cudaStream_t stream) {
    p.rr_strips = pl.strips;
    p.rr_run_max = pl.run_max;
    p.rr_ctas = pl.ctas;
    p.rr_slots_total = pl.slots_total;
    p.rr_rows_total = pl.rows_total;
    p.rr_partials = static_cast<int32_t*>(workspace);
    auto kern = gemv_q8_rrr_rows_kernel;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.ctas, batch, 1);
    cfg.blockDim = dim3(RR_THREADS, 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    // the reduction may be scheduled while the streaming kernel runs; it waits for it on the device
    cudaLaunchConfig_t rcfg = {};
    const int want = (p.n + RR_REDUCE_THREADS - 1) / RR_REDUCE_THREADS;
    rcfg.gridDim = dim3(want < pl.ctas ? want : pl.ctas, batch, 1);
    rcfg.blockDim = dim3(RR_REDUCE_THREADS, 1, 1);
    rcfg.stream = stream;
    rcfg.attrs = attr;
    rcfg.numAttrs = 1;
    auto rkern = p.m <= 1 ? gemv_q8_rrr_rows_reduce_kernel<RAW, 1>
                          : (p.m <= 2 ? gemv_q8_rrr_rows_reduce_kernel<RAW, 2>
                                      : (p.m <= 4 ? gemv_q8_rrr_rows_reduce_kernel<RAW, 4> : gemv_q8_rrr_rows_reduce_kernel<RAW, 8>));
    if (cudaLaunchKernelEx(&rcfg, rkern, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}
