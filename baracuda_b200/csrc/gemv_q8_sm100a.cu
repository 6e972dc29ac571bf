// Skinny int8 GEMV for decode (m = 1..8 activation rows), HBM-bandwidth bound:
//   D[g, r, j] = bf16( alpha * (sa[r]*sb[j]) * sum_k A[g,r,k] * B[g,k,j] + beta * D[g,r,j] )
// or the raw int32 sums.  The weight matrix is streamed exactly once.  Kernels, in the order the dispatcher tries them:
//   gemv_q8_rcr_mma_kernel      weights [N, K], m >= 2 (and m = 1 under dependent launch): bulk copies, mma.sync
//   gemv_q8_rcr_stream_kernel   weights [N, K], m <= 4: bulk copies, dp4a + warp shuffles
//   gemv_q8_rrr_rows_kernel     weights [K, N]: 1 KiB bulk copies of row runs, ldmatrix-transposed fragments, mma.sync;
//                               rows are split over CTAs, partial rows go to the caller's scratch,
//                               gemv_q8_rrr_rows_reduce_kernel adds them (gemv_q8_rrr_rows.cuh)
//   gemv_q8_rcr_kernel / gemv_q8_rrr_kernel   128-bit loads that bypass L1 + dp4a, for shapes the above decline
//   gemv_q8_generic_kernel      byte loads, any alignment
//
// Takes the role of the reference's dense m=1 GEMV
//   crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:101-219 (validation + launcher)
//   crates/baracuda-kernels-sys/kernels/gemm/gemv_dense.cu:128-171 (thread-per-column kernel)
// for int8 weights with the W8A8 dequant of
//   crates/baracuda-kernels-sys/kernels/include/baracuda_quantize_compose.cuh:271-274.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "ptx_sm100a.cuh"

namespace bq {

__device__ int g_gemv_device_status = 0;

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int KB_BYTES = 4096;       // activation bytes per row staged in shared memory at a time
constexpr int RRR_COLS_PER_CTA = 512;  // one warp-wide row segment of 16-byte loads

struct GemvParams {
    const int8_t* a;
    int64_t lda, stride_a;
    const int8_t* b;
    int64_t ldb, stride_b;
    const float* sa;
    int64_t stride_sa;
    const float* sb;
    int64_t stride_sb;
    void* d;
    int64_t ldd, stride_d;
    float alpha, beta;
    int m, n, k;
    // split-K plan of the row-major-weight kernel
    int kslice_rows, num_kslices;
    int32_t* ws_partials;
    unsigned int* ws_tickets;
    // row-major-weight streaming kernel (gemv_q8_rrr_rows.cuh): rr_rows_total 1 KiB row pieces, strip major, over
    // rr_ctas CTAs; rr_run_max = most stages any CTA walks; rr_partials is [batch][rr_slots_total][m][1024],
    // slot(c, strip) = c + strip
    int rr_strips, rr_run_max, rr_ctas, rr_slots_total;
    int64_t rr_rows_total;
    int32_t* rr_partials;
    int mma_groups;  // tensor-core GEMV: 8-column groups per CTA (upper bound), sizes the shared accumulator
    // fused per-token quantiser (XQ kernels): bf16 activations [m, ldx], clamp range, optional scale output [m]
    const __nv_bfloat16* xq_x;
    int64_t xq_ldx;
    int xq_qmin, xq_qmax;
    float* xq_scale_out;
    int pdl;  // launched with programmatic stream serialization: weights may be fetched before the dependency wait
};

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ int dot16(const uint4& w, const uint4& x, int acc) {
    acc = __dp4a(static_cast<int>(w.x), static_cast<int>(x.x), acc);
    acc = __dp4a(static_cast<int>(w.y), static_cast<int>(x.y), acc);
    acc = __dp4a(static_cast<int>(w.z), static_cast<int>(x.z), acc);
    acc = __dp4a(static_cast<int>(w.w), static_cast<int>(x.w), acc);
    return acc;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <bool RAW>
__device__ __forceinline__ void store_result(const GemvParams& p, int64_t batch, int r, int col, int acc) {
    if constexpr (RAW) {
        reinterpret_cast<int32_t*>(p.d)[batch * p.stride_d + static_cast<int64_t>(r) * p.ldd + col] = acc;
    } else {
        __nv_bfloat16* dp =
            reinterpret_cast<__nv_bfloat16*>(p.d) + batch * p.stride_d + static_cast<int64_t>(r) * p.ldd + col;
        const float s = __fmul_rn(__ldg(p.sa + batch * p.stride_sa + r), __ldg(p.sb + batch * p.stride_sb + col));
        float y = __fmul_rn(__fmul_rn(s, static_cast<float>(acc)), p.alpha);
        if (p.beta != 0.0f) y = __fadd_rn(y, __fmul_rn(p.beta, __bfloat162float(*dp)));
        *dp = __float2bfloat16_rn(y);
    }
}

// ---- weights stored [N, K] (K contiguous): one warp owns CPW output columns ----
template <int MR, int CPW, bool RAW>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_q8_rcr_kernel(const GemvParams p) {
    extern __shared__ uint4 xs[];  // MR rows x KB_BYTES/16
    constexpr int KB16 = KB_BYTES / 16;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t g = blockIdx.y;
    const int8_t* a = p.a + g * p.stride_a;
    const int8_t* b = p.b + g * p.stride_b;
    const int col_base = (blockIdx.x * GEMV_WARPS + warp) * CPW;

    int acc[CPW][MR];
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[c][r] = 0;

    const uint4* wrow[CPW];
#pragma unroll
    for (int c = 0; c < CPW; ++c) {
        int col = col_base + c;
        if (col >= p.n) col = p.n - 1;  // clamp; the duplicate result is never stored
        wrow[c] = reinterpret_cast<const uint4*>(b + static_cast<int64_t>(col) * p.ldb);
    }

    for (int k0 = 0; k0 < p.k; k0 += KB_BYTES) {
        const int klen16 = ((p.k - k0 < KB_BYTES) ? (p.k - k0) : KB_BYTES) >> 4;
        __syncthreads();
        for (int i = threadIdx.x; i < MR * klen16; i += GEMV_THREADS) {
            const int r = i / klen16, c = i - r * klen16;
            xs[r * KB16 + c] = __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(r) * p.lda + k0) + c);
        }
        __syncthreads();
        if (col_base < p.n) {
            const int kq = k0 >> 4;
            for (int kk = lane; kk < klen16; kk += 64) {
                const bool second = (kk + 32) < klen16;
                uint4 w0[CPW], w1[CPW];
#pragma unroll
                for (int c = 0; c < CPW; ++c) w0[c] = ldg_stream_v4(wrow[c] + kq + kk);
#pragma unroll
                for (int c = 0; c < CPW; ++c)
                    w1[c] = second ? ldg_stream_v4(wrow[c] + kq + kk + 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int r = 0; r < MR; ++r) {
                    const uint4 x0 = xs[r * KB16 + kk];
                    const uint4 x1 = second ? xs[r * KB16 + kk + 32] : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int c = 0; c < CPW; ++c) {
                        acc[c][r] = dot16(w0[c], x0, acc[c][r]);
                        acc[c][r] = dot16(w1[c], x1, acc[c][r]);
                    }
                }
            }
        }
    }

#pragma unroll
    for (int c = 0; c < CPW; ++c) {
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            const int v = warp_sum(acc[c][r]);
            const int col = col_base + c;
            if (lane == ((c * MR + r) & 31) && col < p.n) store_result<RAW>(p, g, r, col, v);
        }
    }
}

// ---- weights stored [N, K], bulk-copy fed: one persistent CTA per SM, every warp its own
// stream.  Warp w owns the CTA's columns w, w+W, w+2W, ... and a private ring of shared-memory
// slots; its lane 0 keeps the ring full with cp.async.bulk copies of whole weight rows (up to
// 4 KiB of K each, completion counted on an mbarrier), the warp pulls a landed row into
// registers, immediately re-arms the slot with the copy for a later column, then dots the row
// with the activations held in registers (dp4a) and folds the 32 lane sums with shuffles.
// About 190 KiB of weights are in flight per SM regardless of how the warps are scheduled,
// which is what a 9 us HBM-bound kernel needs. ----
constexpr int STREAM_CHUNK = 4096;        // bytes of K per ring slot
constexpr int STREAM_RING_FULL = 196608;  // all warps' rings together, one CTA per SM
constexpr int STREAM_RING_HALF = 98304;   // two CTAs per SM, so the next launch's prologue can overlap this one
constexpr long long STREAM_WAIT_LIMIT = 1LL << 31;

// STREAM_WARPS warps; more activation rows need more registers per thread (the activations
// live in registers), hence fewer warps with deeper rings.
template <int MR, bool RAW, int STREAM_WARPS, int RING_BYTES>
__global__ void __launch_bounds__(STREAM_WARPS * 32, 1)
gemv_q8_rcr_stream_kernel(const GemvParams p) {
    constexpr int STREAM_RING_BYTES = RING_BYTES;
    constexpr int SLOTS = STREAM_RING_BYTES / STREAM_CHUNK / STREAM_WARPS;  // per warp
    extern __shared__ __align__(128) uint8_t stream_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint8_t* ring = stream_smem + warp * SLOTS * STREAM_CHUNK;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(stream_smem + STREAM_RING_BYTES) + warp * SLOTS;
    // one abort word per warp: the warps never meet, so nothing in the prologue needs a CTA-wide barrier
    volatile uint32_t* abort_word =
        reinterpret_cast<volatile uint32_t*>(stream_smem + STREAM_RING_BYTES + STREAM_WARPS * SLOTS * 8) + warp;

    const int64_t g = blockIdx.y;
    const int8_t* a = p.a + g * p.stride_a;
    const int8_t* b = p.b + g * p.stride_b;

    // this CTA's contiguous share of the output columns
    const int ctas = gridDim.x;
    const int base = p.n / ctas, rem = p.n % ctas;
    const int col_begin = blockIdx.x * base + (static_cast<int>(blockIdx.x) < rem ? static_cast<int>(blockIdx.x) : rem);
    const int ncols = base + (static_cast<int>(blockIdx.x) < rem ? 1 : 0);
    const int chunks = (p.k + STREAM_CHUNK - 1) / STREAM_CHUNK;
    // this warp's work items: (its c-th column, K chunk kc), item = c * chunks + kc
    const int my_cols = (ncols > warp) ? (ncols - warp + STREAM_WARPS - 1) / STREAM_WARPS : 0;
    const int my_items = my_cols * chunks;

    if (lane == 0) {
        *abort_word = 0u;
        for (int s = 0; s < SLOTS; ++s) mbar_init(&full_bar[s], 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();

    auto issue = [&](int item) {  // lane 0 only
        const int c = item / chunks, kc = item - c * chunks;
        const int k0 = kc * STREAM_CHUNK;
        const uint32_t bytes = static_cast<uint32_t>((p.k - k0 < STREAM_CHUNK) ? (p.k - k0) : STREAM_CHUNK);
        const int slot = item % SLOTS;
        mbar_arrive_expect_tx(&full_bar[slot], bytes);
        bulk_load_1d(ring + slot * STREAM_CHUNK,
                     b + static_cast<int64_t>(col_begin + warp + c * STREAM_WARPS) * p.ldb + k0, bytes, &full_bar[slot]);
    };
    if (lane == 0) {
        for (int i = 0; i < SLOTS && i < my_items; ++i) issue(i);
    }
    if (p.pdl) {
        // The weights are static, so their first copies are already in flight.  Let the next launch in
        // the stream start its own prologue, then wait until everything before this launch (the producer
        // of the activations, the previous user of the output) has completed and is visible.
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }

    // activations: with a single K chunk every lane keeps its 8 x 16 bytes per row in registers
    uint4 xr[MR][8];
    const bool x_in_regs = (chunks == 1);
    if (x_in_regs) {
#pragma unroll
        for (int r = 0; r < MR; ++r)
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int k16 = s * 32 + lane;
                xr[r][s] = (k16 * 16 < p.k)
                               ? __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(r) * p.lda) + k16)
                               : make_uint4(0, 0, 0, 0);
            }
    }

    // Each warp parks the finished sum of its c-th column in lane (c mod 32) and writes 32 columns
    // at a time, so the scale loads and the stores of the epilogue are paid once per batch, in
    // parallel, instead of once per column on the critical path.
    int keep[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) keep[r] = 0;
    // the scales of the columns this lane will write are fetched now, off the critical path
    float sb_pre = 0.0f, sa_pre[MR];
    if constexpr (!RAW) {
        const int col = col_begin + warp + lane * STREAM_WARPS;
        if (lane < my_cols) sb_pre = __ldg(p.sb + g * p.stride_sb + col);
#pragma unroll
        for (int r = 0; r < MR; ++r) sa_pre[r] = __ldg(p.sa + g * p.stride_sa + r);
    }
    auto flush_batch = [&](int first, int count) {
        if (lane < count) {
            const int col = col_begin + warp + (first + lane) * STREAM_WARPS;
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                if constexpr (RAW) {
                    store_result<RAW>(p, g, r, col, keep[r]);
                } else {
                    const float sbv = (first == 0) ? sb_pre : __ldg(p.sb + g * p.stride_sb + col);
                    __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.d) + g * p.stride_d +
                                        static_cast<int64_t>(r) * p.ldd + col;
                    const float sc = __fmul_rn(sa_pre[r], sbv);
                    float y = __fmul_rn(__fmul_rn(sc, static_cast<float>(keep[r])), p.alpha);
                    if (p.beta != 0.0f) y = __fadd_rn(y, __fmul_rn(p.beta, __bfloat162float(*dp)));
                    *dp = __float2bfloat16_rn(y);
                }
            }
        }
    };
    bool ok = true;
    int done = 0;
    for (int c = 0; ok && c < my_cols; ++c) {
        int acc0[MR], acc1[MR];
#pragma unroll
        for (int r = 0; r < MR; ++r) acc0[r] = acc1[r] = 0;
        for (int kc = 0; kc < chunks; ++kc) {
            const int item = c * chunks + kc;
            const int slot = item % SLOTS;
            const uint32_t parity = (item / SLOTS) & 1;
            if (!mbar_wait_bounded(&full_bar[slot], parity, abort_word, STREAM_WAIT_LIMIT)) {
                *abort_word = 1u;
                atomicCAS(&g_gemv_device_status, 0, 202);
                ok = false;
                break;
            }
            const int k0 = kc * STREAM_CHUNK;
            const int valid16 = ((p.k - k0 < STREAM_CHUNK) ? (p.k - k0) : STREAM_CHUNK) >> 4;
            const uint4* wv = reinterpret_cast<const uint4*>(ring + slot * STREAM_CHUNK);
            uint4 w[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int k16 = s * 32 + lane;
                w[s] = (k16 < valid16) ? wv[k16] : make_uint4(0, 0, 0, 0);
            }
            __syncwarp();  // every lane holds its part of the row: the slot can be refilled
            if (lane == 0 && item + SLOTS < my_items) {
                fence_proxy_async_smem();
                issue(item + SLOTS);
            }
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int k16 = s * 32 + lane;
#pragma unroll
                for (int r = 0; r < MR; ++r) {
                    uint4 x;
                    if (x_in_regs) {
                        x = xr[r][s];
                    } else {
                        x = (k16 < valid16)
                                ? __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(r) * p.lda + k0) + k16)
                                : make_uint4(0, 0, 0, 0);
                    }
                    if (s & 1) {
                        acc1[r] = dot16(w[s], x, acc1[r]);
                    } else {
                        acc0[r] = dot16(w[s], x, acc0[r]);
                    }
                }
            }
        }
        if (!ok) break;
#pragma unroll
        for (int r = 0; r < MR; ++r) {
            const int v = warp_sum(acc0[r] + acc1[r]);
            if (lane == (done & 31)) keep[r] = v;
        }
        ++done;
        if ((done & 31) == 0) flush_batch(done - 32, 32);
    }
    if (ok && (done & 31) != 0) flush_batch(done & ~31, done & 31);
    // on the error path give this warp's copies still in flight a bounded time to land
    __syncwarp();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
}

// ---- weights stored [N, K], several activation rows (m = 2..8): the same per-warp bulk-copy
// streaming, but the dot products run on the tensor cores.  An item is 8 weight rows x 1 KiB of K;
// the warp feeds it to mma.sync m16n8k32 as the B operand (8 output columns), the activations
// (8 rows, zero beyond m) are the A operand read from shared memory, and the instruction itself
// sums over K across the lanes, so no shuffles are needed and the cost per weight byte does not
// grow with m.  Items of one column group that belong to different K chunks (and warps) meet in a
// small shared-memory accumulator. ----
constexpr int MMA_COLS = 8;                    // weight rows (output columns) per item
constexpr int MMA_MAX_GROUPS = 64;             // column groups per CTA the accumulator holds
constexpr int MMA_MAX_K = 8192;

__device__ __forceinline__ void mma_s8_16x8x32(int (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8..15 of A are zero (a1 = a3 = 0): only 8 activation rows exist
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// Same instruction for accumulators that keep only rows 0..7: rows 8..15 start from zero and are dropped, so
// consecutive MMAs share no register.
__device__ __forceinline__ void mma_s8_16x8x32_top(int& c0, int& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    int drop2, drop3;  // written by the instruction, never read
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, {%7, %8}, {%0, %1, %5, %5};"
        : "+r"(c0), "+r"(c1), "=r"(drop2), "=r"(drop3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
    (void)drop2;
    (void)drop3;
}

// MMA_KCHUNK: bytes of K per item and row; MMA_WARPS: streaming warps.  The row pitch in the ring is
// KCHUNK + 64 so that 16-byte reads of 8 rows hit 8 distinct bank groups.
// MMA_RING: items in flight per warp.
// XREG: the number of K chunks divides the number of warps, so a warp meets the same K chunk in all its items and
// keeps its activation fragments in registers (no activation staging, half the shared-memory loads).
// XQ (with XREG): the activations arrive as bf16 and are quantised per token inside the kernel -- every CTA takes the
// absolute maximum of each activation row (m x K bf16 from L2, while the first weight copies are in flight), derives
// scale = absmax / qmax (1.0 for a zero row) and quantises just the fragments its warps keep, with the arithmetic of
// quantize_rows_kernel (multiply by the f32 reciprocal, round half to even, clamp), so the result equals the
// two-kernel path bit for bit and one launch disappears from the decode step.
// XSETS (with XREG): 1 when the number of K chunks divides the number of warps; 2 when it is twice the number of warps, so
// that a warp alternates between two K chunks and keeps two sets of fragments.
template <bool RAW, int MMA_KCHUNK, int MMA_WARPS, int MMA_RING, bool XREG = false, bool XQ = false, int XSETS = 1>
__global__ void __launch_bounds__(MMA_WARPS * 32, 1)
gemv_q8_rcr_mma_kernel(const GemvParams p) {
    static_assert(!XQ || (XREG && XSETS == 1), "the fused quantiser fills one set of register fragments");
    static_assert(XSETS == 1 || XSETS == 2, "one or two K chunks per warp");
    __shared__ float xq_red[XQ ? MMA_WARPS * 8 : 1];
    __shared__ float xq_scale[8];
    // row pitch in the ring chosen so that the 16-byte reads of a quarter-warp (two rows x four pieces) cover all banks
    // (pitch = 64 mod 128 bytes: the two rows of a quarter-warp start 16 banks apart)
    constexpr int MMA_PITCH = (MMA_KCHUNK % 128 == 64) ? MMA_KCHUNK : MMA_KCHUNK + 64;
    constexpr int MMA_ITEM_BYTES = MMA_COLS * MMA_PITCH;
    extern __shared__ __align__(128) uint8_t mma_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int gq = lane >> 2;  // MMA group id: activation row for A and D, weight row (column) for B
    const int tq = lane & 3;
    const int xpitch = p.k + 64;
    uint8_t* ring = mma_smem + warp * MMA_RING * MMA_ITEM_BYTES;
    uint8_t* xs = mma_smem + MMA_WARPS * MMA_RING * MMA_ITEM_BYTES;
    // only the m real activation rows and this launch's groups per CTA take shared memory
    int* acc_s = reinterpret_cast<int*>(xs + (XREG ? 0 : p.m * xpitch));
    float* sb_s = reinterpret_cast<float*>(acc_s + p.mma_groups * 64);  // this CTA's column scales
    uint64_t* bars = reinterpret_cast<uint64_t*>(sb_s + p.mma_groups * MMA_COLS);
    uint64_t* full_bar = bars + warp * MMA_RING;
    volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(bars + MMA_WARPS * MMA_RING) + warp;

    const int64_t g = blockIdx.y;
    const int8_t* a = p.a + g * p.stride_a;
    const int8_t* b = p.b + g * p.stride_b;

    // this CTA's contiguous share of the 8-column groups: whole groups keep every warp's item count
    // equal inside a CTA, which measured faster than balancing single columns across CTAs
    const int total_groups = (p.n + MMA_COLS - 1) / MMA_COLS;
    const int ctas = gridDim.x;
    const int base = total_groups / ctas, rem = total_groups % ctas;
    const int bx = static_cast<int>(blockIdx.x);
    const int group_begin = bx * base + (bx < rem ? bx : rem);
    const int ngroups = base + (bx < rem ? 1 : 0);
    const int col_begin = group_begin * MMA_COLS;
    const int col_end = (col_begin + ngroups * MMA_COLS < p.n) ? (col_begin + ngroups * MMA_COLS) : p.n;
    const int chunks = (p.k + MMA_KCHUNK - 1) / MMA_KCHUNK;
    const int items = ngroups * chunks;
    const int my_items = (items > warp) ? (items - warp + MMA_WARPS - 1) / MMA_WARPS : 0;

    if (lane == 0) {
        *abort_word = 0u;
        for (int s = 0; s < MMA_RING; ++s) mbar_init(&full_bar[s], 1);
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    __syncwarp();

    // whole warp: lane 0 arms the barrier, lanes 0..rows-1 each issue one row's copy (8 copies in one go)
    auto issue = [&](int mine) {  // `mine` counts this warp's items
        const int item = warp + mine * MMA_WARPS;
        const int gi = item / chunks, kc = item - gi * chunks;
        const int k0 = kc * MMA_KCHUNK;
        const uint32_t bytes = static_cast<uint32_t>((p.k - k0 < MMA_KCHUNK) ? (p.k - k0) : MMA_KCHUNK);
        const int col0 = col_begin + gi * MMA_COLS;
        const int rows = (col_end - col0 < MMA_COLS) ? (col_end - col0) : MMA_COLS;
        const int slot = mine % MMA_RING;
        if (lane == 0) {
            fence_proxy_async_smem();
            mbar_arrive_expect_tx(&full_bar[slot], bytes * static_cast<uint32_t>(rows));
        }
        __syncwarp();
        if (lane < rows) {
            bulk_load_1d(ring + slot * MMA_ITEM_BYTES + lane * MMA_PITCH, b + static_cast<int64_t>(col0 + lane) * p.ldb + k0,
                         bytes, &full_bar[slot]);
        }
    };
    // XQ: the last slot's buffer first serves as this warp's staging area for the quantised activations
    for (int i = 0; i < (XQ ? MMA_RING - 1 : MMA_RING) && i < my_items; ++i) issue(i);
    if (p.pdl) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }

    // activations into shared memory (rows beyond m are zero) or, XREG, this warp's K chunk of activation row gq
    // straight into registers in fragment order; accumulators cleared
    uint4 xreg[XREG ? XSETS : 1][XREG ? MMA_KCHUNK / 64 : 1];
    uint4 xraw[XQ ? 8 : 1][2];  // XQ: 16 bf16 values of every activation row, until the row scales are known
    {
        if constexpr (XQ) {
            // This warp's K chunk (MMA_KCHUNK values) of every activation row as bf16, 16 values per lane and row; the
            // sixteen warps' chunks cover every row, so the row maxima come out of the same loads.
            static_assert(MMA_KCHUNK == 512, "16 values per lane and row");
            const int k0 = (warp % chunks) * MMA_KCHUNK;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                float amax = 0.0f;
                if (r < p.m) {
                    const uint4* src = reinterpret_cast<const uint4*>(p.xq_x + static_cast<int64_t>(r) * p.xq_ldx + k0 + lane * 16);
#pragma unroll
                    for (int hv = 0; hv < 2; ++hv) {
                        const uint4 v = __ldg(src + hv);
                        xraw[r][hv] = v;
                        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(h[j]);
                            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                        }
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                }
                if (lane == 0) xq_red[warp * 8 + r] = amax;
            }
        } else if constexpr (XREG) {
#pragma unroll
            for (int xs_i = 0; xs_i < XSETS; ++xs_i) {
                const int k0 = ((warp + xs_i * MMA_WARPS) % chunks) * MMA_KCHUNK;
#pragma unroll
                for (int i = 0; i < MMA_KCHUNK / 64; ++i) {
                    xreg[xs_i][i] = gq < p.m ? __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(gq) * p.lda + k0 + i * 64 + tq * 16))
                                             : make_uint4(0, 0, 0, 0);
                }
            }
        } else {
            const int k16 = p.k >> 4;
            for (int i = threadIdx.x; i < p.m * k16; i += MMA_WARPS * 32) {
                const int r = i / k16, c = i - r * k16;
                *reinterpret_cast<uint4*>(xs + r * xpitch + c * 16) =
                    __ldg(reinterpret_cast<const uint4*>(a + static_cast<int64_t>(r) * p.lda) + c);
            }
        }
        for (int i = threadIdx.x; i < ngroups * 64; i += MMA_WARPS * 32) acc_s[i] = 0;
        if constexpr (!RAW) {  // scales fetched now, off the tail of the kernel
            for (int i = threadIdx.x; i < ngroups * MMA_COLS; i += MMA_WARPS * 32) {
                const int col = col_begin + i;
                sb_s[i] = col < col_end ? __ldg(p.sb + g * p.stride_sb + col) : 0.0f;
            }
        }
    }
    __syncthreads();
    if constexpr (XQ) {
        if (threadIdx.x < p.m) {
            float amax = 0.0f;
            for (int w = 0; w < MMA_WARPS; ++w) amax = fmaxf(amax, xq_red[w * 8 + threadIdx.x]);
            const float sc = (amax > 0.0f) ? __fdiv_rn(amax, static_cast<float>(p.xq_qmax)) : 1.0f;
            xq_scale[threadIdx.x] = sc;
            if (blockIdx.x == 0 && p.xq_scale_out) p.xq_scale_out[threadIdx.x] = sc;
        }
        __syncthreads();
        // quantise the 16 values per row held as bf16 into the staging area (row pitch MMA_KCHUNK bytes), then pick up
        // the fragments: lane (gq, tq) keeps the 16-byte pieces tq, tq + 4, ... of row gq
        uint8_t* stage = ring + (MMA_RING - 1) * MMA_ITEM_BYTES;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < p.m) {
                const float inv = __fdiv_rn(1.0f, xq_scale[r]);
                uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int hv = 0; hv < 2; ++hv) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xraw[r][hv]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        int q0 = __float2int_rn(__fmul_rn(f.x, inv));
                        int q1 = __float2int_rn(__fmul_rn(f.y, inv));
                        q0 = q0 < p.xq_qmin ? p.xq_qmin : (q0 > p.xq_qmax ? p.xq_qmax : q0);
                        q1 = q1 < p.xq_qmin ? p.xq_qmin : (q1 > p.xq_qmax ? p.xq_qmax : q1);
                        const int e = hv * 8 + j * 2;  // element index 0..15 of this lane's piece
                        word[e >> 2] |= (static_cast<uint32_t>(q0) & 0xffu) << (8 * (e & 3));
                        word[(e + 1) >> 2] |= (static_cast<uint32_t>(q1) & 0xffu) << (8 * ((e + 1) & 3));
                    }
                }
                *reinterpret_cast<uint4*>(stage + r * MMA_KCHUNK + lane * 16) = make_uint4(word[0], word[1], word[2], word[3]);
            }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < MMA_KCHUNK / 64; ++i) {
            xreg[0][i] = gq < p.m ? *reinterpret_cast<const uint4*>(stage + gq * MMA_KCHUNK + i * 64 + tq * 16) : make_uint4(0, 0, 0, 0);
        }
        __syncwarp();  // the staging area is free: it becomes the ring's last slot
        if (MMA_RING - 1 < my_items) issue(MMA_RING - 1);
    }

    bool ok = true;
    for (int mine = 0; mine < my_items; ++mine) {
        const int item = warp + mine * MMA_WARPS;
        const int gi = item / chunks, kc = item - gi * chunks;
        const int k0 = kc * MMA_KCHUNK;
        const int bytes = (p.k - k0 < MMA_KCHUNK) ? (p.k - k0) : MMA_KCHUNK;  // a multiple of 64 on this path
        const int slot = mine % MMA_RING;
        const uint32_t parity = (mine / MMA_RING) & 1;
        if (!mbar_wait_bounded(&full_bar[slot], parity, abort_word, STREAM_WAIT_LIMIT)) {
            *abort_word = 1u;
            atomicCAS(&g_gemv_device_status, 0, 203);
            ok = false;
            break;
        }
        const uint8_t* wrow = ring + slot * MMA_ITEM_BYTES + gq * MMA_PITCH + tq * 16;
        const uint8_t* xrow = xs + gq * xpitch + k0 + tq * 16;
        const bool has_row = gq < p.m;  // activation rows beyond m are zero operands, never read
        // four independent accumulators: consecutive MMAs never wait on each other's result
        int d[4] = {0, 0, 0, 0}, d1[4] = {0, 0, 0, 0}, d2[4] = {0, 0, 0, 0}, d3[4] = {0, 0, 0, 0};
        if constexpr (XREG) {
            // whole chunks only on this path: pull the item into registers, re-arm the slot, then multiply
            uint4 w[MMA_KCHUNK / 64];
#pragma unroll
            for (int i = 0; i < MMA_KCHUNK / 64; ++i) w[i] = *reinterpret_cast<const uint4*>(wrow + i * 64);
            __syncwarp();
            if (mine + MMA_RING < my_items) issue(mine + MMA_RING);
            const bool second = XSETS == 2 && (mine & 1);  // which of the warp's K chunks this item belongs to
#pragma unroll
            for (int i = 0; i < MMA_KCHUNK / 64; ++i) {
                const uint4 x = second ? xreg[XSETS - 1][i] : xreg[0][i];
                if (i & 1) {
                    mma_s8_16x8x32(d2, x.x, x.y, w[i].x, w[i].y);
                    mma_s8_16x8x32(d3, x.z, x.w, w[i].z, w[i].w);
                } else {
                    mma_s8_16x8x32(d, x.x, x.y, w[i].x, w[i].y);
                    mma_s8_16x8x32(d1, x.z, x.w, w[i].z, w[i].w);
                }
            }
        } else {
#pragma unroll 2
        for (int kb = 0; kb < bytes; kb += 128) {
            const uint4 w = *reinterpret_cast<const uint4*>(wrow + kb);
            const uint4 x = has_row ? *reinterpret_cast<const uint4*>(xrow + kb) : make_uint4(0, 0, 0, 0);
            mma_s8_16x8x32(d, x.x, x.y, w.x, w.y);
            mma_s8_16x8x32(d1, x.z, x.w, w.z, w.w);
            if (kb + 64 < bytes) {
                const uint4 w2 = *reinterpret_cast<const uint4*>(wrow + kb + 64);
                const uint4 x2 = has_row ? *reinterpret_cast<const uint4*>(xrow + kb + 64) : make_uint4(0, 0, 0, 0);
                mma_s8_16x8x32(d2, x2.x, x2.y, w2.x, w2.y);
                mma_s8_16x8x32(d3, x2.z, x2.w, w2.z, w2.w);
            }
        }
        }
        d[0] += d1[0] + d2[0] + d3[0];
        d[1] += d1[1] + d2[1] + d3[1];
        if constexpr (!XREG) {
            __syncwarp();  // the whole item has been read: its slot can be refilled
            if (mine + MMA_RING < my_items) issue(mine + MMA_RING);
        }
        // d[0], d[1]: activation row gq, columns 2*tq and 2*tq+1 of this group (d[2], d[3] belong to the zero rows)
        if (gq < p.m) {
            atomicAdd(&acc_s[gi * 64 + gq * 8 + 2 * tq], d[0]);
            atomicAdd(&acc_s[gi * 64 + gq * 8 + 2 * tq + 1], d[1]);
        }
    }
    (void)ok;
    __syncthreads();
    for (int i = threadIdx.x; i < ngroups * 64; i += MMA_WARPS * 32) {
        const int gi = i >> 6, r = (i >> 3) & 7, c = i & 7;
        const int col = col_begin + gi * MMA_COLS + c;
        if (r < p.m && col < col_end) {
            if constexpr (RAW) {
                store_result<RAW>(p, g, r, col, acc_s[i]);
            } else {
                __nv_bfloat16* dp =
                    reinterpret_cast<__nv_bfloat16*>(p.d) + g * p.stride_d + static_cast<int64_t>(r) * p.ldd + col;
                const float sa_r = XQ ? xq_scale[r] : __ldg(p.sa + g * p.stride_sa + r);
                const float sc = __fmul_rn(sa_r, sb_s[gi * MMA_COLS + c]);
                float y = __fmul_rn(__fmul_rn(sc, static_cast<float>(acc_s[i])), p.alpha);
                if (p.beta != 0.0f) y = __fadd_rn(y, __fmul_rn(p.beta, __bfloat162float(*dp)));
                *dp = __float2bfloat16_rn(y);
            }
        }
    }
    __syncwarp();
    if (*abort_word != 0u) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
}

// ---- weights stored [K, N] (N contiguous): a thread owns 16 adjacent columns,
// a CTA owns a 512-column strip of one K slice; slices meet in the workspace ----
__device__ __forceinline__ void transpose4x4_bytes(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3,
                                                   uint32_t (&c)[4]) {
    const uint32_t t0 = __byte_perm(r0, r1, 0x5140);
    const uint32_t t1 = __byte_perm(r0, r1, 0x7362);
    const uint32_t t2 = __byte_perm(r2, r3, 0x5140);
    const uint32_t t3 = __byte_perm(r2, r3, 0x7362);
    c[0] = __byte_perm(t0, t2, 0x5410);
    c[1] = __byte_perm(t0, t2, 0x7632);
    c[2] = __byte_perm(t1, t3, 0x5410);
    c[3] = __byte_perm(t1, t3, 0x7632);
}

template <int MR, bool RAW>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_q8_rrr_kernel(const GemvParams p) {
    extern __shared__ uint32_t smem_u32s[];
    // layout: x words [MR][kslice_rows/4], then red [MR][512] int32
    const int xw_per_row = p.kslice_rows >> 2;
    uint32_t* xs = smem_u32s;
    int* red = reinterpret_cast<int*>(smem_u32s + MR * xw_per_row);
    __shared__ int s_is_last;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cb = blockIdx.x;
    const int ks = blockIdx.y;
    const int64_t g = blockIdx.z;
    const int8_t* a = p.a + g * p.stride_a;
    const int8_t* b = p.b + g * p.stride_b;
    const int k_begin = ks * p.kslice_rows;
    const int k_end = (k_begin + p.kslice_rows < p.k) ? (k_begin + p.kslice_rows) : p.k;

    // stage this slice of the activations (zero beyond K) and clear the reduction buffer
    for (int i = threadIdx.x; i < MR * xw_per_row; i += GEMV_THREADS) {
        const int r = i / xw_per_row, w = i - r * xw_per_row;
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kk = k_begin + w * 4 + j;
            if (kk < k_end) word |= static_cast<uint32_t>(static_cast<uint8_t>(a[static_cast<int64_t>(r) * p.lda + kk])) << (8 * j);
        }
        xs[i] = word;
    }
    for (int i = threadIdx.x; i < MR * RRR_COLS_PER_CTA; i += GEMV_THREADS) red[i] = 0;
    __syncthreads();

    const int col0 = cb * RRR_COLS_PER_CTA + lane * 16;
    const bool col_ok = col0 < p.n;  // n is a multiple of 16 on this path
    int acc[16][MR];
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[j][r] = 0;

    const int rows_per_warp = p.kslice_rows / GEMV_WARPS;  // multiple of 4
    const int wk_begin = k_begin + warp * rows_per_warp;
    if (col_ok) {
        for (int kk = wk_begin; kk < wk_begin + rows_per_warp && kk < k_end; kk += 4) {
            uint4 w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (kk + j < k_end) ? ldg_stream_v4(b + static_cast<int64_t>(kk + j) * p.ldb + col0)
                                        : make_uint4(0, 0, 0, 0);
            }
            uint32_t cols[16];
            {
                uint32_t t[4];
                transpose4x4_bytes(w[0].x, w[1].x, w[2].x, w[3].x, t);
                cols[0] = t[0]; cols[1] = t[1]; cols[2] = t[2]; cols[3] = t[3];
                transpose4x4_bytes(w[0].y, w[1].y, w[2].y, w[3].y, t);
                cols[4] = t[0]; cols[5] = t[1]; cols[6] = t[2]; cols[7] = t[3];
                transpose4x4_bytes(w[0].z, w[1].z, w[2].z, w[3].z, t);
                cols[8] = t[0]; cols[9] = t[1]; cols[10] = t[2]; cols[11] = t[3];
                transpose4x4_bytes(w[0].w, w[1].w, w[2].w, w[3].w, t);
                cols[12] = t[0]; cols[13] = t[1]; cols[14] = t[2]; cols[15] = t[3];
            }
            const int xw = (kk - k_begin) >> 2;
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                const int xv = static_cast<int>(xs[r * xw_per_row + xw]);  // same word for every lane
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j][r] = __dp4a(static_cast<int>(cols[j]), xv, acc[j][r]);
            }
        }
#pragma unroll
        for (int r = 0; r < MR; ++r)
#pragma unroll
            for (int j = 0; j < 16; ++j) atomicAdd(&red[r * RRR_COLS_PER_CTA + lane * 16 + j], acc[j][r]);
    }
    __syncthreads();

    const int ncols_here = (p.n - cb * RRR_COLS_PER_CTA < RRR_COLS_PER_CTA) ? (p.n - cb * RRR_COLS_PER_CTA)
                                                                             : RRR_COLS_PER_CTA;
    if (p.num_kslices == 1) {
        for (int i = threadIdx.x; i < MR * ncols_here; i += GEMV_THREADS) {
            const int r = i / ncols_here, c = i - r * ncols_here;
            store_result<RAW>(p, g, r, cb * RRR_COLS_PER_CTA + c, red[r * RRR_COLS_PER_CTA + c]);
        }
        return;
    }

    // publish this slice's partial sums, then take a ticket; the CTA that draws
    // the last ticket of its column strip folds the slices in slice order.
    int32_t* part = p.ws_partials + (g * p.num_kslices + ks) * static_cast<int64_t>(MR) * p.n;
    for (int i = threadIdx.x; i < MR * ncols_here; i += GEMV_THREADS) {
        const int r = i / ncols_here, c = i - r * ncols_here;
        __stcg(part + static_cast<int64_t>(r) * p.n + cb * RRR_COLS_PER_CTA + c, red[r * RRR_COLS_PER_CTA + c]);
    }
    __threadfence();
    __syncthreads();
    unsigned int* ticket = p.ws_tickets + g * gridDim.x + cb;
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        s_is_last = (t == static_cast<unsigned int>(p.num_kslices - 1)) ? 1 : 0;
    }
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();
    const int32_t* all = p.ws_partials + g * p.num_kslices * static_cast<int64_t>(MR) * p.n;
    for (int i = threadIdx.x; i < MR * ncols_here; i += GEMV_THREADS) {
        const int r = i / ncols_here, c = i - r * ncols_here;
        const int col = cb * RRR_COLS_PER_CTA + c;
        int sum = 0;
        for (int s = 0; s < p.num_kslices; ++s) {
            sum += __ldcg(all + (static_cast<int64_t>(s) * MR + r) * p.n + col);
        }
        store_result<RAW>(p, g, r, col, sum);
    }
    if (threadIdx.x == 0) *ticket = 0u;  // leave the ticket ready for the next call
}

// ---- any layout, any alignment: one warp per output column, byte loads ----
template <bool RAW>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_q8_generic_kernel(const GemvParams p, int layout) {
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t g = blockIdx.y;
    const int col = blockIdx.x * GEMV_WARPS + warp;
    if (col >= p.n) return;
    const int8_t* a = p.a + g * p.stride_a;
    const int8_t* b = p.b + g * p.stride_b;
    int acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0;
    for (int kk = lane; kk < p.k; kk += 32) {
        const int wv = (layout == BQ_LAYOUT_RCR) ? b[static_cast<int64_t>(col) * p.ldb + kk]
                                                 : b[static_cast<int64_t>(kk) * p.ldb + col];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < p.m) acc[r] += wv * static_cast<int>(a[static_cast<int64_t>(r) * p.lda + kk]);
        }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < p.m) {
            const int v = warp_sum(acc[r]);
            if (lane == r) store_result<RAW>(p, g, r, col, v);
        }
    }
}

struct RrrPlan {
    int kslice_rows;
    int num_kslices;
    int col_blocks;
};

// Depends on the problem shape only, so workspace_size() and run() agree.
RrrPlan plan_rrr(int32_t n, int32_t k) {
    RrrPlan pl;
    pl.col_blocks = (n + RRR_COLS_PER_CTA - 1) / RRR_COLS_PER_CTA;
    if (pl.col_blocks < 1) pl.col_blocks = 1;
    // aim for about 512 CTAs; a slice is a multiple of 32 rows (4 rows x 8 warps)
    int want_slices = (512 + pl.col_blocks - 1) / pl.col_blocks;
    int rows = (k + want_slices - 1) / want_slices;
    rows = ((rows + 31) / 32) * 32;
    if (rows < 32) rows = 32;
    if (rows > 2048) rows = 2048;
    // no more slices than keep the partial rows (slices x n per activation row) inside the scratch the streaming
    // kernel asks for ((160 + strips of 1024 columns) x 1024), so one workspace size serves both
    const int64_t cap = (160 + (static_cast<int64_t>(n) + 1023) / 1024) * 1024 / (n > 0 ? n : 1);
    if (cap >= 1 && (k + rows - 1) / rows > cap) {
        rows = static_cast<int>((k + cap - 1) / cap);
        rows = ((rows + 31) / 32) * 32;
    }
    pl.kslice_rows = rows;
    pl.num_kslices = (k + rows - 1) / rows;
    if (pl.num_kslices < 1) pl.num_kslices = 1;
    return pl;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// per-device SM count (cached under a mutex by the GEMM file)
int sm_count_cached() { return sm_count_of_current_device(); }

template <int MR, bool RAW, int NW, int RING>
int32_t launch_rcr_stream_cfg(const GemvParams& p, int batch, int sms, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(RING) + (RING / STREAM_CHUNK) * 8 + NW * 4;
    auto kern = gemv_q8_rcr_stream_kernel<MR, RAW, NW, RING>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    const int ctas = p.n < sms ? p.n : sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, batch, 1);
    cfg.blockDim = dim3(NW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

template <int MR, bool RAW>
int32_t launch_rcr_stream(const GemvParams& p, int batch, cudaStream_t stream) {
    const int sms = sm_count_cached();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    if (p.pdl) return launch_rcr_stream_cfg<MR, RAW, 8, STREAM_RING_HALF>(p, batch, sms, stream);
    return launch_rcr_stream_cfg<MR, RAW, (MR == 1) ? 16 : 8, STREAM_RING_FULL>(p, batch, sms, stream);
}

size_t mma_smem_bytes(int kchunk, int warps, int ring, int m, int k, int groups) {
    return static_cast<size_t>(warps) * ring * MMA_COLS * (kchunk + 64) + static_cast<size_t>(m) * (k + 64) +
           static_cast<size_t>(groups) * 64 * 4 + static_cast<size_t>(groups) * MMA_COLS * 4 + warps * ring * 8 + warps * 4 + 16;
}

template <bool RAW, int KCHUNK, int WARPS, int RING, bool XREG = false, bool XQ = false, int XSETS = 1>
int32_t launch_rcr_mma_cfg(GemvParams p, int batch, int sms, cudaStream_t stream) {
    const int want = (p.n + MMA_COLS - 1) / MMA_COLS;  // no more CTAs than 8-column groups
    const int ctas = want < sms ? want : sms;
    p.mma_groups = (want + ctas - 1) / ctas;
    const size_t smem = mma_smem_bytes(KCHUNK, WARPS, RING, XREG ? 0 : p.m, p.k, p.mma_groups);
    auto kern = gemv_q8_rcr_mma_kernel<RAW, KCHUNK, WARPS, RING, XREG, XQ, XSETS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, batch, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return BQ_STATUS_LAUNCH_FAILURE;
    }
    return BQ_STATUS_OK;
}

// Which register-activation configuration serves this K on sixteen warps: 1 = 512-byte chunks, a divisor of 16 of them
// (K = 512 .. 8192); 2 = 32 chunks of 512 (K = 16384) and 3 = 32 chunks of 448 (K = 14336), two chunks per warp;
// 4 = 16 chunks of 448 (K = 7168); 0 = none.
int mma_xreg_config(const GemvParams& p) {
    const int sms = sm_count_cached();
    if (sms <= 0) return 0;
    const int want = (p.n + MMA_COLS - 1) / MMA_COLS;
    const int ctas = want < sms ? want : sms;
    const int groups = (want + ctas - 1) / ctas;
    if (groups > MMA_MAX_GROUPS || mma_smem_bytes(512, 16, 3, 0, p.k, groups) > 232448) return 0;
    if (p.k % 512 == 0 && 16 % (p.k / 512) == 0) return 1;
    if (p.k == 32 * 512) return 2;
    if (p.k == 32 * 448) return 3;
    if (p.k == 16 * 448) return 4;
    return 0;
}

template <bool RAW>
int32_t launch_rcr_mma(const GemvParams& p, int batch, cudaStream_t stream) {
    const int sms = sm_count_cached();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    // 512-byte (or 448-byte) copies on 16 warps, three items in flight, activations in registers -- when K is a whole
    // number of such chunks that divides (or is twice) the warp count: 13.3 us against 16.5 us at m = 2..8,
    // K = 4096, N = 14336
    switch (mma_xreg_config(p)) {
        case 1: return launch_rcr_mma_cfg<RAW, 512, 16, 3, true>(p, batch, sms, stream);
        case 2: return launch_rcr_mma_cfg<RAW, 512, 16, 3, true, false, 2>(p, batch, sms, stream);
        case 3: return launch_rcr_mma_cfg<RAW, 448, 16, 3, true, false, 2>(p, batch, sms, stream);
        case 4: return launch_rcr_mma_cfg<RAW, 448, 16, 3, true>(p, batch, sms, stream);
        default: break;
    }
    if (p.k > MMA_MAX_K) return BQ_STATUS_UNSUPPORTED;  // the staged-activation configuration holds all of K in shared memory
    // any other K: 1 KiB copies on 8 warps, two items in flight per warp (a third measured no faster)
    return launch_rcr_mma_cfg<RAW, 1024, 8, 2>(p, batch, sms, stream);
}

// The tensor-core GEMV serves K-contiguous weights when K is a multiple of 64 bytes, fits the
// activation staging, and every CTA's share of 8-column groups fits the shared accumulator.
bool mma_gemv_ok(const GemvParams& p) {
    const int sms = sm_count_cached();
    if (sms <= 0) return false;
    const int want = (p.n + MMA_COLS - 1) / MMA_COLS;
    const int ctas = want < sms ? want : sms;
    const int per_cta = (want + ctas - 1) / ctas;
    return (p.k % 64 == 0) && (p.k <= MMA_MAX_K || mma_xreg_config(p) != 0) && per_cta <= MMA_MAX_GROUPS;
}

template <int MR, bool RAW>
int32_t launch_rcr(const GemvParams& p, int batch, cudaStream_t stream) {
    // enough warps to cover the machine several times over, else fewer columns per warp
    const size_t smem = static_cast<size_t>(MR) * KB_BYTES;
    auto blocks_for = [&](int cpw) { return (p.n + GEMV_WARPS * cpw - 1) / (GEMV_WARPS * cpw); };
    if (p.n >= 8192) {
        auto kern = gemv_q8_rcr_kernel<MR, 4, RAW>;
        kern<<<dim3(blocks_for(4), batch), GEMV_THREADS, smem, stream>>>(p);
    } else if (p.n >= 2048) {
        auto kern = gemv_q8_rcr_kernel<MR, 2, RAW>;
        kern<<<dim3(blocks_for(2), batch), GEMV_THREADS, smem, stream>>>(p);
    } else {
        auto kern = gemv_q8_rcr_kernel<MR, 1, RAW>;
        kern<<<dim3(blocks_for(1), batch), GEMV_THREADS, smem, stream>>>(p);
    }
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

template <int MR, bool RAW>
int32_t launch_rrr(GemvParams p, int batch, const GemvDesc& gd, cudaStream_t stream) {
    const RrrPlan pl = plan_rrr(p.n, p.k);
    p.kslice_rows = pl.kslice_rows;
    p.num_kslices = pl.num_kslices;
    if (pl.num_kslices > 1) {
        const size_t tickets_bytes = align_up(static_cast<size_t>(batch) * pl.col_blocks * sizeof(unsigned int), 256);
        const size_t need = tickets_bytes + static_cast<size_t>(batch) * pl.num_kslices * p.m * p.n * sizeof(int32_t);
        if (gd.workspace == nullptr || gd.workspace_bytes < need) return BQ_STATUS_WORKSPACE;
        if (!aligned16(gd.workspace)) return BQ_STATUS_MISALIGNED;
        p.ws_tickets = static_cast<unsigned int*>(gd.workspace);
        p.ws_partials = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(gd.workspace) + tickets_bytes);
        // the workspace is opaque scratch: the tickets must start at zero on every call
        if (cudaMemsetAsync(p.ws_tickets, 0, tickets_bytes, stream) != cudaSuccess) {
            (void)cudaGetLastError();
            return BQ_STATUS_LAUNCH_FAILURE;
        }
    }
    const size_t smem = static_cast<size_t>(MR) * (pl.kslice_rows / 4) * 4 + static_cast<size_t>(MR) * RRR_COLS_PER_CTA * 4;
    auto kern = gemv_q8_rrr_kernel<MR, RAW>;
    kern<<<dim3(pl.col_blocks, pl.num_kslices, batch), GEMV_THREADS, smem, stream>>>(p);
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

#include "gemv_q8_rrr_rows.cuh"

template <bool RAW>
int32_t dispatch(const GemvDesc& g, cudaStream_t stream) {
    GemvParams p;
    p.a = g.a; p.lda = g.lda; p.stride_a = g.stride_a;
    p.b = g.b; p.ldb = g.ldb; p.stride_b = g.stride_b;
    p.sa = g.scale_a; p.stride_sa = g.stride_scale_a;
    p.sb = g.scale_b; p.stride_sb = g.stride_scale_b;
    p.d = g.d; p.ldd = g.ldd; p.stride_d = g.stride_d;
    p.alpha = g.alpha; p.beta = g.beta;
    p.m = g.m; p.n = g.n; p.k = g.k;
    p.kslice_rows = 0; p.num_kslices = 1;
    p.ws_partials = nullptr; p.ws_tickets = nullptr;
    p.pdl = g.pdl;
    p.mma_groups = 0;
    p.rr_strips = 0; p.rr_run_max = 0; p.rr_ctas = 0; p.rr_slots_total = 0; p.rr_rows_total = 0; p.rr_partials = nullptr;
    p.xq_x = nullptr; p.xq_ldx = 0; p.xq_qmin = -127; p.xq_qmax = 127; p.xq_scale_out = nullptr;

    // the streaming kernels need 16-byte alignment of every weight row segment they load
    bool fast = g.k > 0 && aligned16(g.a) && aligned16(g.b) && (g.stride_b % 16 == 0) && (g.ldb % 16 == 0);
    if (g.layout == BQ_LAYOUT_RCR) {
        fast = fast && (g.k % 16 == 0) && (g.lda % 16 == 0 || g.m == 1) && (g.stride_a % 16 == 0);
    } else {
        fast = fast && (g.n % 16 == 0);
    }
    if (g.variant == 9) fast = false;  // tests: force the byte-load kernel
    if (!fast) {
        const int blocks = (g.n + GEMV_WARPS - 1) / GEMV_WARPS;
        gemv_q8_generic_kernel<RAW><<<dim3(blocks, g.batch), GEMV_THREADS, 0, stream>>>(p, g.layout);
        return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
    }
    // Test hooks (set_tuning key 1): 1 = bulk-copy dp4a kernel where legal, 2 = register-streaming kernel, 3 = tensor-core
    // streaming kernel also for m == 1, 8 = direct-load split-K kernel for row-major weights, 9 = byte-load kernel.
    // K-contiguous weights, two or more activation rows: tensor-core streaming kernel
    const bool mma_ok = g.layout == BQ_LAYOUT_RCR && mma_gemv_ok(p);
    if (mma_ok &&
        ((g.variant == 0 && g.m >= 2 && g.n * static_cast<int64_t>(g.k) >= (1 << 20)) || g.variant == 3 ||
         // m = 1: the 16-warp tensor-core kernel also wins under dependent launch, and for the long K of a down
         // projection (14.9 us against 16.5 us at K = 14336, N = 4096)
         (g.variant == 0 && g.m == 1 && ((g.pdl && mma_xreg_config(p) != 0) || mma_xreg_config(p) >= 2) &&
          g.n * static_cast<int64_t>(g.k) >= (1 << 20)))) {
        return launch_rcr_mma<RAW>(p, g.batch, stream);
    }
    // K-contiguous weights with few activation rows: the bulk-copy streaming kernel
    // (variant 2 forces it off, variant 1 forces it on where it is legal)
    if (g.layout == BQ_LAYOUT_RCR && g.m <= 4 && g.variant != 2 && (g.n * static_cast<int64_t>(g.k) >= (1 << 20) || g.variant == 1)) {
        switch (g.m) {
            case 1: return launch_rcr_stream<1, RAW>(p, g.batch, stream);
            case 2: return launch_rcr_stream<2, RAW>(p, g.batch, stream);
            case 3: return launch_rcr_stream<3, RAW>(p, g.batch, stream);
            default: return launch_rcr_stream<4, RAW>(p, g.batch, stream);
        }
    }
    // N-contiguous weights: the row-run streaming kernel (1 KiB bulk copies, ldmatrix-transposed fragments).
    // Each path below checks the scratch its own kernel needs.
    const bool rrr_big = g.layout == BQ_LAYOUT_RRR && g.n * static_cast<int64_t>(g.k) >= (1 << 18);
    if (rrr_big && g.variant == 0) {
        const RrPlan pl = plan_rrr_rows(g.m, g.n, g.k, g.batch, sm_count_cached());
        if (pl.ok) {
            if (g.workspace == nullptr || g.workspace_bytes < pl.ws_bytes) return BQ_STATUS_WORKSPACE;
            if (!aligned16(g.workspace)) return BQ_STATUS_MISALIGNED;
            if constexpr (!RAW) {
                // Few 1024-column strips: the row-run kernel's CTAs then share few strips and its reduce pass adds dozens
                // of partial rows per column, while the tensor-core GEMM's split-K kernel (clusters of four CTAs per
                // 128 x 128 tile, MN-major weight operand) is flat in m.  Measured (CUDA graph, rotating weights), this
                // kernel against the GEMM: N = 1024, K = 4096: 11.0 / 20.8 us at m = 1 / 8 against 7.0; N = 4096,
                // K = 14336: 16.7 / 20.1 against 17.0 / 16.8; N = 4096, K = 4096: 9.4 / 12.8 against 10.4 / 10.2.
                // Same arithmetic per element (the GEMM epilogue's alpha, beta * D), so the bits do not change.
                const bool few_strips = g.n <= 2048 || (g.n <= 4096 && g.m >= 4);
                if (few_strips && g.batch == 1 && (g.lda % 16 == 0 || g.m == 1)) {
                    GemmDesc q = {};
                    q.kind = BQ_KIND_S8;
                    q.b_layout = BQ_LAYOUT_RRR;
                    q.m = g.m;
                    q.n = g.n;
                    q.k = g.k;
                    q.a = g.a;
                    q.lda = g.lda;
                    q.b = g.b;
                    q.ldb = g.ldb;
                    q.scale_a = g.scale_a;
                    q.scale_b = g.scale_b;
                    q.scale_mode = 1;
                    q.alpha = g.alpha;
                    q.beta = g.beta;
                    q.c = g.beta != 0.0f ? g.d : nullptr;
                    q.ldc = g.ldd;
                    q.d = g.d;
                    q.ldd = g.ldd;
                    q.pdl = g.pdl;
                    if (gemm_q8_takes_cluster_split_k(q)) return launch_gemm_q8(q, stream);
                }
            }
            return launch_rrr_rows<RAW>(p, g.batch, pl, g.workspace, stream);
        }
    }
#define BQ_GEMV_CASE(MRV)                                                                  \
    case MRV:                                                                              \
        return g.layout == BQ_LAYOUT_RCR ? launch_rcr<MRV, RAW>(p, g.batch, stream)        \
                                         : launch_rrr<MRV, RAW>(p, g.batch, g, stream);
    switch (g.m) {
        BQ_GEMV_CASE(1)
        BQ_GEMV_CASE(2)
        BQ_GEMV_CASE(3)
        BQ_GEMV_CASE(4)
        BQ_GEMV_CASE(5)
        BQ_GEMV_CASE(6)
        BQ_GEMV_CASE(7)
        BQ_GEMV_CASE(8)
        default: return BQ_STATUS_INVALID_PROBLEM;
    }
#undef BQ_GEMV_CASE
}

}  // namespace

size_t gemv_q8_workspace_bytes(int32_t m, int32_t n, int32_t k, int32_t batch, int32_t layout) {
    if (layout != BQ_LAYOUT_RRR || m <= 0 || n <= 0 || k <= 0 || batch <= 0) return 0;
    // the larger of what the row-major-weight kernels ask for: which one runs depends on alignment and device
    const RrrPlan pl = plan_rrr(n, k);
    size_t direct = 0;
    if (pl.num_kslices > 1) {
        const size_t tickets = align_up(static_cast<size_t>(batch) * pl.col_blocks * sizeof(unsigned int), 256);
        const size_t partials = static_cast<size_t>(batch) * pl.num_kslices * m * n * sizeof(int32_t);
        direct = tickets + partials;
    }
    const size_t streamed = n * static_cast<int64_t>(k) >= (1 << 18) ? rrr_rows_workspace_bytes(m, n, k, batch) : 0;
    return direct > streamed ? direct : streamed;
}

// Shapes the fused-quantiser GEMV serves: K a whole number of 512-byte chunks that divides 16, K-contiguous weights.
bool gemv_q8_quant_bf16_supported(int32_t m, int32_t n, int32_t k) {
    if (m < 1 || m > 8 || n < 1 || k < 512 || (k % 512) != 0 || (16 % (k / 512)) != 0) return false;
    const int sms = sm_count_cached();
    if (sms <= 0) return true;  // no device to ask: the shape rules above are all that can be judged
    const int want = (n + MMA_COLS - 1) / MMA_COLS;
    const int ctas = want < sms ? want : sms;
    const int groups = (want + ctas - 1) / ctas;
    return groups <= MMA_MAX_GROUPS && mma_smem_bytes(512, 16, 3, 0, k, groups) + 1024 <= 232448;  // + the static part
}

int32_t launch_gemv_q8_quant_bf16(int32_t m, int32_t n, int32_t k, int32_t qmin, int32_t qmax, float alpha, float beta,
                                  const void* x_bf16, int64_t ldx, const int8_t* b, int64_t ldb, const float* scale_b,
                                  float* scale_a_out, void* d, int64_t ldd, int32_t pdl, cudaStream_t stream) {
    const int sms = sm_count_cached();
    if (sms <= 0) return BQ_STATUS_LAUNCH_FAILURE;
    GemvParams p = {};
    p.a = nullptr; p.lda = 0; p.stride_a = 0;
    p.b = b; p.ldb = ldb; p.stride_b = 0;
    p.sa = nullptr; p.stride_sa = 0;
    p.sb = scale_b; p.stride_sb = 0;
    p.d = d; p.ldd = ldd; p.stride_d = 0;
    p.alpha = alpha; p.beta = beta;
    p.m = m; p.n = n; p.k = k;
    p.num_kslices = 1;
    p.pdl = pdl;
    p.xq_x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.xq_ldx = ldx;
    p.xq_qmin = qmin;
    p.xq_qmax = qmax;
    p.xq_scale_out = scale_a_out;
    return launch_rcr_mma_cfg<false, 512, 16, 3, true, true>(p, 1, sms, stream);
}

int32_t launch_gemv_q8(const GemvDesc& g, cudaStream_t stream) {
    return g.raw_out ? dispatch<true>(g, stream) : dispatch<false>(g, stream);
}

// ---- self-test of the bounded barrier wait every kernel of the library relies on ----
// One thread waits, with the given cycle budget, on an mbarrier that nothing will ever complete.  The wait must
// give up, record status 299 and let the kernel end; the context stays usable.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0u;
        mbar_init(&bar, 1);
        fence_barrier_init();
        if (!mbar_wait_bounded(&bar, 0u, &abort_flag, limit_cycles)) atomicCAS(&g_gemv_device_status, 0, 299);
    }
}

int32_t launch_bounded_wait_selftest(long long limit_cycles, cudaStream_t stream) {
    if (limit_cycles < 1 || limit_cycles > (1LL << 28)) return BQ_STATUS_INVALID_PROBLEM;  // at most ~0.15 s
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_cycles);
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

int32_t read_and_clear_gemv_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_gemv_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
