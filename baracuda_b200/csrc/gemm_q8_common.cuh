// Pieces shared by the 1-CTA and the 2-CTA tcgen05 GEMM kernels: the kernel
// parameter block and the epilogue that turns 32 accumulator columns of one
// output row into bf16 (fused dequant) or raw 32-bit stores.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100a.cuh"

namespace bq {

struct GemmParams {
    void* d;
    int64_t ldd;
    const float* sa;
    const float* sb;
    int scale_mode;  // 0: sa/sb point at one float each; 1: sa[M], sb[N]; 2: sa_const (by value) and sb[N]
    float sa_const;
    float alpha;
    int m, n, k;
    int m_tiles, n_tiles;
    int vec_store;  // 1 when d and ldd allow 16-byte row stores
    // fused replicated output (FUSED kernels only)
    void* peer_d[8];
    void* mc_d;  // multicast address of the same buffers (one store reaches every rank), or null: unicast stores to peer_d
    int n_peers;
    int64_t peer_ld;
    int peer_col0;
    int peer_vec;  // 1 when every peer buffer allows 16-byte row stores at its column offset
    int peer_rank; // this rank: peers are visited starting at the next rank so no buffer is everyone's target at once
    int coalesce;  // 1: 64-column blocks go through the shared-memory staging path
    // 8-bit output mode (the reference's IntGemm / Fp8Gemm contract): d = sat(alpha*acc + beta*C), same type as the inputs
    int out_q8;
    const void* c;
    int64_t ldc;
    float beta;
    // fused epilogue chain of the reference's EpilogueKind: per-column bias (f32 or i32), then an activation
    const void* bias;
    int bias_kind;  // 0 none, 1 float[N], 2 int32[N]
    int act;        // 0 none, 1 relu, 2 gelu (erf form), 3 silu
    int bias_off;   // the epilogue warp's staged bias values sit bias_off floats after its staged column scales
    // raw-accumulator reduce-scatter (K-sharded GEMM): output row r belongs to rank r / rs_rows and is stored
    // into that rank's staging buffer peer_d[owner], slot peer_rank, row r % rs_rows (row pitch ldd); 0 = off
    int rs_world;
    int rs_rows;
    // gated-MLP mode (bf16 output only): the weight rows hold gate and up projections interleaved in blocks of 32
    // (rows 64b..64b+31 = gate 32b..32b+31, rows 64b+32..64b+63 = up 32b..32b+31), n counts both, and the epilogue
    // stores silu(gate) * up as n/2 columns
    int swiglu;
    // CTA-pair kernel, mixed-width schedule (0 = off: tiles of one width handed out round robin).  Tile columns
    // [0, mixed_full_cols) are 256 wide, the rest of N is cut into 128-wide tiles; pair q runs the 256-wide tiles
    // [full_begin[q], full_begin[q + 1]) and then the 128-wide tiles [half_begin[q], half_begin[q + 1]) (each list
    // numbered m fastest).  The host balances the two lists so that the last, partly filled wave of wide tiles is
    // replaced by narrow ones spread over every pair.
    int mixed;
    int mixed_full_cols;
    // Tile order of the round-robin schedule: tiles are numbered group by group, a group being raster_gm tile rows by
    // all tile columns, row fastest inside it.  The tiles in flight at one time then share raster_gm row blocks of A
    // (chosen to stay resident in L2) and a few weight column blocks, instead of every row block of A.
    int raster_gm;
    int pdl;  // launched as a programmatic dependent: weights may be fetched before the dependency wait
    // cluster split-K kernel: CTA s of a cluster walks the K blocks [s * kb_per_slice, (s + 1) * kb_per_slice)
    int kb_per_slice;
    uint16_t full_begin[98];
    uint16_t half_begin[98];
};

// bias then activation on 32 values, in f32 — the chain of the reference's epilogue header
// (crates/baracuda-kernels-sys/kernels/include/baracuda_epilogue_int8.cuh:52-95).  The bias values come from the
// warp's shared-memory copy (staged once per tile next to the column scales).
// gelu = 0.5 z (1 + erf(z / sqrt 2)) with erf from the Abramowitz-Stegun 7.1.26 polynomial (|error| <= 1.5e-7, the
// form the reference's own CPU check uses, crates/baracuda-kernels/tests/int8_rrr_smoke.rs:35-53) and
// silu = z / (1 + exp(-z)) with the fast exponential and division: a dozen instructions each.  The library erff and an
// IEEE division, inlined once per accumulator (32 copies per 32-column block), grew the epilogue loop beyond the
// instruction cache and halved the speed even of launches that never ran them (8-bit-out GEMM 8192 x 8192 x 4096:
// 404 us against 184 us for the bf16 SKU); called out of line they cost 3-6x the identity epilogue.  The results stay
// inside the reference's tolerance for these two chains (+-1 output code, two e4m3 grid steps).
// gelu(z) = 0.5 z (1 + erf(z / sqrt 2)) = relu(z) - 0.5 |z| (1 - erf(|z| / sqrt 2)), and 1 - erf(x) = poly(t) t exp(-x^2)
// with t = 1 / (1 + p x) (Abramowitz-Stegun 7.1.26): fifteen instructions, two of them on the special-function unit,
// and no cancellation for negative z (the direct form subtracts erf from 1 there).
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_erf_poly(float z) {
    const float az = fabsf(z);
    const float t = rcp_approx(fmaf(0.3275911f * 0.70710678118654752440f, az, 1.0f));
    const float e = ex2_approx((z * z) * (-0.5f * 1.44269504088896340736f));  // exp(-z^2 / 2)
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float q = (poly * t) * e;  // 1 - erf(|z| / sqrt 2)
    return fmaf(-0.5f * az, q, fmaxf(z, 0.0f));
}

// silu(z) = z / (1 + exp(-z)): two special-function instructions and three others
__device__ __forceinline__ float silu_fast(float z) { return z * rcp_approx(1.0f + ex2_approx(z * -1.44269504088896340736f)); }

// 32 staged floats (column scales or bias values of one 32-column block; every lane reads the same addresses) as
// eight 16-byte broadcast loads.  The epilogue shares the SM's shared-memory bandwidth with the operand tiles the
// tensor core is reading and TMA is writing; scalar loads here (32 wavefronts per block and operand) cost the main
// loop 6 % on the bias epilogue.  The staged slices are 16-byte aligned by construction.
__device__ __forceinline__ void load_staged_32(const float* src, float (&dst)[32]) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
        const float4 q = reinterpret_cast<const float4*>(src)[v];
        dst[4 * v] = q.x;
        dst[4 * v + 1] = q.y;
        dst[4 * v + 2] = q.z;
        dst[4 * v + 3] = q.w;
    }
}

__device__ __forceinline__ void apply_bias_act_32(const GemmParams& p, float (&z)[32], const float* sb32) {
    if (p.bias_kind != 0) {
        float bias32[32];
        load_staged_32(sb32 + p.bias_off, bias32);
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = __fadd_rn(z[j], bias32[j]);
    }
    if (p.act == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = fmaxf(z[j], 0.0f);
    } else if (p.act == 2) {
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = gelu_erf_poly(z[j]);
    } else if (p.act == 3) {
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = silu_fast(z[j]);
    }
}

// y += beta * C on the bf16-out SKUs (C is bf16 [M, ldc], may be D itself: every element is read by the warp that
// later overwrites it, before that store).  Product and sum are rounded separately in f32.
__device__ __forceinline__ void add_beta_c_bf16_32(const GemmParams& p, int row, int col0, float (&y)[32]) {
    const __nv_bfloat16* crow = reinterpret_cast<const __nv_bfloat16*>(p.c) + static_cast<int64_t>(row) * p.ldc + col0;
    if (col0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(crow) & 15u) == 0) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 q = reinterpret_cast<const uint4*>(crow)[v];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                y[8 * v + 2 * i] = __fadd_rn(y[8 * v + 2 * i], __fmul_rn(p.beta, __uint_as_float(w[i] << 16)));
                y[8 * v + 2 * i + 1] =
                    __fadd_rn(y[8 * v + 2 * i + 1], __fmul_rn(p.beta, __uint_as_float(w[i] & 0xffff0000u)));
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < p.n) y[j] = __fadd_rn(y[j], __fmul_rn(p.beta, __bfloat162float(crow[j])));
        }
    }
}

// One thread, one output row, 32 consecutive columns starting at col0 (a multiple of 32).
// `r` holds the accumulators as read from TMEM, `sb32` the 32 column scales.
template <uint32_t KIND, bool RAW, bool FUSED>
__device__ __forceinline__ void epilogue_store_32(const GemmParams& p, int row, int col0, const uint32_t (&r)[32],
                                                  float sa_row, const float* sb32) {
    if constexpr (RAW) {
        uint32_t* drow;
        if (p.rs_world > 1) {
            const int owner = row / p.rs_rows;
            drow = reinterpret_cast<uint32_t*>(p.peer_d[owner]) +
                   (static_cast<int64_t>(p.peer_rank) * p.rs_rows + (row - owner * p.rs_rows)) * p.ldd + col0;
        } else {
            drow = reinterpret_cast<uint32_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
        }
        if (p.vec_store && col0 + 32 <= p.n) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                reinterpret_cast<uint4*>(drow)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.n) drow[j] = r[j];
            }
        }
    } else if (p.out_q8) {
        // z = alpha * acc (+ beta * C), each product and the sum rounded in f32; s8: round half to even and
        // clamp to [-128, 127]; e4m3: round to nearest even, saturate to +-448 (no infinities)
        uint8_t* drow = reinterpret_cast<uint8_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
        const uint8_t* crow =
            p.c ? reinterpret_cast<const uint8_t*>(p.c) + static_cast<int64_t>(row) * p.ldc + col0 : nullptr;
        float z[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if constexpr (KIND == UMMA_KIND_I8) {
                z[j] = __fmul_rn(p.alpha, static_cast<float>(static_cast<int32_t>(r[j])));
            } else {
                z[j] = __fmul_rn(p.alpha, __uint_as_float(r[j]));
            }
        }
        if (crow) {
            uint8_t cb[32];
            if (col0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(crow) & 15u) == 0) {
                const uint4 lo = __ldg(reinterpret_cast<const uint4*>(crow));
                const uint4 hi = __ldg(reinterpret_cast<const uint4*>(crow) + 1);
                const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int j = 0; j < 32; ++j) cb[j] = static_cast<uint8_t>(w[j >> 2] >> (8 * (j & 3)));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) cb[j] = col0 + j < p.n ? crow[j] : 0;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float cv;
                if constexpr (KIND == UMMA_KIND_I8) {
                    cv = static_cast<float>(static_cast<int8_t>(cb[j]));
                } else {
                    const __half_raw hr = __nv_cvt_fp8_to_halfraw(cb[j], __NV_E4M3);
                    cv = __half2float(__half(hr));
                }
                z[j] = __fadd_rn(z[j], __fmul_rn(p.beta, cv));
            }
        }
        if ((p.bias_kind | p.act) != 0) apply_bias_act_32(p, z, sb32);
        uint32_t packed[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int j = 4 * w + b;
                uint8_t out;
                if constexpr (KIND == UMMA_KIND_I8) {
                    int q = __float2int_rn(z[j]);
                    q = q < -128 ? -128 : (q > 127 ? 127 : q);
                    out = static_cast<uint8_t>(static_cast<int8_t>(q));
                } else {
                    out = static_cast<uint8_t>(__nv_cvt_float_to_fp8(z[j], __NV_SATFINITE, __NV_E4M3));
                }
                word |= static_cast<uint32_t>(out) << (8 * b);
            }
            packed[w] = word;
        }
        if (p.vec_store && col0 + 32 <= p.n) {
            reinterpret_cast<uint4*>(drow)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(drow)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.n) drow[j] = static_cast<uint8_t>(packed[j >> 2] >> (8 * (j & 3)));
            }
        }
    } else {
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0;
        float y[32], sbv[32];
        load_staged_32(sb32, sbv);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float acc;
            if constexpr (KIND == UMMA_KIND_I8) {
                acc = static_cast<float>(static_cast<int32_t>(r[j]));
            } else {
                acc = __uint_as_float(r[j]);
            }
            // (sa*sb) first, then the accumulator, then alpha: the reference's W8A8
            // product order, no fused multiply-add.
            const float s = __fmul_rn(sa_row, sbv[j]);
            y[j] = __fmul_rn(__fmul_rn(s, acc), p.alpha);
        }
        if (p.c != nullptr) add_beta_c_bf16_32(p, row, col0, y);
        if ((p.bias_kind | p.act) != 0) apply_bias_act_32(p, y, sb32);
        uint4 pk[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(y[8 * v + 0], y[8 * v + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(y[8 * v + 2], y[8 * v + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(y[8 * v + 4], y[8 * v + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(y[8 * v + 6], y[8 * v + 7]);
            pk[v].x = *reinterpret_cast<uint32_t*>(&h0);
            pk[v].y = *reinterpret_cast<uint32_t*>(&h1);
            pk[v].z = *reinterpret_cast<uint32_t*>(&h2);
            pk[v].w = *reinterpret_cast<uint32_t*>(&h3);
        }
        if (p.vec_store && col0 + 32 <= p.n) {
#pragma unroll
            for (int v = 0; v < 4; ++v) reinterpret_cast<uint4*>(drow)[v] = pk[v];
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.n) drow[j] = __float2bfloat16_rn(y[j]);
            }
        }
        if constexpr (FUSED) {
            // the replicated output: plain stores into every rank's row-major buffer
            // (peer-mapped memory), at this rank's column offset
            for (int i = 1; i <= p.n_peers; ++i) {
                int pr = p.peer_rank + i;
                if (pr >= p.n_peers) pr -= p.n_peers;
                __nv_bfloat16* prow = reinterpret_cast<__nv_bfloat16*>(p.peer_d[pr]) +
                                      static_cast<int64_t>(row) * p.peer_ld + p.peer_col0 + col0;
                if (p.peer_vec && col0 + 32 <= p.n) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) reinterpret_cast<uint4*>(prow)[v] = pk[v];
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (col0 + j < p.n) prow[j] = __float2bfloat16_rn(y[j]);
                    }
                }
            }
        }
    }
}


// Converts 32 accumulator columns of this thread's row into 32 bf16 (four 16-byte packets).
template <uint32_t KIND>
__device__ __forceinline__ void dequant_pack_32(const GemmParams& p, const uint32_t (&r)[32], float sa_row,
                                                const float* sb32, uint4 (&pk)[4], int row, int col0) {
    float y[32], sbv[32];
    load_staged_32(sb32, sbv);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        float acc;
        if constexpr (KIND == UMMA_KIND_I8) {
            acc = static_cast<float>(static_cast<int32_t>(r[j]));
        } else {
            acc = __uint_as_float(r[j]);
        }
        const float s = __fmul_rn(sa_row, sbv[j]);
        y[j] = __fmul_rn(__fmul_rn(s, acc), p.alpha);
    }
    if (p.c != nullptr && row < p.m) add_beta_c_bf16_32(p, row, col0, y);
    if ((p.bias_kind | p.act) != 0) apply_bias_act_32(p, y, sb32);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(y[8 * v + 0], y[8 * v + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(y[8 * v + 2], y[8 * v + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(y[8 * v + 4], y[8 * v + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(y[8 * v + 6], y[8 * v + 7]);
        pk[v].x = *reinterpret_cast<uint32_t*>(&h0);
        pk[v].y = *reinterpret_cast<uint32_t*>(&h1);
        pk[v].z = *reinterpret_cast<uint32_t*>(&h2);
        pk[v].w = *reinterpret_cast<uint32_t*>(&h3);
    }
}

// bf16 epilogue for a 32-row x 64-column block owned by one warp (lane = row), with the rows
// re-shaped through a 4 KiB shared-memory staging area so that every store instruction writes
// four complete 128-byte row segments (8 lanes x 16 bytes each) instead of 32 scattered 16-byte
// pieces.  That is what the local L2 wants and, in fused mode, what NVLink needs for the peer
// stores.  `t_addr` is the TMEM address of the block's first column for this warp's lanes.
// Requires 16-byte-aligned output rows (vec_store) and the full 64 columns in range.
// `stage` is this warp's private 4 KiB buffer; `row_base` is the global row of lane 0.
template <uint32_t KIND, bool FUSED>
__device__ __forceinline__ void epilogue_block_64(const GemmParams& p, uint32_t t_addr, int row_base, int lane,
                                                  int col0, float sa_row, const float* sb64, uint4* stage) {
    // 16-byte packet c of row r lives at stage[r * 8 + (c ^ (r & 7))]: conflict-free both ways
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr + static_cast<uint32_t>(half * 32), r);
        tmem_ld_wait();
        uint4 pk[4];
        dequant_pack_32<KIND>(p, r, sa_row, sb64 + half * 32, pk, row_base + lane, col0 + half * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const int c = half * 4 + v;
            stage[lane * 8 + (c ^ (lane & 7))] = pk[v];
        }
    }
    __syncwarp();
    const int sub_row = lane >> 3;  // 0..3
    const int c = lane & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + sub_row;
        const int row = row_base + rr;
        const uint4 v = stage[rr * 8 + (c ^ (rr & 7))];
        if (row < p.m) {
            if (p.d != nullptr) {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0 +
                                          c * 8) = v;
            }
            if constexpr (FUSED) {
                if (p.mc_d != nullptr) {
                    multimem_st_16(reinterpret_cast<__nv_bfloat16*>(p.mc_d) + static_cast<int64_t>(row) * p.peer_ld + p.peer_col0 +
                                       col0 + c * 8, v);
                } else {
                    for (int i = 1; i <= p.n_peers; ++i) {
                        int pr = p.peer_rank + i;
                        if (pr >= p.n_peers) pr -= p.n_peers;
                        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer_d[pr]) +
                                                  static_cast<int64_t>(row) * p.peer_ld + p.peer_col0 + col0 + c * 8) = v;
                    }
                }
            }
        }
    }
    __syncwarp();
}

// The same for a 32-column block (the tail of tile widths that are not a multiple of 64): 32 rows x 64 bytes,
// 16-byte packet c of row r at stage[r * 4 + (c ^ ((r >> 1) & 3))]; each store instruction writes eight 64-byte
// row segments.
template <uint32_t KIND, bool FUSED>
__device__ __forceinline__ void epilogue_block_32(const GemmParams& p, uint32_t t_addr, int row_base, int lane,
                                                  int col0, float sa_row, const float* sb32, uint4* stage) {
    {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr, r);
        tmem_ld_wait();
        uint4 pk[4];
        dequant_pack_32<KIND>(p, r, sa_row, sb32, pk, row_base + lane, col0);
#pragma unroll
        for (int v = 0; v < 4; ++v) stage[lane * 4 + (v ^ ((lane >> 1) & 3))] = pk[v];
    }
    __syncwarp();
    const int sub_row = lane >> 2;  // 0..7
    const int c = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = i * 8 + sub_row;
        const int row = row_base + rr;
        const uint4 v = stage[rr * 4 + (c ^ ((rr >> 1) & 3))];
        if (row < p.m) {
            if (p.d != nullptr) {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0 +
                                          c * 8) = v;
            }
            if constexpr (FUSED) {
                if (p.mc_d != nullptr) {
                    multimem_st_16(reinterpret_cast<__nv_bfloat16*>(p.mc_d) + static_cast<int64_t>(row) * p.peer_ld + p.peer_col0 +
                                       col0 + c * 8, v);
                } else {
                    for (int j = 1; j <= p.n_peers; ++j) {
                        int pr = p.peer_rank + j;
                        if (pr >= p.n_peers) pr -= p.n_peers;
                        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer_d[pr]) +
                                                  static_cast<int64_t>(row) * p.peer_ld + p.peer_col0 + col0 + c * 8) = v;
                    }
                }
            }
        }
    }
    __syncwarp();
}

// Gated-MLP epilogue for one 64-column block of an interleaved gate/up weight: columns col0..col0+31 are 32 gate
// projections, col0+32..col0+63 the matching up projections; the warp stores h = silu(z_gate) * z_up as 32 bf16
// columns starting at col0 / 2 (z = alpha * (sa * sb) * acc + bias, as in the plain epilogue).  Rows go through the
// staging buffer like epilogue_block_32.  Requires the full 64 columns in range and 16-byte-aligned output rows.
template <uint32_t KIND>
__device__ __forceinline__ void epilogue_block_64_swiglu(const GemmParams& p, uint32_t t_addr, int row_base, int lane,
                                                         int col0, float sa_row, const float* sb64, uint4* stage) {
    float h[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr + static_cast<uint32_t>(half * 32), r);
        tmem_ld_wait();
        const float* sb32 = sb64 + half * 32;
        float sbv[32], bias32[32];
        load_staged_32(sb32, sbv);
        if (p.bias_kind != 0) load_staged_32(sb32 + p.bias_off, bias32);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float acc;
            if constexpr (KIND == UMMA_KIND_I8) {
                acc = static_cast<float>(static_cast<int32_t>(r[j]));
            } else {
                acc = __uint_as_float(r[j]);
            }
            const float s = __fmul_rn(sa_row, sbv[j]);
            float z = __fmul_rn(__fmul_rn(s, acc), p.alpha);
            if (p.bias_kind != 0) z += bias32[j];
            h[j] = half == 0 ? silu_fast(z) : h[j] * z;
        }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(h[8 * v + 0], h[8 * v + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(h[8 * v + 2], h[8 * v + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(h[8 * v + 4], h[8 * v + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(h[8 * v + 6], h[8 * v + 7]);
        uint4 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2);
        pk.w = *reinterpret_cast<uint32_t*>(&h3);
        stage[lane * 4 + (v ^ ((lane >> 1) & 3))] = pk;
    }
    __syncwarp();
    const int sub_row = lane >> 2;  // 0..7
    const int c = lane & 3;
    const int out_col0 = col0 >> 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = i * 8 + sub_row;
        const int row = row_base + rr;
        const uint4 v = stage[rr * 4 + (c ^ ((rr >> 1) & 3))];
        if (row < p.m) {
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + static_cast<int64_t>(row) * p.ldd + out_col0 +
                                      c * 8) = v;
        }
    }
    __syncwarp();
}

// Raw 32-bit accumulators of a 32-column block (reduce-scatter mode, or the plain raw output): 32 rows x 128 bytes go through the warp's
// staging buffer (16-byte packet c of row r at stage[r * 8 + (c ^ (r & 7))]) so that every store instruction writes
// four complete 128-byte row segments -- what stores that cross NVLink need.  Row r of the tile lands in the staging
// buffer of the rank that owns it (see GemmParams::rs_world).
__device__ __forceinline__ void epilogue_block_raw32_scatter(const GemmParams& p, uint32_t t_addr, int row_base, int lane,
                                                             int col0, uint4* stage) {
    {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            stage[lane * 8 + (v ^ (lane & 7))] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        }
    }
    __syncwarp();
    const int sub_row = lane >> 3;  // 0..3
    const int c = lane & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + sub_row;
        const int row = row_base + rr;
        const uint4 v = stage[rr * 8 + (c ^ (rr & 7))];
        if (row < p.m) {
            uint32_t* dst;
            if (p.rs_world > 1) {
                const int owner = row / p.rs_rows;
                dst = reinterpret_cast<uint32_t*>(p.peer_d[owner]) +
                      (static_cast<int64_t>(p.peer_rank) * p.rs_rows + (row - owner * p.rs_rows)) * p.ldd + col0 + c * 4;
            } else {  // the local raw output, through the same staging: whole 128-byte row segments per store
                dst = reinterpret_cast<uint32_t*>(p.d) + static_cast<int64_t>(row) * p.ldd + col0 + c * 4;
            }
            *reinterpret_cast<uint4*>(dst) = v;
        }
    }
    __syncwarp();
}

template <bool FUSED>
__device__ __forceinline__ bool block_32_ok(const GemmParams& p, int col0) {
    bool ok = p.coalesce && p.vec_store && (col0 + 32 <= p.n);
    if constexpr (FUSED) ok = ok && p.peer_vec;
    return ok;
}

// True when the 64-column block starting at col0 can take the coalesced path.
template <bool FUSED>
__device__ __forceinline__ bool block_64_ok(const GemmParams& p, int col0) {
    bool ok = p.coalesce && p.vec_store && (col0 + 64 <= p.n);
    if constexpr (FUSED) ok = ok && p.peer_vec;
    return ok;
}

}  // namespace bq
