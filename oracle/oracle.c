/*
 * CPU oracle for the quantized-GEMM hot path — TEST INFRASTRUCTURE ONLY.
 * See oracle.h for what each function restates and which reference tests pin it.
 * Parity status: pinned (reference known-answer tests + torch e4m3 cross-check).
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------ */
/* codecs                                                                     */
/* ------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

/* oracle.rs:397-404 — add 0x7fff plus the lsb of the kept half, truncate. */
uint16_t orc_f32_to_bf16_bits(float x) {
    uint32_t bits = f32_bits(x);
    if (x != x) {
        return (uint16_t)((bits >> 16) | 0x0040u);
    }
    uint32_t bias = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}

/* oracle.rs:339-341 — bf16 is the top half of an f32. */
float orc_bf16_bits_to_f32(uint16_t bits) { return bits_f32(((uint32_t)bits) << 16); }

float orc_e4m3_to_f32(uint8_t b) {
    int sign = b >> 7;
    int exp = (b >> 3) & 0xF;
    int man = b & 0x7;
    float v;
    if (exp == 0xF && man == 0x7) {
        v = NAN;
    } else if (exp == 0) {
        v = ldexpf((float)man, -9); /* subnormal: man * 2^-9 */
    } else {
        v = ldexpf((float)(8 + man), exp - 7 - 3);
    }
    return sign ? -v : v;
}

uint8_t orc_f32_to_e4m3_satfinite(float x) {
    uint8_t sign = (uint8_t)((f32_bits(x) >> 31) << 7);
    if (x != x) {
        return (uint8_t)(sign | 0x7Fu);
    }
    double a = fabs((double)x);
    if (a >= 448.0) {
        return (uint8_t)(sign | 0x7Eu); /* saturate to the largest finite value */
    }
    if (a < 0.015625) { /* below 2^-6: fixed quantum 2^-9; q == 8 lands on the first normal */
        int q = (int)nearbyint(a * 512.0);
        return (uint8_t)(sign | (uint8_t)q);
    }
    int e;
    (void)frexp(a, &e); /* a = f * 2^e, f in [0.5, 1) */
    int E = e - 1;      /* 2^E <= a < 2^(E+1) */
    int q = (int)nearbyint(ldexp(a, 3 - E)); /* in [8, 16] */
    if (q == 16) {
        q = 8;
        E += 1;
    }
    return (uint8_t)(sign | (uint8_t)(((E + 7) << 3) | (q - 8)));
}

/* ------------------------------------------------------------------------ */
/* the contraction interpreter (oracle.rs:1289-1372)                          */
/* ------------------------------------------------------------------------ */

/* raw_to_f64 (oracle.rs:451-464): integers sign-extend, bf16 widens. */
static inline double load_as_f64(int dtype, const void* base, int64_t off) {
    switch (dtype) {
        case ORC_F32: return (double)((const float*)base)[off];
        case ORC_F64: return ((const double*)base)[off];
        case ORC_BF16: return (double)orc_bf16_bits_to_f32(((const uint16_t*)base)[off]);
        case ORC_I32: return (double)((const int32_t*)base)[off];
        case ORC_S8: return (double)((const int8_t*)base)[off];
        case ORC_I64: return (double)((const int64_t*)base)[off];
        default: return NAN;
    }
}

/* Rust `f as iN`: truncate toward zero, saturate, NaN -> 0. */
static inline int64_t sat_cast(double f, int64_t lo, int64_t hi) {
    if (f != f) return 0;
    if (f <= (double)lo) return lo;
    if (f >= (double)hi) return hi;
    return (int64_t)f;
}

/* encode_float (oracle.rs:918-933). */
static inline void store_from_f64(int dtype, void* base, int64_t off, double f) {
    switch (dtype) {
        case ORC_F32: ((float*)base)[off] = (float)f; break;
        case ORC_F64: ((double*)base)[off] = f; break;
        case ORC_BF16: ((uint16_t*)base)[off] = orc_f32_to_bf16_bits((float)f); break;
        case ORC_I32: ((int32_t*)base)[off] = (int32_t)sat_cast(f, INT32_MIN, INT32_MAX); break;
        case ORC_S8: ((int8_t*)base)[off] = (int8_t)sat_cast(f, INT8_MIN, INT8_MAX); break;
        case ORC_I64: ((int64_t*)base)[off] = sat_cast(f, INT64_MIN, INT64_MAX); break;
        default: break;
    }
}

int orc_contraction(int dtype, int64_t bdim, int64_t m, int64_t n, int64_t k,
                    const void* lhs, const int64_t ls[3],
                    const void* rhs, const int64_t rs[3],
                    const void* bias,
                    void* out, const int64_t os[3],
                    int epilogue) {
    if (dtype < ORC_F32 || dtype > ORC_I64) return 2;
    if (epilogue < ORC_EPI_IDENTITY || epilogue > ORC_EPI_BIAS_RELU) return 2;
    int needs_bias = (epilogue == ORC_EPI_BIAS || epilogue == ORC_EPI_BIAS_RELU);
    if (needs_bias && bias == NULL) return 2;
    for (int64_t bi = 0; bi < bdim; ++bi) {
        for (int64_t mi = 0; mi < m; ++mi) {
            for (int64_t ni = 0; ni < n; ++ni) {
                double acc = 0.0; /* K-sum, kk ascending */
                for (int64_t kk = 0; kk < k; ++kk) {
                    double a = load_as_f64(dtype, lhs, bi * ls[0] + mi * ls[1] + kk * ls[2]);
                    double b = load_as_f64(dtype, rhs, bi * rs[0] + kk * rs[1] + ni * rs[2]);
                    acc += a * b;
                }
                double v = acc;
                if (needs_bias) v += load_as_f64(dtype, bias, ni);
                if (epilogue == ORC_EPI_RELU || epilogue == ORC_EPI_BIAS_RELU) {
                    if (!(v > 0.0)) v = (v != v) ? v : 0.0;
                }
                store_from_f64(dtype, out, bi * os[0] + mi * os[1] + ni * os[2], v);
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* fast equal cells                                                           */
/* ------------------------------------------------------------------------ */

/* dot of two contiguous s8 rows in int32 (auto-vectorised). */
static inline int32_t dot_s8(const int8_t* __restrict a, const int8_t* __restrict b, int32_t k) {
    int32_t acc = 0;
    for (int32_t i = 0; i < k; ++i) acc += (int32_t)a[i] * (int32_t)b[i];
    return acc;
}

int orc_gemm_s8_s32(int32_t m, int32_t n, int32_t k,
                    const int8_t* a, int64_t lda,
                    const int8_t* b, int64_t ldb, int b_layout,
                    int32_t* acc, int64_t ldacc) {
    if (m < 0 || n < 0 || k < 0) return 2;
    if (b_layout != ORC_LAYOUT_RRR && b_layout != ORC_LAYOUT_RCR) return 2;
    if (b_layout == ORC_LAYOUT_RCR) {
#pragma omp parallel for schedule(static)
        for (int32_t i = 0; i < m; ++i) {
            const int8_t* ar = a + (int64_t)i * lda;
            for (int32_t j = 0; j < n; ++j) {
                acc[(int64_t)i * ldacc + j] = dot_s8(ar, b + (int64_t)j * ldb, k);
            }
        }
    } else {
        /* row-major B: accumulate rank-1 updates along each output row. When
         * there are fewer rows than threads (the decode GEMV), split columns
         * instead so every core streams its own slice of B. */
        int nthreads = orc_num_threads();
        if (m >= nthreads) {
#pragma omp parallel for schedule(static)
            for (int32_t i = 0; i < m; ++i) {
                int32_t* row = acc + (int64_t)i * ldacc;
                for (int32_t j = 0; j < n; ++j) row[j] = 0;
                for (int32_t kk = 0; kk < k; ++kk) {
                    int32_t av = (int32_t)a[(int64_t)i * lda + kk];
                    const int8_t* br = b + (int64_t)kk * ldb;
                    for (int32_t j = 0; j < n; ++j) row[j] += av * (int32_t)br[j];
                }
            }
        } else {
            const int32_t chunk = 512;
            int32_t nchunks = (n + chunk - 1) / chunk;
#pragma omp parallel for schedule(static)
            for (int32_t c = 0; c < nchunks; ++c) {
                int32_t j0 = c * chunk;
                int32_t j1 = j0 + chunk < n ? j0 + chunk : n;
                for (int32_t i = 0; i < m; ++i) {
                    int32_t* row = acc + (int64_t)i * ldacc;
                    for (int32_t j = j0; j < j1; ++j) row[j] = 0;
                    for (int32_t kk = 0; kk < k; ++kk) {
                        int32_t av = (int32_t)a[(int64_t)i * lda + kk];
                        const int8_t* br = b + (int64_t)kk * ldb;
                        for (int32_t j = j0; j < j1; ++j) row[j] += av * (int32_t)br[j];
                    }
                }
            }
        }
    }
    return 0;
}

void orc_dequant_s32_bf16(int32_t m, int32_t n, const int32_t* acc, int64_t ldacc,
                          const float* sa, const float* sb,
                          uint16_t* out, int64_t ldo) {
#pragma omp parallel for schedule(static)
    for (int32_t i = 0; i < m; ++i) {
        for (int32_t j = 0; j < n; ++j) {
            float s = sa[i] * sb[j]; /* (sa*sw) first, then *acc — no contraction */
            float y = s * (float)acc[(int64_t)i * ldacc + j];
            out[(int64_t)i * ldo + j] = orc_f32_to_bf16_bits(y);
        }
    }
}

void orc_dequant_s32_f32(int32_t m, int32_t n, const int32_t* acc, int64_t ldacc,
                         const float* sa, const float* sb,
                         float* out, int64_t ldo) {
#pragma omp parallel for schedule(static)
    for (int32_t i = 0; i < m; ++i) {
        for (int32_t j = 0; j < n; ++j) {
            float s = sa[i] * sb[j];
            out[(int64_t)i * ldo + j] = s * (float)acc[(int64_t)i * ldacc + j];
        }
    }
}

int orc_gemm_e4m3_f32(int32_t m, int32_t n, int32_t k,
                      const uint8_t* a, int64_t lda,
                      const uint8_t* b, int64_t ldb, int b_layout,
                      float* acc, int64_t ldacc) {
    if (m < 0 || n < 0 || k < 0) return 2;
    if (b_layout != ORC_LAYOUT_RRR && b_layout != ORC_LAYOUT_RCR) return 2;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_to_f32((uint8_t)i);
#pragma omp parallel
    {
        float* arow = (float*)malloc(sizeof(float) * (size_t)(k > 0 ? k : 1));
#pragma omp for schedule(static)
        for (int32_t i = 0; i < m; ++i) {
            for (int32_t kk = 0; kk < k; ++kk) arow[kk] = lut[a[(int64_t)i * lda + kk]];
            for (int32_t j = 0; j < n; ++j) {
                double s = 0.0;
                if (b_layout == ORC_LAYOUT_RCR) {
                    const uint8_t* bc = b + (int64_t)j * ldb;
                    for (int32_t kk = 0; kk < k; ++kk) s += (double)arow[kk] * (double)lut[bc[kk]];
                } else {
                    for (int32_t kk = 0; kk < k; ++kk)
                        s += (double)arow[kk] * (double)lut[b[(int64_t)kk * ldb + j]];
                }
                acc[(int64_t)i * ldacc + j] = (float)s;
            }
        }
        free(arow);
    }
    return 0;
}

void orc_scale_f32_bf16(int32_t m, int32_t n, const float* acc, int64_t ldacc,
                        const float* sa, int sa_is_vector,
                        const float* sb, int sb_is_vector,
                        uint16_t* out, int64_t ldo) {
#pragma omp parallel for schedule(static)
    for (int32_t i = 0; i < m; ++i) {
        float a = sa_is_vector ? sa[i] : sa[0];
        for (int32_t j = 0; j < n; ++j) {
            float bsc = sb_is_vector ? sb[j] : sb[0];
            float s = a * bsc;
            out[(int64_t)i * ldo + j] = orc_f32_to_bf16_bits(s * acc[(int64_t)i * ldacc + j]);
        }
    }
}

static inline int32_t sat_add32(int32_t x, int32_t y) {
    int64_t s = (int64_t)x + (int64_t)y;
    if (s > INT32_MAX) return INT32_MAX;
    if (s < INT32_MIN) return INT32_MIN;
    return (int32_t)s;
}

int orc_int_gemm_s8_out(int32_t m, int32_t n, int32_t k,
                        const int8_t* a, int64_t lda,
                        const int8_t* b, int64_t ldb, int b_layout,
                        const int8_t* c, int64_t ldc,
                        const float* bias, float alpha, float beta,
                        int8_t* d, int64_t ldd) {
    if (m < 0 || n < 0 || k < 0) return 2;
    if (b_layout != ORC_LAYOUT_RRR && b_layout != ORC_LAYOUT_RCR) return 2;
#pragma omp parallel for schedule(static)
    for (int32_t i = 0; i < m; ++i) {
        for (int32_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (int32_t kk = 0; kk < k; ++kk) {
                int32_t av = a[(int64_t)i * lda + kk];
                int32_t bv = (b_layout == ORC_LAYOUT_RCR) ? b[(int64_t)j * ldb + kk]
                                                          : b[(int64_t)kk * ldb + j];
                acc = sat_add32(acc, av * bv);
            }
            float z = alpha * (float)acc;
            if (c) {
                float t = beta * (float)c[(int64_t)i * ldc + j];
                z = z + t;
            }
            if (bias) z = z + bias[j];
            float r = nearbyintf(z);
            if (r < -128.0f) r = -128.0f;
            if (r > 127.0f) r = 127.0f;
            d[(int64_t)i * ldd + j] = (int8_t)r;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* quantizers                                                                 */
/* ------------------------------------------------------------------------ */

void orc_quantize_rows_s8(int32_t rows, int32_t cols, int32_t qmin, int32_t qmax,
                          const float* x, int64_t ldx, float* scale, int8_t* q, int64_t ldq) {
#pragma omp parallel for schedule(static)
    for (int32_t r = 0; r < rows; ++r) {
        const float* xr = x + (int64_t)r * ldx;
        float amax = 0.0f;
        for (int32_t c = 0; c < cols; ++c) {
            float v = fabsf(xr[c]);
            if (v > amax) amax = v;
        }
        float s = (amax > 0.0f) ? (amax / (float)qmax) : 1.0f;
        scale[r] = s;
        float inv = (s != 0.0f) ? (1.0f / s) : 0.0f;
        for (int32_t c = 0; c < cols; ++c) {
            float t = xr[c] * inv;
            int32_t v = (int32_t)nearbyintf(t);
            if (v < qmin) v = qmin;
            if (v > qmax) v = qmax;
            q[(int64_t)r * ldq + c] = (int8_t)v;
        }
    }
}

void orc_quantize_rows_e4m3(int32_t rows, int32_t cols,
                            const float* x, int64_t ldx, float* scale, uint8_t* q, int64_t ldq) {
#pragma omp parallel for schedule(static)
    for (int32_t r = 0; r < rows; ++r) {
        const float* xr = x + (int64_t)r * ldx;
        float amax = 0.0f;
        for (int32_t c = 0; c < cols; ++c) {
            float v = fabsf(xr[c]);
            if (v > amax) amax = v;
        }
        float s = (amax > 0.0f) ? (amax / 448.0f) : 1.0f;
        scale[r] = s;
        float inv = 1.0f / s;
        for (int32_t c = 0; c < cols; ++c) {
            float t = xr[c] * inv;
            q[(int64_t)r * ldq + c] = orc_f32_to_e4m3_satfinite(t);
        }
    }
}

void orc_quantize_tensor_e4m3(int64_t count, const float* x, float* scale, uint8_t* q) {
    float amax = 0.0f;
    for (int64_t i = 0; i < count; ++i) {
        float v = fabsf(x[i]);
        if (v > amax) amax = v;
    }
    float s = (amax > 0.0f) ? (amax / 448.0f) : 1.0f;
    *scale = s;
    float inv = 1.0f / s;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float t = x[i] * inv;
        q[i] = orc_f32_to_e4m3_satfinite(t);
    }
}

/* ------------------------------------------------------------------------ */
/* comparator                                                                 */
/* ------------------------------------------------------------------------ */

int64_t orc_compare_bitexact(const void* expected, const void* actual, size_t elem_size, int64_t count) {
    const uint8_t* e = (const uint8_t*)expected;
    const uint8_t* a = (const uint8_t*)actual;
    if (memcmp(e, a, elem_size * (size_t)count) == 0) return -1;
    for (int64_t i = 0; i < count; ++i) {
        if (memcmp(e + (size_t)i * elem_size, a + (size_t)i * elem_size, elem_size) != 0) return i;
    }
    return -1;
}

int64_t orc_compare_tolerant_f32(const float* expected, const float* actual, int64_t count,
                                 double rel, double abs_tol) {
    for (int64_t i = 0; i < count; ++i) {
        double e = expected[i], a = actual[i];
        if (e != e && a != a) continue;
        if (e == a) continue;
        if (isinf(e) || isinf(a)) return i;
        double diff = fabs(e - a);
        double mag = fabs(e) > fabs(a) ? fabs(e) : fabs(a);
        if (diff <= abs_tol + rel * mag) continue;
        return i; /* also catches a NaN on one side only */
    }
    return -1;
}
