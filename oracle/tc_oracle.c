/*
 * TEST INFRASTRUCTURE - not part of the product.  See tc_oracle.h.
 *
 * Plain-C restatement of the reference's portable-CPU arithmetic for the quantized-decode
 * path.  Written from the reference's behaviour, with the same operation order wherever the
 * order changes a rounding, so that results are bit-identical to the reference's CPU backend.
 * Build with -ffp-contract=off (no fused multiply-add may replace a multiply and an add).
 */
#include "tc_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define Q4_BLOCK_BYTES 18u
#define Q8_BLOCK_BYTES 34u

static inline uint32_t bits_of(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float float_of(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* lib/core/cpu_float.h:20-43 - exact widening, including subnormals, infinities and NaN
 * payloads.  A binary16 subnormal is mant * 2^-24, which binary32 represents exactly. */
float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    const uint32_t m = h & 0x3ffu;
    if (e == 0x1fu) return float_of(sign | 0x7f800000u | (m << 13));
    if (e != 0) return float_of(sign | ((e + 112u) << 23) | (m << 13));
    /* zero or subnormal */
    float mag = ldexpf((float)m, -24);
    return float_of(sign | bits_of(mag));
}

/* lib/core/cpu_float.h:45-74 - round to nearest, ties to even; overflow gives infinity;
 * every NaN becomes the quiet pattern 0x7e00 with the input's sign; results below half of the
 * smallest subnormal flush to signed zero. */
uint16_t orc_f32_to_f16(float f) {
    const uint32_t b = bits_of(f);
    const uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    const uint32_t a = b & 0x7fffffffu;

    if (a >= 0x7f800000u) return (uint16_t)(sign | (a > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);          /* >= 65536 */
    if (a < 0x33000000u) return sign;                                  /* < 2^-25   */
    if (a < 0x38800000u) {                                             /* subnormal result */
        const uint32_t e = a >> 23;                                    /* 102..112 */
        const uint32_t m = (a & 0x7fffffu) | 0x800000u;
        const uint32_t sh = 126u - e;                                  /* 14..24 */
        const uint32_t r = m + ((1u << (sh - 1)) - 1u) + ((m >> sh) & 1u);
        return (uint16_t)(sign | (r >> sh));
    }
    /* normal result: add the rounding increment to the whole word so that a mantissa carry
     * moves into the exponent by itself, then re-bias. */
    const uint32_t r = a + 0xfffu + ((a >> 13) & 1u);
    const uint32_t h = (r - 0x38000000u) >> 13;
    return (uint16_t)(sign | (h >= 0x7c00u ? 0x7c00u : h));
}

void orc_f32_to_f16_array(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_f32_to_f16(src[i]);
}
void orc_f16_to_f32_array(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_f16_to_f32(src[i]);
}

static unsigned block_bytes(int fmt) {
    return fmt == 0 ? Q4_BLOCK_BYTES : (fmt == 1 ? Q8_BLOCK_BYTES : 0u);
}

/* lib/ops/quantized_cpu.cpp:90-100 */
size_t orc_quantized_size(int fmt, int N, int K) {
    const unsigned bb = block_bytes(fmt);
    if (N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return 0;
    return (size_t)N * (size_t)(K / 32) * bb;
}

static inline uint16_t load_u16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline void store_u16(uint8_t* p, uint16_t v) { memcpy(p, &v, 2); }

/* lib/ops/quantized_cpu.cpp:102-162.
 * Per 32-weight block: a = max |w| taken in fp32 (a NaN never wins the comparison); the stored
 * scale is fp16(a / d0) with d0 = 8 (Q4_0) or 127 (Q8_0); codes are lround(w * (d0 / a)),
 * biased by +8 and clamped to [0,15] for Q4_0, clamped to [-128,127] for Q8_0.  An all-zero
 * block has scale 0 and inverse 0, hence codes 8 (bytes 0x88) / 0.  Q4_0 byte i carries weight
 * i in its low nibble and weight i+16 in its high nibble. */
int orc_quantize_weights(const uint16_t* W, uint8_t* out, int fmt, int N, int K) {
    const unsigned bb = block_bytes(fmt);
    if (!W || !out || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return -1;
    const int nb = K / 32;
    const float d0 = (fmt == 0) ? 8.0f : 127.0f;
    for (int n = 0; n < N; ++n) {
        for (int b = 0; b < nb; ++b) {
            const uint16_t* src = W + (size_t)n * K + (size_t)b * 32;
            uint8_t* dst = out + ((size_t)n * nb + b) * bb;
            float w[32];
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                w[i] = orc_f16_to_f32(src[i]);
                const float av = fabsf(w[i]);
                if (amax < av) amax = av;
            }
            const float scale = amax / d0;
            const float inv = (scale > 0.0f) ? d0 / amax : 0.0f;
            store_u16(dst, orc_f32_to_f16(scale));
            if (fmt == 0) {
                for (int i = 0; i < 16; ++i) {
                    int lo = (int)lroundf(w[i] * inv) + 8;
                    int hi = (int)lroundf(w[i + 16] * inv) + 8;
                    if (lo < 0) lo = 0; else if (lo > 15) lo = 15;
                    if (hi < 0) hi = 0; else if (hi > 15) hi = 15;
                    dst[2 + i] = (uint8_t)((hi << 4) | lo);
                }
            } else {
                for (int i = 0; i < 32; ++i) {
                    int q = (int)lroundf(w[i] * inv);
                    if (q < -128) q = -128; else if (q > 127) q = 127;
                    dst[2 + i] = (uint8_t)(int8_t)q;
                }
            }
        }
    }
    return 0;
}

/* The dot product of one activation row (already widened to fp32) with one quantized weight
 * row, in the reference's order: blocks ascending; inside a Q4_0 block byte i contributes
 * x[i]*d*(lo-8) then x[i+16]*d*(hi-8); every product is (x*d)*q with two roundings and is then
 * added to a single fp32 accumulator (lib/ops/quantized_cpu.cpp:193-225, 286-314). */
static float row_dot(const float* x, const uint8_t* row, int fmt, int nb) {
    float acc = 0.0f;
    if (fmt == 0) {
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = row + (size_t)b * Q4_BLOCK_BYTES;
            const float d = orc_f16_to_f32(load_u16(blk));
            const float* xb = x + (size_t)b * 32;
            for (int i = 0; i < 16; ++i) {
                const uint8_t p = blk[2 + i];
                acc += xb[i] * d * (float)((int)(p & 0x0f) - 8);
                acc += xb[i + 16] * d * (float)((int)(p >> 4) - 8);
            }
        }
    } else {
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = row + (size_t)b * Q8_BLOCK_BYTES;
            const float d = orc_f16_to_f32(load_u16(blk));
            const int8_t* qs = (const int8_t*)(blk + 2);
            const float* xb = x + (size_t)b * 32;
            for (int i = 0; i < 32; ++i) acc += xb[i] * d * (float)qs[i];
        }
    }
    return acc;
}

int orc_gemv_quantized_rows(const uint16_t* X, const uint8_t* Wq, uint16_t* Y,
                            int fmt, int M, int N, int K, int n_begin, int n_end) {
    const unsigned bb = block_bytes(fmt);
    if (!X || !Wq || !Y || M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return -1;
    if (n_begin < 0 || n_end > N || n_begin > n_end) return -1;
    const int nb = K / 32;
    float* x = (float*)malloc((size_t)K * sizeof(float));
    if (!x) return -1;
    for (int m = 0; m < M; ++m) {
        orc_f16_to_f32_array(X + (size_t)m * K, x, (size_t)K);
        for (int n = n_begin; n < n_end; ++n) {
            const float acc = row_dot(x, Wq + (size_t)n * nb * bb, fmt, nb);
            Y[(size_t)m * N + n] = orc_f32_to_f16(acc);
        }
    }
    free(x);
    return 0;
}

/* lib/ops/quantized_cpu.cpp:164-230 */
int orc_gemv_quantized(const uint16_t* X, const uint8_t* Wq, uint16_t* Y,
                       int fmt, int M, int N, int K) {
    return orc_gemv_quantized_rows(X, Wq, Y, fmt, M, N, K, 0, N);
}

int orc_gemv_quantized_f32(const float* X, const uint8_t* Wq, float* Y,
                           int fmt, int M, int N, int K) {
    const unsigned bb = block_bytes(fmt);
    if (!X || !Wq || !Y || M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return -1;
    const int nb = K / 32;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n)
            Y[(size_t)m * N + n] = row_dot(X + (size_t)m * K, Wq + (size_t)n * nb * bb, fmt, nb);
    return 0;
}

/* lib/ops/quantized_cpu.cpp:272-284: sum of squares in double, rstd = 1/sqrtf(float(ss/K)+eps),
 * normalised row = (x * rstd) * gamma kept in fp32. */
static void rmsnorm_row_f32(const float* x, const float* g, float* out, int K, float eps) {
    double ss = 0.0;
    for (int k = 0; k < K; ++k) ss += (double)x[k] * (double)x[k];
    const float rstd = 1.0f / sqrtf((float)(ss / (double)K) + eps);
    for (int k = 0; k < K; ++k) out[k] = x[k] * rstd * g[k];
}

int orc_fused_rmsnorm_gemv_quantized_f32(const float* X, const float* gamma, const uint8_t* Wq,
                                         float* Y, int fmt, int M, int N, int K, float eps) {
    const unsigned bb = block_bytes(fmt);
    if (!X || !gamma || !Wq || !Y || M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0)
        return -1;
    const int nb = K / 32;
    float* xn = (float*)malloc((size_t)K * sizeof(float));
    if (!xn) return -1;
    for (int m = 0; m < M; ++m) {
        rmsnorm_row_f32(X + (size_t)m * K, gamma, xn, K, eps);
        for (int n = 0; n < N; ++n)
            Y[(size_t)m * N + n] = row_dot(xn, Wq + (size_t)n * nb * bb, fmt, nb);
    }
    free(xn);
    return 0;
}

/* lib/ops/quantized_cpu.cpp:232-320 */
int orc_fused_rmsnorm_gemv_quantized(const uint16_t* X, const uint16_t* gamma,
                                     const uint8_t* Wq, uint16_t* Y,
                                     int fmt, int M, int N, int K, float eps) {
    const unsigned bb = block_bytes(fmt);
    if (!X || !gamma || !Wq || !Y || M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0)
        return -1;
    const int nb = K / 32;
    float* buf = (float*)malloc((size_t)K * 3 * sizeof(float));
    if (!buf) return -1;
    float* x = buf; float* g = buf + K; float* xn = buf + 2 * (size_t)K;
    orc_f16_to_f32_array(gamma, g, (size_t)K);
    for (int m = 0; m < M; ++m) {
        orc_f16_to_f32_array(X + (size_t)m * K, x, (size_t)K);
        rmsnorm_row_f32(x, g, xn, K, eps);
        for (int n = 0; n < N; ++n)
            Y[(size_t)m * N + n] =
                orc_f32_to_f16(row_dot(xn, Wq + (size_t)n * nb * bb, fmt, nb));
    }
    free(buf);
    return 0;
}

/* Dense product of the reference's portable GEMM for fp16 in / fp16 out / fp32 accumulate,
 * alpha = 1, beta = 0 (lib/ops/gemm_cpu.cpp:544-568): k ascending, one fp32 accumulator,
 * stored value = 1*sum + 0*0. */
static void dense_rows_times_w(const uint16_t* xn, const uint16_t* W, uint16_t* Y,
                               int M, int N, int K) {
    float* wcol = (float*)malloc((size_t)K * sizeof(float));
    float* xr = (float*)malloc((size_t)M * K * sizeof(float));
    orc_f16_to_f32_array(xn, xr, (size_t)M * K);
    for (int n = 0; n < N; ++n) {
        for (int k = 0; k < K; ++k) wcol[k] = orc_f16_to_f32(W[(size_t)k * N + n]);
        for (int m = 0; m < M; ++m) {
            const float* x = xr + (size_t)m * K;
            float sum = 0.0f;
            for (int k = 0; k < K; ++k) sum += x[k] * wcol[k];
            const float out = 1.0f * sum + 0.0f * 0.0f;
            Y[(size_t)m * N + n] = orc_f32_to_f16(out);
        }
    }
    free(wcol);
    free(xr);
}

/* lib/ops/training_cpu.cpp:799-856: RMSNorm as above, but the normalised row is rounded to
 * fp16 before the product. */
int orc_fused_rmsnorm_gemv(const uint16_t* X, const uint16_t* gamma, const uint16_t* W,
                           uint16_t* Y, int M, int N, int K, float eps) {
    if (!X || !gamma || !W || !Y || M <= 0 || N <= 0 || K <= 0) return -1;
    uint16_t* xn = (uint16_t*)malloc((size_t)M * K * sizeof(uint16_t));
    if (!xn) return -1;
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = X + (size_t)m * K;
        double ss = 0.0;
        for (int k = 0; k < K; ++k) {
            const float xv = orc_f16_to_f32(xr[k]);
            ss += (double)xv * (double)xv;
        }
        const float rstd = 1.0f / sqrtf((float)(ss / K) + eps);
        for (int k = 0; k < K; ++k)
            xn[(size_t)m * K + k] =
                orc_f32_to_f16(orc_f16_to_f32(xr[k]) * rstd * orc_f16_to_f32(gamma[k]));
    }
    dense_rows_times_w(xn, W, Y, M, N, K);
    free(xn);
    return 0;
}

/* The narrowing the reference's GEMM uses for its result (lib/ops/gemm_cpu.cpp:142-160), which is
 * not the IEEE one of the quantized path: it adds the first dropped bit (ties go up, not to even)
 * and ORs the sum into the exponent field, so a mantissa that carries out lands in the exponent
 * only when the exponent's low bit was 0 (1.9998 becomes 1.0, not 2.0).  Kept for pinning the loop
 * below against the reference bit for bit; parity targets use the IEEE narrowing. */
static uint16_t gemm_ref_f32_to_f16(float x) {
    union { float f; uint32_t u; } v = {x};
    const uint32_t f = v.u;
    const uint32_t sign = (f >> 16) & 0x8000u;
    int32_t exp = (int32_t)((f >> 23) & 0xFF) - 127 + 15;
    uint32_t mant = f & 0x7FFFFFu;
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        mant |= 0x800000u;
        const uint32_t shift = (uint32_t)(14 - exp);
        const uint32_t round = (mant >> (shift - 1)) & 1u;
        return (uint16_t)(sign | ((mant >> shift) + round));
    }
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0u));
    const uint32_t round = (mant >> 12) & 1u;
    return (uint16_t)(sign | ((uint32_t)exp << 10) | ((mant >> 13) + round));
}

/* lib/ops/gemm_cpu.cpp:544-568 (the binary16 case): row-major A [M,K] or, transposed, [K,M] (lda), B [K,N] or, transposed,
 * [N,K] (ldb), C [M,N] (ldc); the products are added in k order in fp32;
 * C = fp16(alpha * sum + beta * C), C not read when beta is 0.  ref_narrowing: 0 = IEEE
 * round-to-nearest-even, 1 = the reference GEMM's own narrowing (see above). */
/* The bfloat16 case of the same loop: widening is a shift, narrowing round-to-nearest-even on the
 * dropped 16 bits (lib/ops/gemm_cpu.cpp:217-230). */
static float gemm_bf16_to_f32(uint16_t b) {
    union { uint32_t u; float f; } v = { (uint32_t)b << 16 };
    return v.f;
}
static uint16_t gemm_f32_to_bf16(float f) {
    union { float f; uint32_t u; } v = { f };
    const uint32_t lower = v.u & 0xFFFFu, upper = v.u >> 16;
    const uint32_t round = (lower > 0x8000u) || ((lower == 0x8000u) && (upper & 1u));
    return (uint16_t)(upper + round);
}
int orc_gemm_bf16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K,
                  int lda, int ldb, int ldc, int transpose_a, int transpose_b, float alpha, float beta) {
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return -1;
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int k = 0; k < K; ++k) {
                const uint16_t av = transpose_a ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k];
                const uint16_t bv = transpose_b ? B[(size_t)n * ldb + k] : B[(size_t)k * ldb + n];
                sum += gemm_bf16_to_f32(av) * gemm_bf16_to_f32(bv);
            }
            const size_t idx = (size_t)m * ldc + n;
            const float prev = (beta == 0.0f) ? 0.0f : gemm_bf16_to_f32(C[idx]);
            C[idx] = gemm_f32_to_bf16(alpha * sum + beta * prev);
        }
    }
    return 0;
}

int orc_gemm_f16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K,
                 int lda, int ldb, int ldc, int transpose_a, int transpose_b, float alpha, float beta, int ref_narrowing) {
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return -1;
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int k = 0; k < K; ++k) {
                const uint16_t av = transpose_a ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k];
                const uint16_t bv = transpose_b ? B[(size_t)n * ldb + k] : B[(size_t)k * ldb + n];
                sum += orc_f16_to_f32(av) * orc_f16_to_f32(bv);
            }
            const size_t idx = (size_t)m * ldc + n;
            const float prev = (beta == 0.0f) ? 0.0f : orc_f16_to_f32(C[idx]);
            const float out = alpha * sum + beta * prev;
            C[idx] = ref_narrowing ? gemm_ref_f32_to_f16(out) : orc_f32_to_f16(out);
        }
    }
    return 0;
}

/* lib/ops/training_cpu.cpp:858-935: mean in double then narrowed to fp32; centred second
 * moment in double; rstd = 1/sqrtf(float(var)+eps); row = fp16(((x-mean)*rstd)*gamma + beta). */
int orc_fused_layernorm_gemv(const uint16_t* X, const uint16_t* gamma, const uint16_t* beta,
                             const uint16_t* W, uint16_t* Y, int M, int N, int K, float eps) {
    if (!X || !gamma || !beta || !W || !Y || M <= 0 || N <= 0 || K <= 0) return -1;
    uint16_t* xn = (uint16_t*)malloc((size_t)M * K * sizeof(uint16_t));
    if (!xn) return -1;
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = X + (size_t)m * K;
        double sum = 0.0;
        for (int k = 0; k < K; ++k) sum += orc_f16_to_f32(xr[k]);
        const float mean = (float)(sum / K);
        double ss = 0.0;
        for (int k = 0; k < K; ++k) {
            const float c = orc_f16_to_f32(xr[k]) - mean;
            ss += (double)c * (double)c;
        }
        const float rstd = 1.0f / sqrtf((float)(ss / K) + eps);
        for (int k = 0; k < K; ++k) {
            const float xv = orc_f16_to_f32(xr[k]);
            const float gv = orc_f16_to_f32(gamma[k]);
            const float bv = orc_f16_to_f32(beta[k]);
            xn[(size_t)m * K + k] = orc_f32_to_f16((xv - mean) * rstd * gv + bv);
        }
    }
    dense_rows_times_w(xn, W, Y, M, N, K);
    free(xn);
    return 0;
}

/* lib/ops/training_cpu.cpp:126-186: sum of squares in double, rstd = 1/sqrtf(float(ss/D)+eps),
 * y = fp16((x*rstd)*gamma); rstd saved per row. */
int orc_rmsnorm_forward(const uint16_t* X, const uint16_t* gamma, uint16_t* Y, float* rstd_out,
                        int N, int D, float eps) {
    if (!X || !gamma || !Y || !rstd_out || N <= 0 || D <= 0) return -1;
    for (int n = 0; n < N; ++n) {
        const uint16_t* xr = X + (size_t)n * D;
        uint16_t* yr = Y + (size_t)n * D;
        double ss = 0.0;
        for (int d = 0; d < D; ++d) {
            const float xv = orc_f16_to_f32(xr[d]);
            ss += (double)xv * xv;
        }
        const float rstd = 1.0f / sqrtf((float)(ss / D) + eps);
        rstd_out[n] = rstd;
        for (int d = 0; d < D; ++d)
            yr[d] = orc_f32_to_f16(orc_f16_to_f32(xr[d]) * rstd * orc_f16_to_f32(gamma[d]));
    }
    return 0;
}

/* lib/ops/training_cpu.cpp:287-350: mean in double narrowed to fp32, centred second moment in
 * double, y = fp16(((x-mean)*rstd)*gamma + beta); mean and rstd saved per row. */
int orc_layernorm_forward(const uint16_t* X, const uint16_t* gamma, const uint16_t* beta,
                          uint16_t* Y, float* mean_out, float* rstd_out, int N, int D, float eps) {
    if (!X || !gamma || !beta || !Y || !mean_out || !rstd_out || N <= 0 || D <= 0) return -1;
    for (int n = 0; n < N; ++n) {
        const uint16_t* xr = X + (size_t)n * D;
        uint16_t* yr = Y + (size_t)n * D;
        double s = 0.0;
        for (int d = 0; d < D; ++d) s += orc_f16_to_f32(xr[d]);
        const float mean = (float)(s / D);
        double sq = 0.0;
        for (int d = 0; d < D; ++d) {
            const float c = orc_f16_to_f32(xr[d]) - mean;
            sq += (double)c * c;
        }
        const float rstd = 1.0f / sqrtf((float)(sq / D) + eps);
        mean_out[n] = mean;
        rstd_out[n] = rstd;
        for (int d = 0; d < D; ++d)
            yr[d] = orc_f32_to_f16((orc_f16_to_f32(xr[d]) - mean) * rstd * orc_f16_to_f32(gamma[d]) +
                                   orc_f16_to_f32(beta[d]));
    }
    return 0;
}

/* lib/ops/training_cpu.cpp:94-101,541-573: out = fp16(silu(gate) * up), silu(x) = x/(1+expf(-x)),
 * 0 below -50, x above 50. */
int orc_swiglu_forward(const uint16_t* gate, const uint16_t* up, uint16_t* out, int n) {
    if (!gate || !up || !out || n <= 0) return -1;
    for (int i = 0; i < n; ++i) {
        const float g = orc_f16_to_f32(gate[i]), u = orc_f16_to_f32(up[i]);
        float s;
        if (g < -50.0f) s = 0.0f;
        else if (g > 50.0f) s = g;
        else s = g / (1.0f + expf(-g));
        out[i] = orc_f32_to_f16(s * u);
    }
    return 0;
}

/* lib/ops/training_cpu.cpp:427-482: in place on X[B,H,S,D]; pairs (k, k + D/2) rotated by the
 * angle whose cosine and sine are cos_t / sin_t[s][k] (fp32 tables [S, D/2]). */
int orc_rope_forward(uint16_t* X, const float* cos_t, const float* sin_t, int batch, int heads,
                     int seq, int head_dim) {
    if (!X || !cos_t || !sin_t || batch <= 0 || heads <= 0 || seq <= 0 || head_dim <= 0 || head_dim % 2)
        return -1;
    const int half = head_dim / 2;
    const long total = (long)batch * heads * seq;
    for (long bhs = 0; bhs < total; ++bhs) {
        const int s_idx = (int)(bhs % seq);
        uint16_t* xr = X + (size_t)bhs * head_dim;
        for (int k = 0; k < half; ++k) {
            const float x0 = orc_f16_to_f32(xr[k]), x1 = orc_f16_to_f32(xr[k + half]);
            const float c = cos_t[(size_t)s_idx * half + k], si = sin_t[(size_t)s_idx * half + k];
            xr[k] = orc_f32_to_f16(x0 * c - x1 * si);
            xr[k + half] = orc_f32_to_f16(x0 * si + x1 * c);
        }
    }
    return 0;
}

/* lib/ops/attention_cpu.cpp:62-83 (dot_order 1: eight running sums updated with fused multiply-adds,
 * then folded 8 -> 4 -> 2 -> 1, the tail added element by element) and :100-106 (dot_order 0: one
 * running sum, multiply then add).  The reference picks the first on x86 CPUs with AVX2, F16C and FMA. */
static float attn_dot(const uint16_t* a, const uint16_t* b, int n, int dot_order) {
    if (dot_order == 0) {
        float acc = 0.0f;
        for (int i = 0; i < n; ++i) acc += orc_f16_to_f32(a[i]) * orc_f16_to_f32(b[i]);
        return acc;
    }
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 7 < n; i += 8)
        for (int k = 0; k < 8; ++k) acc[k] = fmaf(orc_f16_to_f32(a[i + k]), orc_f16_to_f32(b[i + k]), acc[k]);
    float s4[4];
    for (int k = 0; k < 4; ++k) s4[k] = acc[k] + acc[k + 4];
    const float s2a = s4[0] + s4[2], s2b = s4[1] + s4[3];
    float result = s2a + s2b;
    for (; i < n; ++i) result += orc_f16_to_f32(a[i]) * orc_f16_to_f32(b[i]);
    return result;
}

/* lib/ops/attention_cpu.cpp:131-277: Q [B,Hq,Sq,D], K/V [B,Hkv,Sk,D], O [B,Hq,Sq,D] fp16, LSE
 * [B,Hq,Sq] fp32 or NULL.  Tiles of 32 query rows x 32 keys with a running maximum, denominator and
 * unnormalised output per row (:57-58, :185-255); mask order causal, window, then ALiBi (:203-214). */
int orc_attention_forward(const uint16_t* Q, const uint16_t* K, const uint16_t* V, uint16_t* O, float* LSE,
                          int B, int Hq, int Hkv, int Sq, int Sk, int D, float softmax_scale, int causal,
                          int window, const float* alibi_slopes, int dot_order) {
    if (!Q || !K || !V || !O || B <= 0 || Hq <= 0 || Sq <= 0 || Sk <= 0 || D <= 0) return -1;
    if (Hkv <= 0) Hkv = Hq;
    if (Hq % Hkv != 0) return -1;
    enum { BR = 32, BC = 32 };
    const int per = Hq / Hkv;
    const float scale = softmax_scale > 0 ? softmax_scale : 1.0f / sqrtf((float)D);
    float* o_state = (float*)malloc(sizeof(float) * BR * (size_t)D);
    if (!o_state) return -2;
    float m_state[BR], l_state[BR], s_tile[BR * BC];
    for (long bh = 0; bh < (long)B * Hq; ++bh) {
        const int b = (int)(bh / Hq), h = (int)(bh % Hq), hkv = h / per;
        const uint16_t* Qbh = Q + ((size_t)b * Hq + h) * Sq * D;
        const uint16_t* Kbh = K + ((size_t)b * Hkv + hkv) * Sk * D;
        const uint16_t* Vbh = V + ((size_t)b * Hkv + hkv) * Sk * D;
        uint16_t* Obh = O + ((size_t)b * Hq + h) * Sq * D;
        float* Lbh = LSE ? LSE + ((size_t)b * Hq + h) * Sq : NULL;
        for (int qb = 0; qb < Sq; qb += BR) {
            const int br = Sq - qb < BR ? Sq - qb : BR;
            for (int r = 0; r < br; ++r) { m_state[r] = -INFINITY; l_state[r] = 0.0f; }
            memset(o_state, 0, sizeof(float) * (size_t)br * D);
            for (int kb = 0; kb < Sk; kb += BC) {
                const int bc = Sk - kb < BC ? Sk - kb : BC;
                for (int r = 0; r < br; ++r)
                    for (int cidx = 0; cidx < bc; ++cidx) {
                        float sc = attn_dot(Qbh + (size_t)(qb + r) * D, Kbh + (size_t)(kb + cidx) * D, D, dot_order) * scale;
                        if (causal && (kb + cidx) > (qb + r)) sc = -INFINITY;
                        if (window > 0 && (qb + r) - (kb + cidx) > window) sc = -INFINITY;
                        if (alibi_slopes) sc -= alibi_slopes[h] * (float)((qb + r) - (kb + cidx));
                        s_tile[r * BC + cidx] = sc;
                    }
                for (int r = 0; r < br; ++r) {
                    float m_new = m_state[r];
                    for (int cidx = 0; cidx < bc; ++cidx)
                        if (s_tile[r * BC + cidx] > m_new) m_new = s_tile[r * BC + cidx];
                    if (!isfinite(m_new)) m_new = m_state[r];
                    const float scale_old = (m_state[r] == -INFINITY) ? 0.0f : expf(m_state[r] - m_new);
                    float l_new = l_state[r] * scale_old;
                    for (int d = 0; d < D; ++d) o_state[r * D + d] *= scale_old;
                    for (int cidx = 0; cidx < bc; ++cidx) {
                        const float p = expf(s_tile[r * BC + cidx] - m_new);
                        if (!isfinite(p)) continue;
                        l_new += p;
                        const uint16_t* Vrow = Vbh + (size_t)(kb + cidx) * D;
                        for (int d = 0; d < D; ++d) o_state[r * D + d] += p * orc_f16_to_f32(Vrow[d]);
                    }
                    m_state[r] = m_new;
                    l_state[r] = l_new;
                }
            }
            for (int r = 0; r < br; ++r) {
                const float inv_l = l_state[r] != 0.0f ? 1.0f / l_state[r] : 0.0f;
                for (int d = 0; d < D; ++d) Obh[(size_t)(qb + r) * D + d] = orc_f32_to_f16(o_state[r * D + d] * inv_l);
                if (Lbh) Lbh[qb + r] = m_state[r] + logf(l_state[r] > 1e-30f ? l_state[r] : 1e-30f);
            }
        }
    }
    free(o_state);
    return 0;
}

int orc_dequantize(const uint8_t* Wq, float* out, int fmt, int N, int K) {
    const unsigned bb = block_bytes(fmt);
    if (!Wq || !out || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return -1;
    const size_t nblk = (size_t)N * (size_t)(K / 32);
    for (size_t t = 0; t < nblk; ++t) {
        const uint8_t* blk = Wq + t * bb;
        const float d = orc_f16_to_f32(load_u16(blk));
        float* o = out + t * 32;
        if (fmt == 0) {
            for (int i = 0; i < 16; ++i) {
                o[i] = d * (float)((int)(blk[2 + i] & 0x0f) - 8);
                o[i + 16] = d * (float)((int)(blk[2 + i] >> 4) - 8);
            }
        } else {
            for (int i = 0; i < 32; ++i) o[i] = d * (float)(int8_t)blk[2 + i];
        }
    }
    return 0;
}

/* tests/test_quantized.c:48-94 - the fp64 yardstick: dequantise each stored block in double
 * and dot it with the activations in double. */
int orc_dequant_dot_f64(const double* X, const uint8_t* Wq, double* Y,
                        int fmt, int M, int N, int K) {
    const unsigned bb = block_bytes(fmt);
    if (!X || !Wq || !Y || M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || bb == 0) return -1;
    const int nb = K / 32;
    for (int n = 0; n < N; ++n) {
        const uint8_t* row = Wq + (size_t)n * nb * bb;
        for (int m = 0; m < M; ++m) {
            const double* x = X + (size_t)m * K;
            double acc = 0.0;
            for (int b = 0; b < nb; ++b) {
                const uint8_t* blk = row + (size_t)b * bb;
                const double d = (double)orc_f16_to_f32(load_u16(blk));
                const double* xb = x + (size_t)b * 32;
                if (fmt == 0) {
                    for (int i = 0; i < 16; ++i) {
                        acc += xb[i] * d * (double)((int)(blk[2 + i] & 0x0f) - 8);
                        acc += xb[i + 16] * d * (double)((int)(blk[2 + i] >> 4) - 8);
                    }
                } else {
                    for (int i = 0; i < 32; ++i) acc += xb[i] * d * (double)(int8_t)blk[2 + i];
                }
            }
            Y[(size_t)m * N + n] = acc;
        }
    }
    return 0;
}
