/*
 * TEST INFRASTRUCTURE - not part of the product.
 *
 * CPU restatement, in plain C, of the arithmetic that tsotchke/tensorcore's portable-CPU
 * backend performs on the quantized-decode path.  Only the test suite, the smoke check and
 * the benchmark's CPU-baseline legs may load this; the shipped library never does.
 *
 * Every function works on plain host pointers.  "f16" buffers hold IEEE binary16 bit
 * patterns in uint16_t.  fmt: 0 = Q4_0 (18-byte blocks), 1 = Q8_0 (34-byte blocks).
 * Functions returning int give 0 on success, -1 on a rejected argument.
 *
 * Parity status: pinned.  tests/test_oracle.py checks this file against (a) the golden
 * vectors the reference's own tests hold for the path and (b) outputs of the reference's
 * CPU backend compiled from its sources (oracle/_ref), bit for bit.
 */
#ifndef TC_ORACLE_H
#define TC_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* binary16 <-> binary32, bit-compatible with lib/core/cpu_float.h:20-74. */
float    orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);
void     orc_f32_to_f16_array(const float* src, uint16_t* dst, size_t n);
void     orc_f16_to_f32_array(const uint16_t* src, float* dst, size_t n);

/* lib/ops/quantized_cpu.cpp:90-100 */
size_t orc_quantized_size(int fmt, int N, int K);

/* lib/ops/quantized_cpu.cpp:102-162 */
int orc_quantize_weights(const uint16_t* W_f16, uint8_t* W_quant, int fmt, int N, int K);

/* lib/ops/quantized_cpu.cpp:164-230.  X [M,K] f16, Y [M,N] f16. */
int orc_gemv_quantized(const uint16_t* X, const uint8_t* W_quant, uint16_t* Y,
                       int fmt, int M, int N, int K);

/* Same loop nest as orc_gemv_quantized with the binary16 conversions of X and Y removed:
 * fp32 activations in, fp32 results out (the reference ABI has no such entry point; this is
 * the checker for the additive fp32 entry points of the CUDA library). */
int orc_gemv_quantized_f32(const float* X, const uint8_t* W_quant, float* Y,
                           int fmt, int M, int N, int K);

/* lib/ops/quantized_cpu.cpp:232-320.  gamma [K] f16. */
int orc_fused_rmsnorm_gemv_quantized(const uint16_t* X, const uint16_t* gamma,
                                     const uint8_t* W_quant, uint16_t* Y,
                                     int fmt, int M, int N, int K, float eps);
/* fp32 X / gamma / Y form of the above (same arithmetic, no binary16 rounding). */
int orc_fused_rmsnorm_gemv_quantized_f32(const float* X, const float* gamma,
                                         const uint8_t* W_quant, float* Y,
                                         int fmt, int M, int N, int K, float eps);

/* lib/ops/training_cpu.cpp:799-856 with the GEMM of lib/ops/gemm_cpu.cpp:544-568.
 * W is dense f16 [K,N], N contiguous. */
int orc_fused_rmsnorm_gemv(const uint16_t* X, const uint16_t* gamma, const uint16_t* W,
                           uint16_t* Y, int M, int N, int K, float eps);
/* lib/ops/gemm_cpu.cpp:544-568, fp16 storage and fp32 accumulation in k order. */
int orc_gemm_f16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K,
                 int lda, int ldb, int ldc, int transpose_a, int transpose_b, float alpha, float beta, int ref_narrowing);
/* The bfloat16 case (conversions lib/ops/gemm_cpu.cpp:217-230); operands as raw 16-bit patterns. */
int orc_gemm_bf16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K,
                  int lda, int ldb, int ldc, int transpose_a, int transpose_b, float alpha, float beta);
/* lib/ops/training_cpu.cpp:858-935. */
int orc_fused_layernorm_gemv(const uint16_t* X, const uint16_t* gamma, const uint16_t* beta,
                             const uint16_t* W, uint16_t* Y, int M, int N, int K, float eps);

/* The operations between the GEMVs of a decode step.
 * lib/ops/training_cpu.cpp:126-186 / 287-350 / 541-573 / 427-482. */
int orc_rmsnorm_forward(const uint16_t* X, const uint16_t* gamma, uint16_t* Y, float* rstd_out,
                        int N, int D, float eps);
int orc_layernorm_forward(const uint16_t* X, const uint16_t* gamma, const uint16_t* beta,
                          uint16_t* Y, float* mean_out, float* rstd_out, int N, int D, float eps);
int orc_swiglu_forward(const uint16_t* gate, const uint16_t* up, uint16_t* out, int n);
int orc_rope_forward(uint16_t* X, const float* cos_t, const float* sin_t, int batch, int heads,
                     int seq, int head_dim);
int orc_attention_forward(const uint16_t* Q, const uint16_t* K, const uint16_t* V, uint16_t* O, float* LSE,
                          int B, int Hq, int Hkv, int Sq, int Sk, int D, float softmax_scale, int causal,
                          int window, const float* alibi_slopes, int dot_order);

/* Double-precision dequantise-and-dot of the stored blocks against X given as double,
 * the yardstick of tests/test_quantized.c:48-94.  Y is [M,N] double. */
int orc_dequant_dot_f64(const double* X, const uint8_t* W_quant, double* Y,
                        int fmt, int M, int N, int K);

/* Dequantise blocks to fp32 ([N,K]); value = d * (q - 8) for Q4_0, d * q for Q8_0. */
int orc_dequantize(const uint8_t* W_quant, float* W_out, int fmt, int N, int K);

/* Row-range form of orc_gemv_quantized used by the multi-threaded CPU baseline: computes
 * output rows [n_begin, n_end) only.  Same arithmetic, same results for those rows. */
int orc_gemv_quantized_rows(const uint16_t* X, const uint8_t* W_quant, uint16_t* Y,
                            int fmt, int M, int N, int K, int n_begin, int n_end);

#ifdef __cplusplus
}
#endif
#endif
