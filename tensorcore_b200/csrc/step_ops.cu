// The small operations that sit between the GEMVs of a decode step: RMSNorm and LayerNorm
// forward (with the saved statistics the reference's backward passes read), SwiGLU, rotary
// embedding, and a plain fp16 GEMM for the few rows a decode step has.  All are streaming or
// tiny; they follow the reference's portable-CPU arithmetic (fp32 math on fp16 data, one rounding
// per stored value; statistics accumulated in double, lib/ops/training_cpu.cpp:126-186,287-350,
// 427-482,541-573).
#include "kernels.h"

#include <cuda_fp16.h>

namespace tcb {
namespace {

__device__ double block_sum_d(double v, double* scratch) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) scratch[w] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; ++i) t += scratch[i];
    return t;
}

// One CTA per row.  beta == nullptr: RMSNorm, else LayerNorm (mean subtracted, two passes).
__global__ void __launch_bounds__(256) norm_forward_kernel(const __half* X, const __half* gamma,
                                                           const __half* beta, __half* Y, float* mean_out,
                                                           float* rstd_out, int D, float eps) {
    __shared__ double scratch[8];
    // A kernel launched behind this one with programmatic serialization (the batched GEMV that
    // reads the normalised rows) may begin its prologue and weight copies while the rows are made.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int n = blockIdx.x;
    const __half* xr = X + static_cast<size_t>(n) * D;
    __half* yr = Y + static_cast<size_t>(n) * D;
    float mean = 0.f;
    if (beta != nullptr) {
        double s = 0.0;
        for (int d = threadIdx.x; d < D; d += blockDim.x) s += static_cast<double>(__half2float(xr[d]));
        mean = static_cast<float>(block_sum_d(s, scratch) / D);
    }
    double sq = 0.0;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float c = __fsub_rn(__half2float(xr[d]), mean);
        sq += static_cast<double>(c) * static_cast<double>(c);
    }
    const float rstd = 1.0f / sqrtf(static_cast<float>(block_sum_d(sq, scratch) / D) + eps);
    if (threadIdx.x == 0) {
        rstd_out[n] = rstd;
        if (mean_out) mean_out[n] = mean;
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float xv = __half2float(xr[d]), gv = __half2float(gamma[d]);
        float y;
        if (beta != nullptr)
            y = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xv, mean), rstd), gv), __half2float(beta[d]));
        else
            y = __fmul_rn(__fmul_rn(xv, rstd), gv);
        yr[d] = __float2half_rn(y);
    }
}

// out = silu(gate) * up, silu(x) = x / (1 + exp(-x)) with the reference's tail clamps.
__global__ void swiglu_kernel(const __half* gate, const __half* up, __half* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = __half2float(gate[i]), u = __half2float(up[i]);
    float s;
    if (g < -50.0f) s = 0.0f;
    else if (g > 50.0f) s = g;
    else s = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    out[i] = __float2half_rn(__fmul_rn(s, u));
}

// In-place rotation of the halves of every [head_dim] vector of X[B,H,S,D]; tables [S, D/2] fp32.
__global__ void rope_kernel(__half* X, const float* cos_t, const float* sin_t, long total_pairs, int seq, int half) {
    const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total_pairs) return;
    const long bhs = i / half;
    const int k = static_cast<int>(i - bhs * half);
    const int s = static_cast<int>(bhs % seq);
    __half* xr = X + bhs * 2 * half;
    const float x0 = __half2float(xr[k]), x1 = __half2float(xr[k + half]);
    const float c = cos_t[static_cast<size_t>(s) * half + k], si = sin_t[static_cast<size_t>(s) * half + k];
    xr[k] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, si)));
    xr[k + half] = __float2half_rn(__fadd_rn(__fmul_rn(x0, si), __fmul_rn(x1, c)));
}

// C[M,N] = alpha * A[M,K] . B[K,N] + beta * C, fp16 storage, fp32 accumulation in k order (the
// reference's triple loop, lib/ops/gemm_cpu.cpp:544-568).  A thread per output column and a CTA
// row of A in shared memory: meant for the handful of rows of a decode step, not for training.
__global__ void __launch_bounds__(128) gemm_f16_rows_kernel(const __half* A, const __half* B, __half* C, int N, int K,
                                                            int lda, int ldb, int ldc, float alpha, float beta) {
    extern __shared__ float a_row[];
    const int m = blockIdx.y, n = blockIdx.x * blockDim.x + threadIdx.x;
    for (int k = threadIdx.x; k < K; k += blockDim.x) a_row[k] = __half2float(A[static_cast<size_t>(m) * lda + k]);
    __syncthreads();
    if (n >= N) return;
    float acc = 0.f;
    for (int k = 0; k < K; ++k) acc = fmaf(a_row[k], __half2float(B[static_cast<size_t>(k) * ldb + n]), acc);
    float v = alpha * acc;
    if (beta != 0.f) v += beta * __half2float(C[static_cast<size_t>(m) * ldc + n]);
    C[static_cast<size_t>(m) * ldc + n] = __float2half_rn(v);
}

}  // namespace

cudaError_t launch_norm_forward(const void* X, const void* gamma, const void* beta, void* Y, float* mean_out,
                                float* rstd_out, int N, int D, float eps, cudaStream_t stream) {
    norm_forward_kernel<<<N, 256, 0, stream>>>(static_cast<const __half*>(X), static_cast<const __half*>(gamma),
                                               static_cast<const __half*>(beta), static_cast<__half*>(Y), mean_out,
                                               rstd_out, D, eps);
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const void* gate, const void* up, void* out, int n, cudaStream_t stream) {
    swiglu_kernel<<<(n + 255) / 256, 256, 0, stream>>>(static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                                       static_cast<__half*>(out), n);
    return cudaGetLastError();
}

cudaError_t launch_rope(void* X, const float* cos_t, const float* sin_t, int batch, int heads, int seq, int head_dim,
                        cudaStream_t stream) {
    const int half = head_dim / 2;
    const long pairs = static_cast<long>(batch) * heads * seq * half;
    rope_kernel<<<static_cast<unsigned>((pairs + 255) / 256), 256, 0, stream>>>(static_cast<__half*>(X), cos_t, sin_t,
                                                                                pairs, seq, half);
    return cudaGetLastError();
}

cudaError_t launch_gemm_f16_rows(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                 float alpha, float beta, cudaStream_t stream) {
    if (static_cast<size_t>(K) * sizeof(float) > 48 * 1024 || M > 65535) return cudaErrorNotSupported;
    const dim3 grid((N + 127) / 128, M);
    gemm_f16_rows_kernel<<<grid, 128, static_cast<size_t>(K) * sizeof(float), stream>>>(
        static_cast<const __half*>(A), static_cast<const __half*>(B), static_cast<__half*>(C), N, K, lda, ldb, ldc,
        alpha, beta);
    return cudaGetLastError();
}

}  // namespace tcb
