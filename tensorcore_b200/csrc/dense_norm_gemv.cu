// Fused RMSNorm / LayerNorm + dense fp16 GEMV for sm_100a:
//   Y[M,N] = fp16( norm(X)[M,K] . W[K,N] ),  W row-major with N contiguous.
//
// The normalised row is rounded to fp16 before the product (as the reference's CPU path does)
// and products are accumulated in fp32 with the mixed-precision FMA.  HBM-bound: W is read
// once, 2 bytes per weight.  A CTA owns a strip of 32 columns (64-byte row segments) and all of
// K; its 256 threads are 64 k-lanes x 4 column chunks of 16 bytes, each thread keeps several
// independent 128-bit loads in flight.  The norm statistics are recomputed per CTA (K values
// from L2), which is cheaper than a separate kernel and an fp16 round trip.
#include "kernels.h"

#include <cuda_fp16.h>

namespace tcb {
namespace {

constexpr int kDThreads = 256;
constexpr int kDWarps = kDThreads / 32;
constexpr int kStripCols = 32;
constexpr int kKLanes = kDThreads / 4;  // 64
constexpr int kDMaxMB = 4;

__device__ __forceinline__ float fma_h16(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float hf(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ double dblock_sum(double v, double* scratch) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < kDWarps; ++i) t += scratch[i];
    return t;
}

struct DenseParams {
    const __half* X;
    const __half* gamma;
    const __half* beta;   // null => RMSNorm
    const __half* W;
    __half* Y;
    int M, N, K;
    float eps;
};

// Normalises MB rows into shared memory as fp16.
//   RMSNorm:   ss = sum x^2 (double); rstd = 1/sqrtf(float(ss/K)+eps); xn = fp16((x*rstd)*g)
//   LayerNorm: mean = float(sum x (double) / K); var = sum (x-mean)^2 (double) / K;
//              rstd = 1/sqrtf(float(var)+eps); xn = fp16(((x-mean)*rstd)*g + b)
template <int MB>
__device__ void normalise_rows(const DenseParams& p, __half* xn, double* scratch) {
    const int tid = threadIdx.x, K = p.K;
    for (int m = 0; m < MB; ++m) {
        const __half* xr = p.X + static_cast<size_t>(m) * K;
        float mean = 0.f;
        if (p.beta != nullptr) {
            double s = 0.0;
            for (int k = tid; k < K; k += kDThreads) s += static_cast<double>(__half2float(xr[k]));
            s = dblock_sum(s, scratch);
            mean = static_cast<float>(s / K);
        }
        double ss = 0.0;
        for (int k = tid; k < K; k += kDThreads) {
            const float c = __fsub_rn(__half2float(xr[k]), mean);
            ss += static_cast<double>(c) * static_cast<double>(c);
        }
        ss = dblock_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(static_cast<float>(ss / K) + p.eps);
        for (int k = tid; k < K; k += kDThreads) {
            const float xv = __half2float(xr[k]);
            const float gv = __half2float(p.gamma[k]);
            float o;
            if (p.beta != nullptr) {
                const float bv = __half2float(p.beta[k]);
                o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xv, mean), rstd), gv), bv);
            } else {
                o = __fmul_rn(__fmul_rn(xv, rstd), gv);
            }
            xn[static_cast<size_t>(m) * K + k] = __float2half_rn(o);
        }
    }
    __syncthreads();
}

template <int MB>
__global__ void __launch_bounds__(kDThreads) dense_norm_gemv_kernel(const DenseParams p) {
    extern __shared__ __align__(16) uint8_t dsm[];
    double* scratch = reinterpret_cast<double*>(dsm);                 // kDWarps doubles
    float* red = reinterpret_cast<float*>(dsm + 64);                  // [kDWarps][4][8][MB]
    __half* xn = reinterpret_cast<__half*>(dsm + 64 + kDWarps * 4 * 8 * kDMaxMB * 4);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    normalise_rows<MB>(p, xn, scratch);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cc = tid & 3, kl = tid >> 2;
    const int col = blockIdx.x * kStripCols + cc * 8;
    const bool active = col < p.N;
    float acc[MB][8];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[m][e] = 0.f;

    if (active) {
        const uint4* wp = reinterpret_cast<const uint4*>(p.W + col);
        const size_t ldw = static_cast<size_t>(p.N) / 8;  // row stride in uint4
        constexpr int U = 4;
        int k = kl;
        for (; k + (U - 1) * kKLanes < p.K; k += U * kKLanes) {
            uint4 wv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) wv[u] = __ldg(wp + static_cast<size_t>(k + u * kKLanes) * ldw);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const uint16_t xb = __half_as_ushort(xn[static_cast<size_t>(m) * p.K + k + u * kKLanes]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[m][2 * e] = fma_h16(xb, static_cast<uint16_t>(ww[e]), acc[m][2 * e]);
                        acc[m][2 * e + 1] = fma_h16(xb, static_cast<uint16_t>(ww[e] >> 16), acc[m][2 * e + 1]);
                    }
                }
            }
        }
        for (; k < p.K; k += kKLanes) {
            const uint4 wv = __ldg(wp + static_cast<size_t>(k) * ldw);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const uint16_t xb = __half_as_ushort(xn[static_cast<size_t>(m) * p.K + k]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[m][2 * e] = fma_h16(xb, static_cast<uint16_t>(ww[e]), acc[m][2 * e]);
                    acc[m][2 * e + 1] = fma_h16(xb, static_cast<uint16_t>(ww[e] >> 16), acc[m][2 * e + 1]);
                }
            }
        }
    }
    // Reduce over the 8 k-lanes of a warp (lane bits 2..4), then over the 8 warps.
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float v = acc[m][e];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[m][e] = v;
        }
    if (lane < 4) {
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int e = 0; e < 8; ++e) red[((warp * 4 + lane) * 8 + e) * MB + m] = acc[m][e];
    }
    __syncthreads();
    if (tid < kStripCols * MB) {
        const int c = tid / MB, m = tid - c * MB;  // c = column within the strip
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kDWarps; ++w) v += red[((w * 4 + (c >> 3)) * 8 + (c & 7)) * MB + m];
        const int n = blockIdx.x * kStripCols + c;
        if (n < p.N) p.Y[static_cast<size_t>(m) * p.N + n] = __float2half_rn(v);
    }
}

// Fallback for N % 8 != 0 or unaligned W: one thread per column, scalar loads (still
// coalesced across the warp).
template <int MB>
__global__ void __launch_bounds__(kDThreads) dense_norm_gemv_scalar_kernel(const DenseParams p) {
    extern __shared__ __align__(16) uint8_t dsm[];
    double* scratch = reinterpret_cast<double*>(dsm);
    __half* xn = reinterpret_cast<__half*>(dsm + 64);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    normalise_rows<MB>(p, xn, scratch);
    const int n = blockIdx.x * kDThreads + threadIdx.x;
    if (n >= p.N) return;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f;
    for (int k = 0; k < p.K; ++k) {
        const uint16_t wb = __half_as_ushort(p.W[static_cast<size_t>(k) * p.N + n]);
#pragma unroll
        for (int m = 0; m < MB; ++m)
            acc[m] = fma_h16(__half_as_ushort(xn[static_cast<size_t>(m) * p.K + k]), wb, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) p.Y[static_cast<size_t>(m) * p.N + n] = __float2half_rn(acc[m]);
}

template <int MB>
cudaError_t launch_dense_mb(const DenseParams& p, bool vec, int smem_optin, cudaStream_t st,
                            bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kDThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const size_t xn_bytes = static_cast<size_t>(MB) * p.K * 2;
    if (vec) {
        cfg.gridDim = dim3((p.N + kStripCols - 1) / kStripCols);
        cfg.dynamicSmemBytes = 64 + kDWarps * 4 * 8 * kDMaxMB * 4 + xn_bytes;
        if (static_cast<int>(cfg.dynamicSmemBytes) > smem_optin) return cudaErrorInvalidValue;
        cudaError_t e = cudaFuncSetAttribute(dense_norm_gemv_kernel<MB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(cfg.dynamicSmemBytes));
        if (e != cudaSuccess) return e;
        return cudaLaunchKernelEx(&cfg, dense_norm_gemv_kernel<MB>, p);
    }
    cfg.gridDim = dim3((p.N + kDThreads - 1) / kDThreads);
    cfg.dynamicSmemBytes = 64 + xn_bytes;
    if (static_cast<int>(cfg.dynamicSmemBytes) > smem_optin) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(dense_norm_gemv_scalar_kernel<MB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(cfg.dynamicSmemBytes));
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, dense_norm_gemv_scalar_kernel<MB>, p);
}

}  // namespace

cudaError_t launch_dense_norm_gemv(const DenseNormGemvArgs& a, const LaunchEnv& env,
                                   cudaStream_t stream, int* launches, const char** name) {
    const bool vec = (a.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.W) & 15u) == 0);
    const int optin = env.smem_optin > 0 ? env.smem_optin : 48 * 1024;
    cudaError_t err = cudaSuccess;
    int count = 0;
    for (int m0 = 0; m0 < a.M && err == cudaSuccess; m0 += kDMaxMB) {
        const int mb = (a.M - m0) < kDMaxMB ? (a.M - m0) : kDMaxMB;
        DenseParams p;
        p.X = static_cast<const __half*>(a.X) + static_cast<size_t>(m0) * a.K;
        p.gamma = static_cast<const __half*>(a.gamma);
        p.beta = static_cast<const __half*>(a.beta);
        p.W = static_cast<const __half*>(a.W);
        p.Y = static_cast<__half*>(a.Y) + static_cast<size_t>(m0) * a.N;
        p.M = mb; p.N = a.N; p.K = a.K; p.eps = a.eps;
        switch (mb) {
            case 1: err = launch_dense_mb<1>(p, vec, optin, stream, env.pdl); break;
            case 2: err = launch_dense_mb<2>(p, vec, optin, stream, env.pdl); break;
            case 3: err = launch_dense_mb<3>(p, vec, optin, stream, env.pdl); break;
            default: err = launch_dense_mb<4>(p, vec, optin, stream, env.pdl); break;
        }
        ++count;
    }
    if (launches) *launches += count;
    if (name) *name = a.beta ? "layernorm_gemv_f16_sm100" : "rmsnorm_gemv_f16_sm100";
    return err;
}

}  // namespace tcb
