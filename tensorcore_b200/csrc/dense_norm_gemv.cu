// Fused RMSNorm / LayerNorm + dense fp16 GEMV for sm_100a:
//   Y[M,N] = fp16( norm(X)[M,K] . W[K,N] ),  W row-major with N contiguous.
//
// The normalised row is rounded to fp16 before the product (as the reference's CPU path does)
// and products are accumulated in fp32 with the mixed-precision FMA.  HBM-bound: W is read
// once, 2 bytes per weight.
//
// Main kernel (dense_norm_gemv_split_kernel): W is cut into tiles of 256 columns (512-byte row
// segments: a warp copies one, 16 bytes per lane) by a K range chosen so that there are about
// four tiles per SM - the hardware spreads them evenly, and three CTAs per SM keep 144 KB of
// copies in flight.  A CTA starts the asynchronous copies of its first stages (cp.async into a
// four-stage ring in shared memory; a thread reads back exactly the pieces it copied, so the
// ring needs no barrier), works out the row statistics meanwhile (K values from L2; cheaper than
// a separate kernel and an fp16 round trip), normalises its K range into shared memory, streams
// its tile and leaves its partial sums in scratch;
// the CTA that finishes a column strip last adds the strip's partial sums in K order - the result
// does not depend on which CTA that is - and writes fp16 Y.  The scratch (partial sums and one
// ticket counter per strip, which the last CTA resets) belongs to the stream the call runs on.
//
// Without scratch, for N not a multiple of 8 or an unaligned W: a CTA owns a strip of 32 columns
// and all of K (dense_norm_gemv_kernel), or one thread owns a column (scalar kernel).
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

// Statistics of row m for the split kernel: mean (LayerNorm) and 1/std or 1/rms, the reference's
// arithmetic (double-precision sums, lib/ops/training_cpu.cpp:799-935).
__device__ void row_stats(const DenseParams& p, int m, double* scratch, float& mean, float& rstd) {
    const int tid = threadIdx.x, K = p.K;
    const __half* xr = p.X + static_cast<size_t>(m) * K;
    mean = 0.f;
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
    rstd = 1.0f / sqrtf(static_cast<float>(ss / K) + p.eps);
}

constexpr int kSplitCols = 256;          // columns of a tile: 512 contiguous bytes per row, one warp-wide copy
constexpr int kRowGroups = kDThreads / 32;   // 8: a warp per row
constexpr int kStageRows = 32;           // rows of W per ring stage: 16 KB
constexpr int kStages = 4;               // ring depth: three stages (48 KB) in flight per CTA
constexpr int kStageBytes = kStageRows * kSplitCols * 2;

struct SplitParams {
    DenseParams d;
    float* partial;      // [chunks][M][N]
    int* counters;       // [strips], zero between launches
    int kc;              // K rows per tile (a multiple of kStageRows)
    int chunks;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool live) {
    // zero-fills when the row lies beyond the tile
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int MB>
__global__ void __launch_bounds__(kDThreads) dense_norm_gemv_split_kernel(const SplitParams sp) {
    extern __shared__ __align__(128) uint8_t dsm[];
    double* scratch = reinterpret_cast<double*>(dsm);                 // kDWarps doubles
    int* ticket_s = reinterpret_cast<int*>(dsm + 64);
    uint8_t* ring = dsm + 128;                                        // kStages x 16 KB; reused for the reduction
    float* red = reinterpret_cast<float*>(ring);                      // [8][MB][256] floats <= 32 KB
    __half* xn = reinterpret_cast<__half*>(ring + kStages * kStageBytes);   // [MB][kc]
    const DenseParams& p = sp.d;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int strip = blockIdx.x, chunk = blockIdx.y;
    const int k0 = chunk * sp.kc, k1 = min(p.K, k0 + sp.kc);

    // A thread copies, and later reads back, its own 16-byte pieces: rows (tid >> 5) + 8 * j of a
    // stage, columns 8 * (tid & 31) .. + 7 of the strip.  So the ring needs no barrier: a copy
    // group's completion is all a thread waits for.
    const int hl = tid & 31, r0 = tid >> 5;
    const int col = strip * kSplitCols + hl * 8;
    const bool active = col < p.N;
    const __half* wcol = p.W + (active ? col : 0);
    const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
    const int n_stages = (k1 - k0 + kStageRows - 1) / kStageRows;
    auto issue = [&](int st) {
        if (st < n_stages) {
            const uint32_t dst = ring_s + (st % kStages) * kStageBytes + r0 * (kSplitCols * 2) + hl * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = k0 + st * kStageRows + r0 + kRowGroups * j;
                cp_async16(dst + j * kRowGroups * (kSplitCols * 2), wcol + static_cast<size_t>(k < k1 ? k : k0) * p.N, active && k < k1);
            }
        }
        cp_async_commit();
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int st = 0; st < kStages - 1; ++st) issue(st);      // the weights do not depend on the statistics

    for (int m = 0; m < MB; ++m) {
        float mean, rstd;
        row_stats(p, m, scratch, mean, rstd);
        const __half* xr = p.X + static_cast<size_t>(m) * p.K;
        for (int k = k0 + tid; k < k1; k += kDThreads) {
            const float xv = __half2float(xr[k]), gv = __half2float(p.gamma[k]);
            float o;
            if (p.beta != nullptr) {
                const float bv = __half2float(p.beta[k]);
                o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xv, mean), rstd), gv), bv);
            } else {
                o = __fmul_rn(__fmul_rn(xv, rstd), gv);
            }
            xn[m * sp.kc + (k - k0)] = __float2half_rn(o);
        }
    }
    __syncthreads();

    float acc[MB][8];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[m][e] = 0.f;
    for (int st = 0; st < n_stages; ++st) {
        issue(st + kStages - 1);
        cp_async_wait<kStages - 1>();
        const uint8_t* src = ring + (st % kStages) * kStageBytes + r0 * (kSplitCols * 2) + hl * 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kk = st * kStageRows + r0 + kRowGroups * j;     // row within the tile
            if (k0 + kk >= k1) break;
            const uint4 wv = *reinterpret_cast<const uint4*>(src + j * kRowGroups * (kSplitCols * 2));
            // fp16 x fp16 products are exact in fp32, so converting both sides first and using the
            // fp32 FMA gives the same bits as the mixed-precision FMA, with one conversion per pair
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
            float2 wf[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) wf[e] = __half22float2(wh[e]);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float xf = __half2float(xn[m * sp.kc + kk]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[m][2 * e] = fmaf(xf, wf[e].x, acc[m][2 * e]);
                    acc[m][2 * e + 1] = fmaf(xf, wf[e].y, acc[m][2 * e + 1]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();         // every thread is done with the ring: it now holds the partial sums
    // 8 row groups per column: through shared memory, added in a fixed order
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[(r0 * MB + m) * kSplitCols + hl * 8 + e] = acc[m][e];
    __syncthreads();
    for (int i = tid; i < MB * kSplitCols; i += kDThreads) {
        const int m = i / kSplitCols, c = i - m * kSplitCols;
        float v = 0.f;
#pragma unroll
        for (int g = 0; g < kRowGroups; ++g) v += red[(g * MB + m) * kSplitCols + c];
        const int n = strip * kSplitCols + c;
        if (n < p.N) sp.partial[(static_cast<size_t>(chunk) * p.M + m) * p.N + n] = v;
    }
    // The last CTA of the strip adds the K ranges in order and writes the result.
    __threadfence();
    __syncthreads();
    if (tid == 0) *ticket_s = atomicAdd(&sp.counters[strip], 1);
    __syncthreads();
    if (*ticket_s != sp.chunks - 1) return;
    __threadfence();
    for (int i = tid; i < MB * kSplitCols; i += kDThreads) {
        const int m = i / kSplitCols, c = i - m * kSplitCols;
        const int n = strip * kSplitCols + c;
        if (n >= p.N) continue;
        float v = 0.f;
        for (int ch = 0; ch < sp.chunks; ++ch)
            v += __ldcg(sp.partial + (static_cast<size_t>(ch) * p.M + m) * p.N + n);
        p.Y[static_cast<size_t>(m) * p.N + n] = __float2half_rn(v);
    }
    if (tid == 0) sp.counters[strip] = 0;      // ready for the next launch on this stream
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

template <int MB>
cudaError_t launch_dense_split(const SplitParams& sp, int strips, int smem_optin, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kDThreads);
    cfg.gridDim = dim3(strips, sp.chunks);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cfg.dynamicSmemBytes = 128 + kStages * kStageBytes + static_cast<size_t>(MB) * sp.kc * 2;
    if (static_cast<int>(cfg.dynamicSmemBytes) > smem_optin) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(dense_norm_gemv_split_kernel<MB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(cfg.dynamicSmemBytes));
    if (e != cudaSuccess) return e;
    return cudaLaunchKernelEx(&cfg, dense_norm_gemv_split_kernel<MB>, sp);
}

// Tiles of the split kernel for one launch of up to kDMaxMB rows.
void dense_split_shape(int N, int K, int sm_count, int* strips, int* chunks, int* kc) {
    // about four tiles per SM (three CTAs are resident per SM; more, shorter tiles measured slower:
    // every tile pays for the row statistics and for a fence before its ticket), K ranges of whole
    // ring stages
    const int st = (N + kSplitCols - 1) / kSplitCols;
    int ch = (4 * sm_count + st - 1) / st;
    const int most = (K + 2 * kStageRows - 1) / (2 * kStageRows);
    if (ch > most) ch = most;
    if (ch < 1) ch = 1;
    int rows = (K + ch - 1) / ch;
    rows = (rows + kStageRows - 1) / kStageRows * kStageRows;
    *strips = st;
    *kc = rows;
    *chunks = (K + rows - 1) / rows;
}

}  // namespace

void dense_norm_gemv_scratch(int M, int N, int K, int sm_count, size_t* floats, size_t* ints) {
    int strips, chunks, kc;
    dense_split_shape(N, K, sm_count, &strips, &chunks, &kc);
    const int mb = M < kDMaxMB ? M : kDMaxMB;
    *floats = static_cast<size_t>(chunks) * mb * N;
    *ints = static_cast<size_t>(strips);
}

cudaError_t launch_dense_norm_gemv(const DenseNormGemvArgs& a, const LaunchEnv& env,
                                   cudaStream_t stream, int* launches, const char** name) {
    const bool vec = (a.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.W) & 15u) == 0);
    const int optin = env.smem_optin > 0 ? env.smem_optin : 48 * 1024;
    cudaError_t err = cudaSuccess;
    int count = 0;
    size_t need_f = 0, need_i = 0;
    dense_norm_gemv_scratch(a.M, a.N, a.K, env.sm_count > 0 ? env.sm_count : 148, &need_f, &need_i);
    const bool split = vec && a.scratch && a.counters && a.scratch_floats >= need_f && a.counters_n >= need_i;
    // Five rows or more: the kernels below would read W once per four rows.  Instead the rows are
    // normalised once into the stream's scratch (fp16, as the reference rounds them before its GEMM,
    // lib/ops/training_cpu.cpp:799-935) and multiplied by W on the tensor cores: W is read once.
    const size_t rows_bytes = static_cast<size_t>(a.M) * a.K * 2;
    if (a.M >= 5 && a.norm_scratch && a.norm_scratch_bytes >= rows_bytes + static_cast<size_t>(a.M) * 8) {
        float* stats = reinterpret_cast<float*>(static_cast<uint8_t*>(a.norm_scratch) + rows_bytes);
        cudaError_t e = launch_norm_forward(a.X, a.gamma, a.beta, a.norm_scratch, stats, stats + a.M, a.M, a.K, a.eps, stream);
        if (e == cudaSuccess) {
            e = launch_gemm_f16_tc(a.norm_scratch, a.W, a.Y, a.M, a.N, a.K, a.K, a.N, a.N, false, 1.0f, 0.0f, env, stream);
            if (e == cudaSuccess) {
                if (launches) *launches += 2;
                if (name) *name = a.beta ? "layernorm_rows_gemm_tcgen05_sm100" : "rmsnorm_rows_gemm_tcgen05_sm100";
                return cudaSuccess;
            }
            if (e != cudaErrorNotSupported) return e;
            (void)cudaGetLastError();      // shapes the tiled copies cannot describe: the kernels below
        } else {
            return e;
        }
    }
    for (int m0 = 0; m0 < a.M && err == cudaSuccess; m0 += kDMaxMB) {
        const int mb = (a.M - m0) < kDMaxMB ? (a.M - m0) : kDMaxMB;
        DenseParams p;
        p.X = static_cast<const __half*>(a.X) + static_cast<size_t>(m0) * a.K;
        p.gamma = static_cast<const __half*>(a.gamma);
        p.beta = static_cast<const __half*>(a.beta);
        p.W = static_cast<const __half*>(a.W);
        p.Y = static_cast<__half*>(a.Y) + static_cast<size_t>(m0) * a.N;
        p.M = mb; p.N = a.N; p.K = a.K; p.eps = a.eps;
        if (split) {
            SplitParams sp;
            sp.d = p;
            sp.partial = a.scratch;
            sp.counters = a.counters;
            int strips = 0;
            dense_split_shape(a.N, a.K, env.sm_count > 0 ? env.sm_count : 148, &strips, &sp.chunks, &sp.kc);
            switch (mb) {
                case 1: err = launch_dense_split<1>(sp, strips, optin, stream, env.pdl); break;
                case 2: err = launch_dense_split<2>(sp, strips, optin, stream, env.pdl); break;
                case 3: err = launch_dense_split<3>(sp, strips, optin, stream, env.pdl); break;
                default: err = launch_dense_split<4>(sp, strips, optin, stream, env.pdl); break;
            }
            ++count;
            continue;
        }
        switch (mb) {
            case 1: err = launch_dense_mb<1>(p, vec, optin, stream, env.pdl); break;
            case 2: err = launch_dense_mb<2>(p, vec, optin, stream, env.pdl); break;
            case 3: err = launch_dense_mb<3>(p, vec, optin, stream, env.pdl); break;
            default: err = launch_dense_mb<4>(p, vec, optin, stream, env.pdl); break;
        }
        ++count;
    }
    if (launches) *launches += count;
    if (name) *name = a.beta ? (split ? "layernorm_gemv_f16_split_sm100" : "layernorm_gemv_f16_sm100")
                             : (split ? "rmsnorm_gemv_f16_split_sm100" : "rmsnorm_gemv_f16_sm100");
    return err;
}

}  // namespace tcb
