// Quantized GEMV for sm_100a: Y[M,N] = X[M,K] . dequant(W)^T with W in GGUF Q4_0 / Q8_0 blocks.
//
// The weight matrix is one contiguous byte array ([N] rows of K/32 blocks).  Each CTA owns a
// contiguous range of rows, i.e. one contiguous byte range, and streams it exactly once from
// HBM with 1-D bulk async copies (cp.async.bulk, the TMA engine) into per-warp shared-memory
// rings guarded by mbarriers.  The unit of work is a "group" of 8 consecutive blocks:
// 8*18 = 144 bytes (Q4_0) or 8*34 = 272 bytes (Q8_0) are the smallest runs of whole blocks
// whose size is a multiple of 16 bytes, so a lane can pull its group out of shared memory
// with conflict-free 128-bit loads (9 resp. 17 of them; the 16-byte stride count is odd) and
// pick scales and codes out of registers at compile-time-known positions.
//
// Codes become fp16 operands without an integer->float conversion: a 4-bit (8-bit) code c
// placed in the low mantissa bits of a binary16 is the subnormal c * 2^-24, so masking the
// packed word yields two ready fp16 values.  Products are taken with the sm_100 mixed
// precision FMA (fp16 x fp16 + fp32 -> fp32), which is exact in the product and rounds once
// in fp32; the zero point (-8 resp. the +128 bias used to make Q8_0 codes unsigned) is removed
// per block with a precomputed sum of the block's activations.
//
// Activations (M <= 4 rows per pass) live in shared memory in a chunk-transposed layout so that
// the 32 lanes of a warp, which work on 32 consecutive groups, read consecutive 16-byte
// chunks.  Per-lane partial sums are combined with a segmented warp-shuffle reduction (a warp's
// 32 groups may span several weight rows) and added to per-row accumulators in shared memory.
//
// With programmatic dependent launch the kernel starts its weight stream before waiting for
// the previous kernel in the stream, so consecutive GEMVs of a decode step overlap their
// fill/drain phases.  Every mbarrier wait is bounded; on expiry the kernel records
// ERR_WAIT_TIMEOUT, drains its outstanding copies (again bounded) and exits.
#include "kernels.h"
#include "sm100_prims.cuh"
#include "tensor_map.h"

#include <cuda_fp16.h>

#include <cstdlib>

namespace tcb {
cudaError_t init_mma_kernels(int smem_optin);
cudaError_t launch_gemv_q4_mma(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                               const char** name);
cudaError_t init_tc_kernels(int smem_optin);
cudaError_t launch_gemv_q4_tc(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                              const char** name);
namespace {

constexpr int kWarps = 8;               // generic kernel
constexpr int kThreads = kWarps * 32;
constexpr int kMaxStreamWarps = 16;     // streaming kernel: 8 or 16 warps, chosen per launch
constexpr int kMaxStreamThreads = kMaxStreamWarps * 32;
constexpr int kGroupBlocks = 8;
constexpr int kMaxMB = 4;
#ifndef TCB_ACT_I16
#define TCB_ACT_I16 1
#endif
#ifndef TCB_MEGA_TRACE
#define TCB_MEGA_TRACE 0
#endif
constexpr int kMaxPhaseOps = 4;             // persistent kernel: operations merged into one phase
constexpr bool kActI16 = TCB_ACT_I16 != 0;   // integer activation path (see stage_activations_i16)
constexpr int kTcMinBatch = 5;            // smallest M the tcgen05 kernel takes by default (measured: faster from M = 5 on every decode shape)

template <int FMT> struct Fmt;
template <> struct Fmt<FMT_Q4_0> {
    static constexpr int kBlockBytes = 18;
    static constexpr int kGroupBytes = 144;
    static constexpr int kGroupV4 = 9;
    static constexpr float kZeroPoint = 8.0f;
};
template <> struct Fmt<FMT_Q8_0> {
    static constexpr int kBlockBytes = 34;
    static constexpr int kGroupBytes = 272;
    static constexpr int kGroupV4 = 17;
    static constexpr float kZeroPoint = 128.0f;
};

struct StreamParams {
    const uint8_t* W;
    const void* X;
    void* Y;
    const void* gamma;
    uint32_t* err;
    int M, N, K;
    int nb;        // blocks per row
    int gpr;       // groups per row
    int ns;        // ring stages per warp
    int y_f32;
    int x_src_f16; // activations (and gamma) are fp16 in global memory
    float eps;
    // shared-memory offsets (bytes)
    int off_rowacc, off_sx, off_x, off_ring;
    int max_rows;  // rows per CTA upper bound
    int dbg_skip;  // measurement aid: stream the weights but skip the arithmetic
    long long* trace = nullptr;  // debug builds: stamps of the staging phases (CTA 0, thread 0)
};

// ---------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2e9 clocks (about a second) and reports false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 2000000000LL) return false;
    }
    return true;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// fp16 x fp16 + fp32 -> fp32, exact product, one rounding (PTX ISA 8.6, sm_100).
__device__ __forceinline__ float fma_h(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint16_t lo16(uint32_t v) { return static_cast<uint16_t>(v); }
__device__ __forceinline__ uint16_t hi16(uint32_t v) { return static_cast<uint16_t>(v >> 16); }
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// fp32 activations in shared memory: low half = fp16 head, high half = fp16 remainder
// (x = head + remainder to 2^-22 relative); both multiply the code with the mixed-precision FMA.
__device__ __forceinline__ uint32_t split_f32(float x) {
    const __half h = __float2half_rn(x);
    const __half l = __float2half_rn(x - __half2float(h));
    return static_cast<uint32_t>(__half_as_ushort(h)) |
           (static_cast<uint32_t>(__half_as_ushort(l)) << 16);
}
__device__ __forceinline__ float joined_f32(uint32_t w) { return h2f(lo16(w)) + h2f(hi16(w)); }
__device__ __forceinline__ float fma_hl(uint16_t code, uint32_t xw, float acc) {
    return fma_h(code, hi16(xw), fma_h(code, lo16(xw), acc));
}

__device__ __forceinline__ uint32_t get4(const uint4& v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// ---------------------------------------------------------------------------------------
// Activation staging.  Element k of row m sits at
//   fp16: ((c*gpr + kg)*16 + (k&7)*2)   with kg = k>>8, c = (k&255)>>3   (32 chunks / group)
//   fp32: ((c*gpr + kg)*16 + (k&3)*4)   with kg = k>>8, c = (k&255)>>2   (64 chunks / group)
// so lanes holding consecutive groups kg read consecutive 16-byte chunks.
// ---------------------------------------------------------------------------------------
template <bool XF32>
__device__ __forceinline__ int x_chunk_index(int k_chunk, int gpr) {
    // k_chunk = index of a 16-byte chunk in natural order (8 halves or 4 floats)
    constexpr int per_group = XF32 ? 64 : 32;
    const int kg = k_chunk / per_group;
    const int c = k_chunk % per_group;
    return c * gpr + kg;
}

// Sum over a thread block of one double per thread (result broadcast to all threads).
__device__ double block_sum_f64(double v, double* scratch /* one double per warp */) {
    const int nwarps = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) scratch[w] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nwarps; ++i) t += scratch[i];
    return t;
}

// Sum over a thread block of one float per thread (result broadcast to all threads): shuffles,
// one shared-memory slot per warp, and the per-warp partials added in a fixed order.
__device__ float block_sum_f32(float v, float* scratch /* one float per warp */) {
    const int nwarps = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) scratch[w] = v;
    __syncthreads();
    // every warp adds the partials in the same tree order: same bits in every thread
    float t = l < nwarps ? scratch[l] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// Loads MB activation rows into shared memory and fills
// sx[m][j*gpr+kg] = zero_point * (sum of the 32 staged activations of block kg*8+j).
// Without gamma the rows are copied as they are (staging type == source type).  With gamma the
// RMSNorm prologue runs first: sum of squares in double, rstd = 1/sqrtf(float(ss/K)+eps),
// row = (x*rstd)*gamma, kept in fp32 (XF32 staging) whether the source is fp16 or fp32.
// COHERENT: the activations may have been written by other CTAs of the same (persistent)
// kernel, so they are read with L2-coherent loads instead of the read-only path.
template <bool COHERENT, typename T>
__device__ __forceinline__ T ld_act(const T* ptr) {
    return COHERENT ? __ldcg(ptr) : __ldg(ptr);
}

template <bool XF32, int MB, bool COHERENT = false>
__device__ void stage_activations(const StreamParams& p, uint8_t* smem, float zero_point,
                                  double* red_scratch) {
    const int K = p.K, gpr = p.gpr, nb = p.nb;
    uint8_t* xs = smem + p.off_x;
    float* sx = reinterpret_cast<float*>(smem + p.off_sx);
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const size_t row_bytes = static_cast<size_t>(K) * (XF32 ? 4 : 2);

    for (int m = 0; m < MB; ++m) {
        uint4* dst = reinterpret_cast<uint4*>(xs + m * row_bytes);
        if (p.gamma == nullptr) {
            const int nchunks = K / (XF32 ? 4 : 8);
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const uint8_t*>(p.X) + m * row_bytes);
            for (int i = tid; i < nchunks; i += nthreads) {
                uint4 v = ld_act<COHERENT>(src + i);
                if (XF32)   // fp32 activations are staged as fp16 head + fp16 remainder
                    v = make_uint4(split_f32(__uint_as_float(v.x)), split_f32(__uint_as_float(v.y)),
                                   split_f32(__uint_as_float(v.z)), split_f32(__uint_as_float(v.w)));
                dst[x_chunk_index<XF32>(i, gpr)] = v;
            }
        } else if (XF32) {
            const int nquads = K / 4;
            double ss = 0.0;
            if (p.x_src_f16) {
                const uint2* xr = reinterpret_cast<const uint2*>(
                    static_cast<const __half*>(p.X) + static_cast<size_t>(m) * K);
                for (int i = tid; i < nquads; i += nthreads) {
                    const uint2 v = ld_act<COHERENT>(xr + i);
                    const double a = h2f(lo16(v.x)), b = h2f(hi16(v.x));
                    const double c = h2f(lo16(v.y)), d = h2f(hi16(v.y));
                    ss += a * a + b * b + c * c + d * d;
                }
            } else {
                const float4* xr = reinterpret_cast<const float4*>(
                    static_cast<const float*>(p.X) + static_cast<size_t>(m) * K);
                for (int i = tid; i < nquads; i += nthreads) {
                    const float4 v = ld_act<COHERENT>(xr + i);
                    const double a = v.x, b = v.y, c = v.z, d = v.w;
                    ss += a * a + b * b + c * c + d * d;
                }
            }
            ss = block_sum_f64(ss, red_scratch);
            const float rstd =
                1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(K)) + p.eps);
            for (int i = tid; i < nquads; i += nthreads) {
                float4 xv, gv;
                if (p.x_src_f16) {
                    const uint2 xb = ld_act<COHERENT>(reinterpret_cast<const uint2*>(
                        static_cast<const __half*>(p.X) + static_cast<size_t>(m) * K) + i);
                    const uint2 gb = __ldg(reinterpret_cast<const uint2*>(p.gamma) + i);
                    xv = make_float4(h2f(lo16(xb.x)), h2f(hi16(xb.x)), h2f(lo16(xb.y)), h2f(hi16(xb.y)));
                    gv = make_float4(h2f(lo16(gb.x)), h2f(hi16(gb.x)), h2f(lo16(gb.y)), h2f(hi16(gb.y)));
                } else {
                    xv = ld_act<COHERENT>(reinterpret_cast<const float4*>(
                        static_cast<const float*>(p.X) + static_cast<size_t>(m) * K) + i);
                    gv = __ldg(reinterpret_cast<const float4*>(p.gamma) + i);
                }
                float4 o;
                o.x = __fmul_rn(__fmul_rn(xv.x, rstd), gv.x);
                o.y = __fmul_rn(__fmul_rn(xv.y, rstd), gv.y);
                o.z = __fmul_rn(__fmul_rn(xv.z, rstd), gv.z);
                o.w = __fmul_rn(__fmul_rn(xv.w, rstd), gv.w);
                dst[x_chunk_index<true>(i, gpr)] =
                    make_uint4(split_f32(o.x), split_f32(o.y), split_f32(o.z), split_f32(o.w));
            }
        }
    }
    __syncthreads();
    for (int t = tid; t < MB * nb; t += nthreads) {
        const int m = t / nb, b = t % nb;
        const int kg = b >> 3, j = b & 7;
        const uint4* xrow = reinterpret_cast<const uint4*>(xs + m * row_bytes);
        float s = 0.f;
        if (XF32) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint4 v = xrow[(8 * j + q) * gpr + kg];
                s += joined_f32(v.x);
                s += joined_f32(v.y);
                s += joined_f32(v.z);
                s += joined_f32(v.w);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = xrow[(4 * j + q) * gpr + kg];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t w = get4(v, e);
                    s += h2f(lo16(w));
                    s += h2f(hi16(w));
                }
            }
        }
        sx[m * nb + j * gpr + kg] = zero_point * s;
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------
// One group (8 blocks, 256 weights) against MB activation rows.
// w[] holds the group's bytes as 32-bit words; all indexing below is compile-time.
// ---------------------------------------------------------------------------------------
template <int FMT, bool XF32, int MB>
__device__ __forceinline__ void group_dot(const uint32_t (&w)[Fmt<FMT>::kGroupV4 * 4],
                                          const uint8_t* xs, const float* sx, int kg, int gpr,
                                          int K, int nb, float (&out)[MB]) {
    const size_t row_bytes = static_cast<size_t>(K) * (XF32 ? 4 : 2);
#pragma unroll
    for (int j = 0; j < kGroupBlocks; ++j) {
        constexpr int kHwPerBlock = Fmt<FMT>::kBlockBytes / 2;  // 9 or 17 halfwords
        const int hw = kHwPerBlock * j;                          // halfword index of the scale
        const uint32_t sw = w[hw >> 1];
        const float d = h2f((hw & 1) ? hi16(sw) : lo16(sw));
        const int qhw = hw + 1;                                  // first halfword of the codes
        constexpr int kQWords = (Fmt<FMT>::kBlockBytes - 2) / 4; // 4 or 8 code words
        uint32_t q[kQWords];
#pragma unroll
        for (int t = 0; t < kQWords; ++t) {
            if (qhw & 1) q[t] = __funnelshift_r(w[(qhw >> 1) + t], w[(qhw >> 1) + t + 1], 16);
            else q[t] = w[(qhw >> 1) + t];
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const uint4* xrow = reinterpret_cast<const uint4*>(xs + m * row_bytes);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (FMT == FMT_Q4_0) {
                // byte i of the block: low nibble <-> x[i], high nibble <-> x[i+16].
                // Word t covers bytes 4t..4t+3.  (q & 0x000f000f) = codes of bytes 4t, 4t+2 as
                // two fp16 subnormals (c * 2^-24); ((q>>8) & ...) = bytes 4t+1, 4t+3.  The high
                // nibbles masked in place carry an extra factor 16 (c * 2^-20).
                if (!XF32) {
                    uint4 xv[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) xv[c] = xrow[(4 * j + c) * gpr + kg];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint32_t l01 = get4(xv[t >> 1], (t & 1) * 2);
                        const uint32_t l23 = get4(xv[t >> 1], (t & 1) * 2 + 1);
                        const uint32_t h01 = get4(xv[2 + (t >> 1)], (t & 1) * 2);
                        const uint32_t h23 = get4(xv[2 + (t >> 1)], (t & 1) * 2 + 1);
                        const uint32_t v0 = q[t] & 0x000f000fu;
                        const uint32_t v1 = q[t] & 0x00f000f0u;
                        const uint32_t s8 = q[t] >> 8;
                        const uint32_t v2 = s8 & 0x000f000fu;
                        const uint32_t v3 = s8 & 0x00f000f0u;
                        a0 = fma_h(lo16(v0), lo16(l01), a0);
                        a1 = fma_h(lo16(v2), hi16(l01), a1);
                        a0 = fma_h(hi16(v0), lo16(l23), a0);
                        a1 = fma_h(hi16(v2), hi16(l23), a1);
                        a2 = fma_h(lo16(v1), lo16(h01), a2);
                        a3 = fma_h(lo16(v3), hi16(h01), a3);
                        a2 = fma_h(hi16(v1), lo16(h23), a2);
                        a3 = fma_h(hi16(v3), hi16(h23), a3);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint4 xl = xrow[(8 * j + t) * gpr + kg];       // x[4t..4t+3]
                        const uint4 xh = xrow[(8 * j + 4 + t) * gpr + kg];   // x[16+4t..]
                        const uint32_t v0 = q[t] & 0x000f000fu;
                        const uint32_t v1 = q[t] & 0x00f000f0u;
                        const uint32_t s8 = q[t] >> 8;
                        const uint32_t v2 = s8 & 0x000f000fu;
                        const uint32_t v3 = s8 & 0x00f000f0u;
                        a0 = fma_hl(lo16(v0), xl.x, a0);
                        a1 = fma_hl(lo16(v2), xl.y, a1);
                        a0 = fma_hl(hi16(v0), xl.z, a0);
                        a1 = fma_hl(hi16(v2), xl.w, a1);
                        a2 = fma_hl(lo16(v1), xh.x, a2);
                        a3 = fma_hl(lo16(v3), xh.y, a3);
                        a2 = fma_hl(hi16(v1), xh.z, a2);
                        a3 = fma_hl(hi16(v3), xh.w, a3);
                    }
                }
                const float s = sx[m * nb + j * gpr + kg];
                // undo 2^-24 / 2^-20, remove the zero point, apply the block scale
                const float blk = fmaf(a0 + a1, 16777216.0f, fmaf(a2 + a3, 1048576.0f, -s));
                out[m] = fmaf(d, blk, out[m]);
            } else {
                // Q8_0: flip the sign bit of every code byte (c + 128, unsigned), widen byte
                // pairs to fp16 subnormals with a byte permute.
                if (!XF32) {
                    uint4 xv[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) xv[c] = xrow[(4 * j + c) * gpr + kg];
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const uint32_t u = q[t] ^ 0x80808080u;
                        const uint32_t p01 = __byte_perm(u, 0u, 0x4140);
                        const uint32_t p23 = __byte_perm(u, 0u, 0x4342);
                        const uint32_t x01 = get4(xv[t >> 1], (t & 1) * 2);
                        const uint32_t x23 = get4(xv[t >> 1], (t & 1) * 2 + 1);
                        a0 = fma_h(lo16(p01), lo16(x01), a0);
                        a1 = fma_h(hi16(p01), hi16(x01), a1);
                        a2 = fma_h(lo16(p23), lo16(x23), a2);
                        a3 = fma_h(hi16(p23), hi16(x23), a3);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const uint4 xq = xrow[(8 * j + t) * gpr + kg];
                        const uint32_t u = q[t] ^ 0x80808080u;
                        const uint32_t p01 = __byte_perm(u, 0u, 0x4140);
                        const uint32_t p23 = __byte_perm(u, 0u, 0x4342);
                        a0 = fma_hl(lo16(p01), xq.x, a0);
                        a1 = fma_hl(hi16(p01), xq.y, a1);
                        a2 = fma_hl(lo16(p23), xq.z, a2);
                        a3 = fma_hl(hi16(p23), xq.w, a3);
                    }
                }
                const float s = sx[m * nb + j * gpr + kg];
                const float blk = fmaf((a0 + a1) + (a2 + a3), 16777216.0f, -s);
                out[m] = fmaf(d, blk, out[m]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Integer activation path.
//
// Activations are staged once per CTA as int16 with one fp32 scale per 32-element block
// (scale = max|x| / 32767 over the block, so every element is within 2^-16 of its block's
// maximum, insensitive to outliers elsewhere in the row; fp16 inputs use a power-of-two scale
// and are exact down to 1/16 of the block maximum).  Measured against an fp64 dequantise-and-dot
// on Gaussian rows: 2.2e-5 scaled RMS for fp32 rows (5e-5 for heavy-tailed ones), 7e-6 for fp16.  The dot product of a block is then exact integer arithmetic
// on the dp2a unit (two 16-bit x two 8-bit products per lane per instruction):
//     y += d_w * s_x * (sum_k q_k * xq_k  -  zp * sum_k xq_k)
// which needs about one issued instruction per weight where the fp16-FMA formulation needs
// three.  Layout of the staged row: the fp16 chunk layout above (16-byte chunks of 8 values,
// chunk c of group kg at (c*gpr + kg)*16).  sx2[m*nb + j*gpr + kg] = {scale, zp * sum(xq)}.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int dp2a_lo_su(uint32_t x_s16x2, uint32_t q_u8x4, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x_s16x2), "r"(q_u8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t x_s16x2, uint32_t q_u8x4, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x_s16x2), "r"(q_u8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_lo_ss(uint32_t x_s16x2, uint32_t q_s8x4, int c) {
    int d;
    asm("dp2a.lo.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x_s16x2), "r"(q_s8x4), "r"(c));
    return d;
}
__device__ __forceinline__ int dp2a_hi_ss(uint32_t x_s16x2, uint32_t q_s8x4, int c) {
    int d;
    asm("dp2a.hi.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x_s16x2), "r"(q_s8x4), "r"(c));
    return d;
}

// Eight consecutive activations (and, fused, their gammas) of row m starting at k = 8*i.
template <bool COHERENT>
__device__ __forceinline__ void load8(const void* base, bool f16, size_t elem0, float (&v)[8]) {
    if (f16) {
        const uint4 t = ld_act<COHERENT>(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + elem0));
        v[0] = h2f(lo16(t.x)); v[1] = h2f(hi16(t.x)); v[2] = h2f(lo16(t.y)); v[3] = h2f(hi16(t.y));
        v[4] = h2f(lo16(t.z)); v[5] = h2f(hi16(t.z)); v[6] = h2f(lo16(t.w)); v[7] = h2f(hi16(t.w));
    } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem0);
        const float4 a = ld_act<COHERENT>(src), b = ld_act<COHERENT>(src + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// Stages MB rows as int16 + per-block scales.  With gamma the RMSNorm prologue runs first: sum of
// squares in double, rstd = 1/sqrtf(float(ss/K)+eps), row = (x*rstd)*gamma in fp32 - the
// reference's order - and that row is what gets quantised.  `zp` is the weight zero point (8 for
// Q4_0 codes taken as unsigned nibbles, 0 for Q8_0's signed bytes).
// Quantises one 8-value chunk (index i of row m) held in v[] and stores it; the four lanes of a
// quad hold the four chunks of a 32-element block and share its scale.  Every lane of the warp
// calls this (dead lanes with live = false and zeros) so the quad shuffles are among live lanes.
template <bool NATURAL>
__device__ __forceinline__ void quantise_chunk(const float (&v)[8], bool live, int i, int m, int zp,
                                               bool pow2, int gpr, int nb, uint4* dst, float2* sx2) {
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // fp16 sources get a power-of-two scale (block maximum mapped into [16384, 32768)): every
    // element within a factor 16 of the maximum is then represented exactly.
    float scale = amax * (1.0f / 32767.0f), inv = amax > 0.f ? 32767.0f / amax : 0.f;
    if (pow2 && amax > 0.f) {
        const uint32_t e = __float_as_uint(amax) & 0x7f800000u;
        scale = __uint_as_float(e - (14u << 23));
        inv = __uint_as_float((254u << 23) - (e - (14u << 23)));
    }
    int q[8], isum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        // round to nearest even without the conversion unit: adding 1.5 * 2^23 leaves the
        // integer in the low mantissa bits (|v * inv| <= 32767.5 by construction)
        q[e] = __float_as_int(__fadd_rn(v[e] * inv, 12582912.0f)) - 0x4B400000;
        q[e] = max(-32767, min(32767, q[e]));
        isum += q[e];
    }
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    if (live) {
        uint4 o;
        o.x = (static_cast<uint32_t>(q[0]) & 0xffffu) | (static_cast<uint32_t>(q[1]) << 16);
        o.y = (static_cast<uint32_t>(q[2]) & 0xffffu) | (static_cast<uint32_t>(q[3]) << 16);
        o.z = (static_cast<uint32_t>(q[4]) & 0xffffu) | (static_cast<uint32_t>(q[5]) << 16);
        o.w = (static_cast<uint32_t>(q[6]) & 0xffffu) | (static_cast<uint32_t>(q[7]) << 16);
        dst[NATURAL ? i : x_chunk_index<false>(i, gpr)] = o;
        if ((i & 3) == 0) {
            const int b = i >> 2, kg = b >> 3, j = b & 7;
            sx2[m * nb + (NATURAL ? b : j * gpr + kg)] = make_float2(scale, __int_as_float(zp * isum));
        }
    }
}

// Stages MB rows as int16 + per-block scales.  With gamma the RMSNorm prologue runs first: sum of
// squares in double, rstd = 1/sqrtf(float(ss/K)+eps), row = (x*rstd)*gamma in fp32 - the
// reference's order - and that row is what gets quantised.  `zp` is the weight zero point (8 for
// Q4_0 codes taken as unsigned nibbles, 0 for Q8_0's signed bytes).
// NATURAL: the staged row and the scales keep the order of k (every lane of a warp then reads the
// same activations: one broadcast per load); otherwise the chunk-transposed layout above.
// Rows of up to 4 chunks per thread (K <= 32 * blockDim) are loaded once, activations and gamma
// in the same round trip, and held in registers across the reduction; longer rows are read twice.
template <int MB, bool COHERENT = false, bool NATURAL = false>
__device__ void stage_activations_i16(const StreamParams& p, uint8_t* smem, int zp, double* red_scratch) {
    const int K = p.K, gpr = p.gpr, nb = p.nb;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int nchunks = K >> 3;
    const bool f16 = p.x_src_f16 != 0;
    const bool fused = p.gamma != nullptr;
    const bool pow2 = f16 && !fused;
    float2* sx2 = reinterpret_cast<float2*>(smem + p.off_sx);
    constexpr int kHold = 4;
    for (int m = 0; m < MB; ++m) {
        uint4* dst = reinterpret_cast<uint4*>(smem + p.off_x + static_cast<size_t>(m) * K * 2);
        const size_t row0 = static_cast<size_t>(m) * K;
        if (nchunks <= kHold * nthreads) {
            float v[kHold][8], g[kHold][8];
#pragma unroll
            for (int r = 0; r < kHold; ++r) {
                const int i = tid + r * nthreads;
#pragma unroll
                for (int e = 0; e < 8; ++e) { v[r][e] = 0.f; g[r][e] = 1.f; }
                if (i < nchunks) {
                    load8<COHERENT>(p.X, f16, row0 + 8 * static_cast<size_t>(i), v[r]);
                    if (fused) load8<false>(p.gamma, f16, 8 * static_cast<size_t>(i), g[r]);
                }
            }
#if TCB_MEGA_TRACE
#define STR(C) do { if (p.trace && blockIdx.x == 0 && tid == 0) p.trace[C] = clock64(); } while (0)
#else
#define STR(C) do { } while (0)
#endif
            STR(0);
            {
                float dep = 0.f;
#pragma unroll
                for (int r = 0; r < kHold; ++r) dep += v[r][0] + g[r][7];
                if (dep == 1.2345e-30f) sx2[0].x = dep;   // forces the loads to have landed
            }
            STR(1);
            float rstd = 1.0f;
            if (fused) {
                // Sum of squares in fp32, pairwise within the thread and across the block: the
                // relative error (about 1e-7) is far below what the int16 staging resolves, and
                // fp64 arithmetic is slow on this part (the fp64 version of this reduction took
                // 2200 cycles per call).
                float part[kHold];
#pragma unroll
                for (int r = 0; r < kHold; ++r) {
                    const float s01 = fmaf(v[r][0], v[r][0], v[r][1] * v[r][1]);
                    const float s23 = fmaf(v[r][2], v[r][2], v[r][3] * v[r][3]);
                    const float s45 = fmaf(v[r][4], v[r][4], v[r][5] * v[r][5]);
                    const float s67 = fmaf(v[r][6], v[r][6], v[r][7] * v[r][7]);
                    part[r] = (s01 + s23) + (s45 + s67);
                }
                float ss = 0.f;
#pragma unroll
                for (int r = 0; r < kHold; r += 2) ss += part[r] + (r + 1 < kHold ? part[r + 1] : 0.f);
                ss = block_sum_f32(ss, reinterpret_cast<float*>(red_scratch));
                rstd = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
            }
            STR(2);
#pragma unroll
            for (int r = 0; r < kHold; ++r) {
                const int i = tid + r * nthreads;
                if (r * nthreads >= nchunks) break;   // uniform: no lane has a chunk in this round
                if (fused) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[r][e] = __fmul_rn(__fmul_rn(v[r][e], rstd), g[r][e]);
                }
                quantise_chunk<NATURAL>(v[r], i < nchunks, i, m, zp, pow2, gpr, nb, dst, sx2);
            }
            STR(3);
        } else {
            float rstd = 1.0f;
            if (fused) {
                double ss = 0.0;
                for (int i = tid; i < nchunks; i += nthreads) {
                    float v[8];
                    load8<COHERENT>(p.X, f16, row0 + 8 * static_cast<size_t>(i), v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss += static_cast<double>(v[e]) * static_cast<double>(v[e]);
                }
                ss = block_sum_f64(ss, red_scratch);
                rstd = 1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(K)) + p.eps);
            }
            for (int base = 0; base < nchunks; base += nthreads) {
                const int i = base + tid;
                const bool live = i < nchunks;
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
                if (live) {
                    load8<COHERENT>(p.X, f16, row0 + 8 * static_cast<size_t>(i), v);
                    if (fused) {
                        float g[8];
                        load8<false>(p.gamma, f16, 8 * static_cast<size_t>(i), g);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(__fmul_rn(v[e], rstd), g[e]);
                    }
                }
                quantise_chunk<NATURAL>(v, live, i, m, zp, pow2, gpr, nb, dst, sx2);
            }
        }
    }
    __syncthreads();
}

// One group (8 blocks, 256 weights) against MB staged rows, integer dot products.
template <int FMT, int MB, bool NATURAL = false>
__device__ __forceinline__ void group_dot_i16(const uint32_t (&w)[Fmt<FMT>::kGroupV4 * 4],
                                              const uint8_t* xs, const float2* sx2, int kg, int gpr,
                                              int K, int nb, float (&out)[MB]) {
#pragma unroll
    for (int j = 0; j < kGroupBlocks; ++j) {
        constexpr int kHwPerBlock = Fmt<FMT>::kBlockBytes / 2;  // 9 or 17 halfwords
        const int hw = kHwPerBlock * j;                          // halfword index of the scale
        const uint32_t sw = w[hw >> 1];
        const float d = h2f((hw & 1) ? hi16(sw) : lo16(sw));
        const int qhw = hw + 1;                                  // first halfword of the codes
        constexpr int kQWords = (Fmt<FMT>::kBlockBytes - 2) / 4; // 4 or 8 code words
        uint32_t q[kQWords];
#pragma unroll
        for (int t = 0; t < kQWords; ++t) {
            if (qhw & 1) q[t] = __funnelshift_r(w[(qhw >> 1) + t], w[(qhw >> 1) + t + 1], 16);
            else q[t] = w[(qhw >> 1) + t];
        }
        uint32_t lo4[4], hi4[4];
        if (FMT == FMT_Q4_0) {
            // byte i of the block: low nibble <-> x[i], high nibble <-> x[i+16]
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                lo4[t] = q[t] & 0x0f0f0f0fu;
                hi4[t] = q[t] & 0xf0f0f0f0u;   // 16 x the high nibbles: shifted out of the sum below
            }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const uint4* xrow = reinterpret_cast<const uint4*>(xs + static_cast<size_t>(m) * K * 2);
            uint4 xv[4];   // x[8c .. 8c+7] of this block as int16 pairs
#pragma unroll
            for (int c = 0; c < 4; ++c) xv[c] = NATURAL ? xrow[(kg * 8 + j) * 4 + c] : xrow[(4 * j + c) * gpr + kg];
            int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
            if (FMT == FMT_Q4_0) {
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const uint32_t l01 = get4(xv[t >> 1], (t & 1) * 2), l23 = get4(xv[t >> 1], (t & 1) * 2 + 1);
                    const uint32_t h01 = get4(xv[2 + (t >> 1)], (t & 1) * 2), h23 = get4(xv[2 + (t >> 1)], (t & 1) * 2 + 1);
                    a0 = dp2a_lo_su(l01, lo4[t], a0);
                    a1 = dp2a_lo_su(h01, hi4[t], a1);
                    a2 = dp2a_hi_su(l23, lo4[t], a2);
                    a3 = dp2a_hi_su(h23, hi4[t], a3);
                }
            } else {
                // Q8_0: byte i <-> x[i], signed
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const uint32_t x01 = get4(xv[t >> 1], (t & 1) * 2), x23 = get4(xv[t >> 1], (t & 1) * 2 + 1);
                    if (t & 1) { a2 = dp2a_lo_ss(x01, q[t], a2); a3 = dp2a_hi_ss(x23, q[t], a3); }
                    else { a0 = dp2a_lo_ss(x01, q[t], a0); a1 = dp2a_hi_ss(x23, q[t], a1); }
                }
            }
            const float2 sc = sx2[m * nb + (NATURAL ? kg * 8 + j : j * gpr + kg)];
            // Q4_0: a1 and a3 hold 16 x the high-nibble sums (exact multiples of 16, at most
            // 16 * 240 * 32767 in magnitude), a0 and a2 the low-nibble sums
            const int dot = FMT == FMT_Q4_0 ? (a0 + a2) + ((a1 + a3) >> 4) - __float_as_int(sc.y)
                                            : (a0 + a1) + (a2 + a3) - __float_as_int(sc.y);
            out[m] = fmaf(d * sc.x, static_cast<float>(dot), out[m]);
        }
    }
}

// ---------------------------------------------------------------------------------------
// The streaming kernel.
// ---------------------------------------------------------------------------------------
template <int FMT, bool XF32, int MB>
__global__ void __launch_bounds__(kMaxStreamThreads, 1) gemv_q_stream_kernel(const StreamParams p) {
    using F = Fmt<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                  // [nwarps*ns]
    double* red_scratch = reinterpret_cast<double*>(smem + 8 * kMaxStreamWarps * 4);  // after the barriers
    float* rowacc = reinterpret_cast<float*>(smem + p.off_rowacc);
    uint8_t* ring = smem + p.off_ring;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = blockDim.x >> 5, nthreads = blockDim.x;
    const int ns = p.ns, gpr = p.gpr;
    constexpr int kChunkBytes = 32 * F::kGroupBytes;

    // Row range of this CTA and the corresponding run of groups.
    const int r0 = static_cast<int>(static_cast<long long>(p.N) * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>(static_cast<long long>(p.N) * (blockIdx.x + 1) / gridDim.x);
    const int rows = r1 - r0;
    const long long g_base = static_cast<long long>(r0) * gpr;
    const int g_count = rows * gpr;
    const int nchunks = (g_count + 31) >> 5;
    const int my_n = nchunks > warp ? (nchunks - warp + nwarps - 1) / nwarps : 0;

    pdl_launch_dependents();

    if (tid == 0) {
        for (int i = 0; i < nwarps * ns; ++i) mbar_init(&bars[i], 1);
        fence_barrier_init();
    }
    for (int i = tid; i < rows * MB; i += nthreads) rowacc[i] = 0.f;
    __syncthreads();

    auto issue = [&](int i) {  // lane 0 only: start the copy of this warp's i-th chunk
        const int c = warp + nwarps * i;
        const int first = c << 5;
        const int ng = min(32, g_count - first);
        const uint32_t bytes = static_cast<uint32_t>(ng) * F::kGroupBytes;
        const int s = i % ns;
        uint64_t* bar = &bars[warp * ns + s];
        mbar_expect_tx(bar, bytes);
        bulk_g2s(ring + static_cast<size_t>(warp * ns + s) * kChunkBytes,
                 p.W + (g_base + first) * F::kGroupBytes, bytes, bar);
    };
    // Weights do not depend on the previous kernel in the stream: start streaming now.
    if (lane == 0) {
        const int pre = min(ns, my_n);
        for (int i = 0; i < pre; ++i) issue(i);
    }

    // Activations may be the previous kernel's output: wait for it, then stage them.
    pdl_wait();
    if (kActI16) stage_activations_i16<MB>(p, smem, FMT == FMT_Q4_0 ? 8 : 0, red_scratch);
    else stage_activations<XF32, MB>(p, smem, F::kZeroPoint, red_scratch);

    const uint8_t* xs = smem + p.off_x;
    const float* sx = reinterpret_cast<const float*>(smem + p.off_sx);
    bool failed = false;
    int waited = 0;  // number of this warp's chunks whose barrier has been consumed

    for (int i = 0; i < my_n; ++i) {
        const int s = i % ns;
        uint64_t* bar = &bars[warp * ns + s];
        if (!mbar_wait_bounded(bar, static_cast<uint32_t>((i / ns) & 1))) {
            failed = true;
            break;
        }
        waited = i + 1;
        const int c = warp + nwarps * i;
        const int gl = (c << 5) + lane;           // group index local to the CTA
        const bool valid = gl < g_count;

        uint32_t w[F::kGroupV4 * 4];
        if (valid) {
            const uint4* src = reinterpret_cast<const uint4*>(
                ring + static_cast<size_t>(warp * ns + s) * kChunkBytes +
                static_cast<size_t>(lane) * F::kGroupBytes);
#pragma unroll
            for (int v = 0; v < F::kGroupV4; ++v) {
                const uint4 t = src[v];
                w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int v = 0; v < F::kGroupV4 * 4; ++v) w[v] = 0u;
        }
        __syncwarp();
        if (lane == 0 && i + ns < my_n) {
            fence_proxy_async();
            issue(i + ns);
        }

        float out[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) out[m] = 0.f;
        int row = -1 - lane;  // distinct negatives for idle lanes
        if (valid) {
            row = gl / gpr;
            const int kg = gl - row * gpr;
            if (p.dbg_skip) out[0] = __uint_as_float(w[0] ^ w[35]);
            else
            if (kActI16) group_dot_i16<FMT, MB>(w, xs, reinterpret_cast<const float2*>(sx), kg, gpr, p.K, p.nb, out);
            else group_dot<FMT, XF32, MB>(w, xs, sx, kg, gpr, p.K, p.nb, out);
        }
        // Segmented reduction over lanes that hold groups of the same row (contiguous runs).
#pragma unroll
        for (int dlt = 1; dlt < 32; dlt <<= 1) {
            const int r2 = __shfl_down_sync(0xffffffffu, row, dlt);
            const bool take = (lane + dlt < 32) && (r2 == row);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float v2 = __shfl_down_sync(0xffffffffu, out[m], dlt);
                if (take) out[m] += v2;
            }
        }
        const int rprev = __shfl_up_sync(0xffffffffu, row, 1);
        if (valid && (lane == 0 || rprev != row)) {
#pragma unroll
            for (int m = 0; m < MB; ++m) atomicAdd(&rowacc[row * MB + m], out[m]);
        }
    }

    if (failed) {
        if (lane == 0) atomicOr(p.err, ERR_WAIT_TIMEOUT);
        // Drain copies this warp still has in flight (bounded), so that none lands after exit.
        const int issued = min(my_n, waited + ns);
        for (int i = waited; i < issued; ++i)
            (void)mbar_wait_bounded(&bars[warp * ns + (i % ns)], static_cast<uint32_t>((i / ns) & 1));
    }
    __syncthreads();

    for (int i = tid; i < rows * MB; i += nthreads) {
        const int r = i / MB, m = i - r * MB;
        const size_t o = static_cast<size_t>(m) * p.N + (r0 + r);
        const float v = rowacc[i];
        if (p.y_f32) static_cast<float*>(p.Y)[o] = v;
        else static_cast<__half*>(p.Y)[o] = __float2half_rn(v);
    }
}

// ---------------------------------------------------------------------------------------
// The box kernel: one operation, a row per lane.
//
// Same arithmetic as the streaming kernel, different geometry: the unit of work is a box of 32
// weight rows x one group (144 / 272 bytes per row) fetched by one tiled TMA copy; a lane owns a
// row, so every lane of a warp reads the same staged activations (one shared-memory broadcast per
// load instead of 32 different 16-byte chunks - with a lane per K group the activation reads are
// 2 bytes per weight and saturate shared-memory bandwidth) and no shuffle reduction is needed:
// a lane adds its partial dot product to its row's accumulator.  Up to MB activation rows.
// ---------------------------------------------------------------------------------------
template <int FMT, int MB>
__global__ void __launch_bounds__(kMaxStreamThreads, 1)
gemv_q_box_kernel(const StreamParams p, const __grid_constant__ CUtensorMap wmap) {
    using F = Fmt<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                               // [nwarps*ns]
    double* red_scratch = reinterpret_cast<double*>(smem + 8 * kMaxStreamWarps * 4);  // after the barriers
    float* rowacc = reinterpret_cast<float*>(smem + p.off_rowacc);
    uint8_t* ring = smem + p.off_ring;
    constexpr int kBoxBytes = 32 * F::kGroupBytes;
    constexpr int kElem = FMT == FMT_Q4_0 ? 1 : 4;     // tensor-map element size (see the launcher)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = blockDim.x >> 5, nthreads = blockDim.x;
    const int ns = p.ns, gpr = p.gpr;
    const int r0 = static_cast<int>(static_cast<long long>(p.N) * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>(static_cast<long long>(p.N) * (blockIdx.x + 1) / gridDim.x);
    const int rows = r1 - r0;
    const int rows_pad = (rows + 31) & ~31;
    const int n_units = (rows_pad >> 5) * gpr;
    const int my_n = n_units > warp ? (n_units - warp + nwarps - 1) / nwarps : 0;

    pdl_launch_dependents();
    if (tid == 0) {
        sm100::prefetch_tensormap(&wmap);
        for (int i = 0; i < nwarps * ns; ++i) mbar_init(&bars[i], 1);
        fence_barrier_init();
    }
    for (int i = tid; i < rows_pad * MB; i += nthreads) rowacc[i] = 0.f;
    __syncthreads();

    auto issue = [&](int i) {  // lane 0 only: start the copy of this warp's i-th box
        const int u = warp + nwarps * i;
        const int rb = u / gpr, kg = u - rb * gpr;
        const int s = i % ns;
        uint64_t* bar = &bars[warp * ns + s];
        mbar_expect_tx(bar, kBoxBytes);
        sm100::tensor_load_2d(ring + static_cast<size_t>(warp * ns + s) * kBoxBytes, &wmap,
                              kg * (F::kGroupBytes / kElem), r0 + rb * 32, bar);
    };
    // Weights do not depend on the previous kernel in the stream: start streaming now.
    if (lane == 0) {
        const int pre = min(ns, my_n);
        for (int i = 0; i < pre; ++i) issue(i);
    }
    // Activations may be the previous kernel's output: wait for it, then stage them.
    pdl_wait();
    stage_activations_i16<MB, false, true>(p, smem, FMT == FMT_Q4_0 ? 8 : 0, red_scratch);

    const uint8_t* xs = smem + p.off_x;
    const float2* sx2 = reinterpret_cast<const float2*>(smem + p.off_sx);
    bool failed = false;
    int waited = 0;
    for (int i = 0; i < my_n; ++i) {
        const int s = i % ns;
        uint64_t* bar = &bars[warp * ns + s];
        if (!mbar_wait_bounded(bar, static_cast<uint32_t>((i / ns) & 1))) { failed = true; break; }
        waited = i + 1;
        const int u = warp + nwarps * i;
        const int rb = u / gpr, kg = u - rb * gpr;
        const int rl = rb * 32 + lane;
        uint32_t w[F::kGroupV4 * 4];
        {
            const uint4* src = reinterpret_cast<const uint4*>(
                ring + static_cast<size_t>(warp * ns + s) * kBoxBytes + static_cast<size_t>(lane) * F::kGroupBytes);
#pragma unroll
            for (int v = 0; v < F::kGroupV4; ++v) {
                const uint4 t = src[v];
                w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
            }
        }
        __syncwarp();
        if (lane == 0 && i + ns < my_n) {
            fence_proxy_async();
            issue(i + ns);
        }
        float out[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) out[m] = 0.f;
        if (p.dbg_skip) out[0] = __uint_as_float(w[0] ^ w[F::kGroupV4 * 4 - 1]);
        else group_dot_i16<FMT, MB, true>(w, xs, sx2, kg, gpr, p.K, p.nb, out);
        if (rl < rows) {
#pragma unroll
            for (int m = 0; m < MB; ++m) atomicAdd(&rowacc[m * rows_pad + rl], out[m]);
        }
    }
    if (failed) {
        if (lane == 0 && p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
        // let copies that are still in flight land before the CTA's shared memory is released
        const int issued = min(my_n, waited + ns);
        for (int i = waited; i < issued; ++i)
            (void)mbar_wait_bounded(&bars[warp * ns + (i % ns)], static_cast<uint32_t>((i / ns) & 1));
    }
    __syncthreads();
    if (failed) return;
    for (int i = tid; i < rows * MB; i += nthreads) {
        const int m = i / rows, r = i - m * rows;
        const float v = rowacc[m * rows_pad + r];
        const size_t o = static_cast<size_t>(m) * p.N + r0 + r;
        if (p.y_f32) static_cast<float*>(p.Y)[o] = v;
        else static_cast<__half*>(p.Y)[o] = __float2half_rn(v);
    }
}

// ---------------------------------------------------------------------------------------
// Persistent decode kernel: a whole recorded list of Q4_0, M = 1 GEMVs in ONE launch.
//
// One CTA per SM (cooperative launch: all CTAs are co-resident).  The unit of work is a box of 32
// weight rows x one 8-block group (144 bytes per row), fetched by one tiled TMA copy through a
// per-operation tensor map.  A lane owns a ROW of the box, so all lanes of a warp read the same
// activations from shared memory (one broadcast per load instead of 32 different 16-byte chunks:
// the activation reads were what saturated shared-memory bandwidth with a lane per K group), and
// a lane adds its partial dot product to its row's accumulator.  Every warp keeps its ring of
// boxes full ACROSS operations: when it has issued the last chunk of operation i it
// goes on with the first chunks of operation i+1, so HBM keeps streaming while the CTA finishes
// i, writes its rows and waits for the other CTAs.  Operations that read what an earlier one
// wrote are separated by a grid-wide barrier (one 64-bit counter in global memory, release /
// acquire, bounded spin); operations that share their input (q/k/v, gate/up) are not, and reuse
// the staged activations.  Activations written earlier in the same launch are read with
// L2-coherent loads.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

struct WarpGeom {            // one operation as seen by one warp of one CTA
    int r0, rows, gpr;       // the CTA's row range, groups per row
    int n_units;             // (32-row block, group) pairs of the CTA
    int my_n;                // how many of them this warp takes: units warp, warp + nwarps, ...
};

__device__ __forceinline__ WarpGeom make_geom(const MegaOp& op, int warp, int nwarps) {
    WarpGeom g;
    // 32-bit arithmetic: the launcher refuses N * gridDim >= 2^32
    g.r0 = static_cast<int>(static_cast<uint32_t>(op.N) * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>(static_cast<uint32_t>(op.N) * (blockIdx.x + 1) / gridDim.x);
    g.rows = r1 - g.r0;
    g.gpr = op.K >> 8;
    g.n_units = ((g.rows + 31) >> 5) * g.gpr;
    g.my_n = g.n_units > warp ? (g.n_units - warp + nwarps - 1) / nwarps : 0;
    return g;
}

__global__ void __launch_bounds__(kMaxStreamThreads, 1) gemv_q4_decode_kernel(const MegaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                               // [nwarps*ns]
    double* red_scratch = reinterpret_cast<double*>(smem + 8 * kMaxStreamWarps * 4);  // after barriers
    volatile int* abort_s = reinterpret_cast<volatile int*>(smem + 8 * kMaxStreamWarps * 4 +
                                                            8 * kMaxStreamWarps);
    float* rowacc = reinterpret_cast<float*>(smem + p.off_rowacc);
    uint8_t* ring = smem + p.off_ring;
    const uint8_t* xs = smem + p.off_x;
    const float* sx = reinterpret_cast<const float*>(smem + p.off_sx);
    constexpr int kChunkBytes = 32 * 144;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = blockDim.x >> 5, nthreads = blockDim.x;
    const int ns = p.ns, n_ops = p.n_ops;

    if (tid == 0) {
        for (int i = 0; i < nwarps * ns; ++i) mbar_init(&bars[i], 1);
        *abort_s = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // ---- per-warp weight stream: issue cursor runs ahead of the consume cursor ----
    const uint8_t* maps = static_cast<const uint8_t*>(p.maps);   // one 128-byte tensor map per operation
    // The operation table is read many times by every thread: keep it in shared memory when it
    // fits (a global read costs an L2 round trip at every operation boundary).
    const MegaOp* ops = p.ops;
    if (p.off_ops >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(smem + p.off_ops);
        const uint4* src = reinterpret_cast<const uint4*>(p.ops);
        for (int i = tid; i < n_ops * 4; i += nthreads) dst[i] = src[i];
        ops = reinterpret_cast<const MegaOp*>(smem + p.off_ops);
        __syncthreads();
    }
    int iop = 0, ii = 0;                 // next box to issue: operation, index within it
    MegaOp op_i = ops[0];
    WarpGeom gi = make_geom(op_i, warp, nwarps);
    int islot = 0, cslot = 0;            // ring slots of the next issue / next consume
    uint32_t cphase = 0;                 // parity of the consume slot's current use
    int inflight = 0;
    auto try_issue = [&]() {
        while (iop < n_ops && ii >= gi.my_n) {
            ++iop;
            ii = 0;
            if (iop < n_ops) { op_i = ops[iop]; gi = make_geom(op_i, warp, nwarps); }
        }
        if (iop >= n_ops || inflight >= ns) return;
        if (lane == 0) {
            const int u = warp + nwarps * ii;
            const int rb = u / gi.gpr, kg = u - rb * gi.gpr;
            uint64_t* bar = &bars[warp * ns + islot];
            fence_proxy_async();
            mbar_expect_tx(bar, kChunkBytes);
            sm100::tensor_load_2d(ring + static_cast<size_t>(warp * ns + islot) * kChunkBytes,
                                  maps + static_cast<size_t>(iop) * 128, kg * 144, gi.r0 + rb * 32, bar);
        }
        ++ii;
        ++inflight;
        if (++islot == ns) islot = 0;
    };
    for (int i = 0; i < ns; ++i) try_issue();

#if TCB_MEGA_TRACE
#define MTR(COL) do { if (p.trace && blockIdx.x == 0 && tid == 0) p.trace[o * 8 + (COL)] = clock64(); } while (0)
#else
#define MTR(COL) do { } while (0)
#endif
    unsigned long long target = p.base;
    bool failed = false;
    // Operations run in phases: a phase is a run of up to kMaxPhaseOps operations that share their
    // staged activations and need no barrier between them (q/k/v, gate/up).  A phase zeroes its row
    // accumulators once, runs all its boxes back to back and writes all its outputs at the end.
    for (int o = 0; o < n_ops && !failed;) {
        int oe = o + 1;
        while (oe < n_ops && oe - o < kMaxPhaseOps &&
               !(ops[oe].flags & (MOP_BARRIER | MOP_RESTAGE)))
            ++oe;
        const MegaOp op = ops[o];
        // Everyone must be done with the previous phase's shared memory; if this phase reads
        // another CTA's output, everyone in the grid must be done with the previous one.
        __syncthreads();
        MTR(0);
        if (op.flags & MOP_BARRIER) {
            // One 64-bit arrival counter that is never reset: barrier j of this launch is
            // complete when it reaches base + (j+1) * gridDim.  One thread per CTA arrives
            // (release) and polls (acquire); the wait is bounded.  (Measured alternatives - a
            // separately published generation word, per-CTA flag words, back-off - were slower.)
            target += gridDim.x;
            if (tid == 0) {
                // Arrival is a release-reduction: no value comes back, so the thread goes
                // straight to polling (an atomicAdd costs a full L2 round trip before the first
                // poll), and the release orders this CTA's outputs - made visible to this thread
                // by the block barrier above - before the arrival.  The acquire loads order
                // everyone's outputs before what follows the block barrier below.
                red_release_add_u64(p.counter, 1ULL);
                const long long t0 = clock64();
                while (ld_acquire_u64(p.counter) < target) {
                    if (clock64() - t0 > 2000000000LL) {
                        *abort_s = 1;
                        atomicOr(p.err, ERR_WAIT_TIMEOUT);
                        break;
                    }
                }
            }
            __syncthreads();
            if (*abort_s) { failed = true; break; }
        }
        MTR(1);
        if (op.flags & MOP_RESTAGE) {
            StreamParams sp;
            sp.X = op.X; sp.gamma = (op.flags & MOP_FUSED) ? op.gamma : nullptr;
            sp.K = op.K; sp.nb = op.K >> 5; sp.gpr = op.K >> 8; sp.eps = op.eps;
            sp.x_src_f16 = (op.flags & MOP_X_F32) ? 0 : 1;
            sp.off_x = p.off_x; sp.off_sx = p.off_sx;
#if TCB_MEGA_TRACE
            sp.trace = p.trace ? p.trace + 256 * 8 + o * 4 : nullptr;
#endif
            stage_activations_i16<1, true, true>(sp, smem, 8, red_scratch);
        }
        int acc_off[kMaxPhaseOps + 1];
        acc_off[0] = 0;
        for (int k = o; k < oe; ++k) {
            const WarpGeom g = make_geom(ops[k], warp, nwarps);
            acc_off[k - o + 1] = acc_off[k - o] + ((g.rows + 31) & ~31);
        }
        for (int i = tid; i < acc_off[oe - o]; i += nthreads) rowacc[i] = 0.f;
        __syncthreads();
        MTR(2);

        for (int k = o; k < oe && !failed; ++k) {
            const MegaOp opk = ops[k];
            const WarpGeom gc = make_geom(opk, warp, nwarps);
            float* acc = rowacc + acc_off[k - o];
            for (int i = 0; i < gc.my_n; ++i) {
                uint64_t* bar = &bars[warp * ns + cslot];
                if (!mbar_wait_bounded(bar, cphase)) { failed = true; break; }
                if (i == 0 && k == o) MTR(3);
                const int u = warp + nwarps * i;
                const int rb = u / gc.gpr, kg = u - rb * gc.gpr;
                const int rl = rb * 32 + lane;              // row within the CTA's range
                const bool valid = rl < gc.rows;
                uint32_t w[36];
                {
                    const uint4* src = reinterpret_cast<const uint4*>(
                        ring + static_cast<size_t>(warp * ns + cslot) * kChunkBytes +
                        static_cast<size_t>(lane) * 144);
#pragma unroll
                    for (int v = 0; v < 9; ++v) {
                        const uint4 t = src[v];
                        w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
                    }
                }
                __syncwarp();
                --inflight;
                if (++cslot == ns) { cslot = 0; cphase ^= 1u; }
                try_issue();                           // refill: this or a later operation's weights
                if (p.dbg_skip) {
                    if (valid && lane == 0) atomicAdd(&acc[0], __uint_as_float(w[0] ^ w[35]));
                } else {
                    float out[1] = {0.f};
                    group_dot_i16<FMT_Q4_0, 1, true>(w, xs, reinterpret_cast<const float2*>(sx), kg, gc.gpr,
                                                     opk.K, opk.K >> 5, out);
                    if (valid) atomicAdd(&acc[rl], out[0]);
                }
            }
        }
        MTR(4);
        if (__any_sync(0xffffffffu, failed)) { failed = true; }
        if (failed) { if (lane == 0) { *abort_s = 1; atomicOr(p.err, ERR_WAIT_TIMEOUT); } }
        __syncthreads();
        MTR(5);
        if (*abort_s) { failed = true; break; }
        for (int k = o; k < oe; ++k) {
            const MegaOp opk = ops[k];
            const WarpGeom gc = make_geom(opk, warp, nwarps);
            const float* acc = rowacc + acc_off[k - o];
            for (int i = tid; i < gc.rows; i += nthreads) {
                const float v = acc[i];
                if (opk.flags & MOP_Y_F32) static_cast<float*>(opk.Y)[gc.r0 + i] = v;
                else static_cast<__half*>(opk.Y)[gc.r0 + i] = __float2half_rn(v);
            }
        }
        o = oe;
    }
    if (failed) {
        // let copies that are still in flight land before the CTA's shared memory is released
        for (int i = 0; i < inflight; ++i) {
            (void)mbar_wait_bounded(&bars[warp * ns + cslot], cphase);
            if (++cslot == ns) { cslot = 0; cphase ^= 1u; }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Generic kernel: any K % 32 == 0, any alignment, any N.  One warp per output row, lanes over
// blocks, byte-granular loads.  Correctness path for shapes the streaming kernel rejects.
// ---------------------------------------------------------------------------------------
struct GenericParams {
    const uint8_t* W;
    const void* X;
    void* Y;
    const void* gamma;
    int M, N, K, nb;
    int fmt, x_f32, y_f32;
    float eps;
};

__device__ __forceinline__ float load_x(const void* X, size_t idx, int x_f32) {
    return x_f32 ? static_cast<const float*>(X)[idx]
                 : __half2float(static_cast<const __half*>(X)[idx]);
}

__global__ void __launch_bounds__(kThreads) gemv_q_generic_kernel(const GenericParams p) {
    __shared__ double red[kWarps];
    __shared__ float rstd_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bb = p.fmt == FMT_Q4_0 ? 18 : 34;
    pdl_launch_dependents();
    pdl_wait();
    for (int m = 0; m < p.M; ++m) {
        float rstd = 1.f;
        if (p.gamma != nullptr) {
            double ss = 0.0;
            for (int k = tid; k < p.K; k += kThreads) {
                const double v = static_cast<double>(load_x(p.X, static_cast<size_t>(m) * p.K + k, p.x_f32));
                ss += v * v;
            }
            ss = block_sum_f64(ss, red);
            if (tid == 0)
                rstd_s = 1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(p.K)) + p.eps);
            __syncthreads();
            rstd = rstd_s;
        }
        for (int n = blockIdx.x * kWarps + warp; n < p.N; n += gridDim.x * kWarps) {
            const uint8_t* row = p.W + static_cast<size_t>(n) * p.nb * bb;
            float acc = 0.f;
            for (int b = lane; b < p.nb; b += 32) {
                const uint8_t* blk = row + static_cast<size_t>(b) * bb;
                const float d = h2f(static_cast<uint16_t>(blk[0] | (blk[1] << 8)));
                float part = 0.f;
                for (int i = 0; i < 32; ++i) {
                    const size_t xi = static_cast<size_t>(m) * p.K + static_cast<size_t>(b) * 32 + i;
                    float xv = load_x(p.X, xi, p.x_f32);
                    if (p.gamma != nullptr)
                        xv = __fmul_rn(__fmul_rn(xv, rstd), load_x(p.gamma, b * 32 + i, p.x_f32));
                    int q;
                    if (p.fmt == FMT_Q4_0) {
                        const uint8_t byte = blk[2 + (i & 15)];
                        q = static_cast<int>((i < 16) ? (byte & 0x0f) : (byte >> 4)) - 8;
                    } else {
                        q = static_cast<int>(static_cast<int8_t>(blk[2 + i]));
                    }
                    part = fmaf(xv, static_cast<float>(q), part);
                }
                acc = fmaf(d, part, acc);
            }
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) {
                const size_t o = static_cast<size_t>(m) * p.N + n;
                if (p.y_f32) static_cast<float*>(p.Y)[o] = acc;
                else static_cast<__half*>(p.Y)[o] = __float2half_rn(acc);
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
template <typename KernelT, typename ParamT>
cudaError_t launch_with_attrs(KernelT kernel, dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, bool pdl, const ParamT& params) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

struct StreamPlan {
    bool ok = false;
    int warps = 8;
    int ns = 0;
    int grid = 0;
    int smem = 0;
    StreamParams p{};
};

// Decides whether the streaming kernel can take (fmt, K, alignment, MB rows of activations
// staged as fp16/fp32) and lays out its shared memory.
StreamPlan plan_stream(const GemvQArgs& a, int mb, bool stage_f32, const LaunchEnv& env) {
    StreamPlan pl;
    if (a.K % 256 != 0) return pl;
    if ((reinterpret_cast<uintptr_t>(a.W) & 15u) != 0) return pl;
    if ((reinterpret_cast<uintptr_t>(a.X) & 15u) != 0) return pl;
    if (a.gamma && (reinterpret_cast<uintptr_t>(a.gamma) & 15u) != 0) return pl;
    const int nb = a.K / 32, gpr = nb / 8;
    const int group_bytes = a.fmt == FMT_Q4_0 ? 144 : 272;
    const int chunk_bytes = 32 * group_bytes;
    static const int ctas_per_sm = [] {
        const char* v = std::getenv("TC_GEMV_CTAS_PER_SM");
        const int n = v ? std::atoi(v) : 1;
        return n >= 1 && n <= 4 ? n : 1;
    }();
    const int want = env.sm_count * ctas_per_sm;
    const int grid = a.N < want ? a.N : want;
    const int max_rows = (a.N + grid - 1) / grid + 1;

    int off = 8 * kMaxStreamWarps * 4 + 8 * kMaxStreamWarps;  // barriers (<= 4 stages) + scratch
    off = align_up(off, 16);
    const int off_rowacc = off;
    off += align_up(max_rows * mb * 4, 16);
    const int off_sx = off;
    off += align_up(mb * nb * 8, 16);
    const int off_x = off;
    off += align_up(mb * a.K * (stage_f32 ? 4 : 2), 128);
    const int off_ring = off;

    const int optin = env.smem_optin > 0 ? env.smem_optin : 232448;
    const int half_budget = optin / 2 - 1024;
    // Warp count: 16 warps (one CTA fills the SM: no co-resident successor, but twice the
    // latency hiding) when each SM has enough work to amortise it, else 8 warps with a ring
    // small enough for two CTAs (this kernel and the next one in the stream) per SM.
    static const int force_warps = [] {
        const char* v = std::getenv("TC_GEMV_WARPS");
        return v ? std::atoi(v) : 0;
    }();
    const long long bytes_per_cta = static_cast<long long>(a.N) * nb * (a.fmt == FMT_Q4_0 ? 18 : 34) / grid;
    int warps = bytes_per_cta >= (256 << 10) ? 16 : 8;
    if (force_warps == 8 || force_warps == 16) warps = force_warps;
    int ns = 0;
    if (warps == 16) {
        for (int cand = 3; cand >= 2; --cand)
            if (off_ring + 16 * cand * chunk_bytes <= optin - 2048) { ns = cand; break; }
        if (ns == 0) warps = 8;
    }
    if (warps == 8) {
        for (int cand = 4; cand >= 2; --cand)
            if (off_ring + 8 * cand * chunk_bytes <= half_budget) { ns = cand; break; }
        if (ns == 0)
            for (int cand = 3; cand >= 1; --cand)
                if (off_ring + 8 * cand * chunk_bytes <= optin) { ns = cand; break; }
    }
    if (ns == 0) return pl;

    pl.ok = true;
    pl.ns = ns;
    pl.grid = grid;
    pl.warps = warps;
    pl.smem = off_ring + warps * ns * chunk_bytes;
    StreamParams& p = pl.p;
    p.W = a.W; p.X = a.X; p.Y = a.Y; p.gamma = a.gamma; p.err = env.err_word;
    p.M = mb; p.N = a.N; p.K = a.K; p.nb = nb; p.gpr = gpr; p.ns = ns;
    p.y_f32 = a.y_f32 ? 1 : 0; p.eps = a.eps;
    p.off_rowacc = off_rowacc; p.off_sx = off_sx; p.off_x = off_x; p.off_ring = off_ring;
    p.max_rows = max_rows;
    static const int dbg_skip = [] { const char* v = std::getenv("TC_GEMV_DBG_SKIP"); return v ? std::atoi(v) : 0; }();
    p.dbg_skip = dbg_skip;
    return pl;
}

template <int FMT, bool XF32>
cudaError_t launch_stream_mb(int mb, const StreamPlan& pl, cudaStream_t st, bool pdl) {
    const dim3 grid(pl.grid), block(pl.warps * 32);
    switch (mb) {
        case 1: return launch_with_attrs(gemv_q_stream_kernel<FMT, XF32, 1>, grid, block, pl.smem, st, pdl, pl.p);
        case 2: return launch_with_attrs(gemv_q_stream_kernel<FMT, XF32, 2>, grid, block, pl.smem, st, pdl, pl.p);
        case 3: return launch_with_attrs(gemv_q_stream_kernel<FMT, XF32, 3>, grid, block, pl.smem, st, pdl, pl.p);
        default: return launch_with_attrs(gemv_q_stream_kernel<FMT, XF32, 4>, grid, block, pl.smem, st, pdl, pl.p);
    }
}

// Shared-memory plan of the box kernel for mb activation rows; pl.ok = false when the operation
// is outside its domain (K % 256, alignment) or the activations do not fit beside a ring.
StreamPlan plan_box(const GemvQArgs& a, int mb, const LaunchEnv& env) {
    StreamPlan pl;
    if (a.K % 256 != 0) return pl;
    if ((reinterpret_cast<uintptr_t>(a.W) & 15u) != 0) return pl;
    if ((reinterpret_cast<uintptr_t>(a.X) & 15u) != 0) return pl;
    if (a.gamma && (reinterpret_cast<uintptr_t>(a.gamma) & 15u) != 0) return pl;
    const int nb = a.K / 32, gpr = nb / 8;
    const int box_bytes = 32 * (a.fmt == FMT_Q4_0 ? 144 : 272);
    const int grid = a.N < env.sm_count * 8 ? (a.N + 7) / 8 < env.sm_count ? (a.N + 7) / 8 : env.sm_count
                                            : env.sm_count;
    const int max_rows = (a.N + grid - 1) / grid + 1;
    int off = 8 * kMaxStreamWarps * 4 + 8 * kMaxStreamWarps;  // barriers (<= 4 stages) + scratch
    off = align_up(off, 16);
    const int off_rowacc = off;
    off += align_up(mb * ((max_rows + 31) & ~31) * 4, 16);
    const int off_sx = off;
    off += align_up(mb * nb * 8, 16);
    const int off_x = off;
    off += align_up(mb * a.K * 2, 128);
    const int off_ring = align_up(off, 128);
    const int optin = env.smem_optin > 0 ? env.smem_optin : 232448;
    // 16 warps when every warp gets at least one box, else 8 (fewer barriers to initialise)
    const int units = ((max_rows + 31) / 32) * gpr;
    int warps = units >= 16 ? 16 : 8;
    int ns = 0;
    for (; warps >= 8 && ns == 0; warps -= 8)
        for (int cand = 4; cand >= 2; --cand)
            if (off_ring + warps * cand * box_bytes <= optin - 1024) { ns = cand; break; }
    if (ns == 0) return pl;
    warps += 8;
    // A box always spans 32 rows: rows per CTA that fall just past a multiple of 32 (74 -> 96 for
    // 11008 rows on 148 SMs) waste lanes and copies.  When that padding exceeds 25 % and the
    // operation is only a few rounds long, the streaming kernel (no padding) is faster
    // (measured: 11008 x 4096 8.8 us against 11.4 us; every other decode shape favours the box).
    const double rows_avg = static_cast<double>(a.N) / grid;
    const double padded = 32.0 * ((static_cast<int>(rows_avg + 0.999) + 31) / 32);
    if (padded > 1.25 * rows_avg && units <= 3 * warps) return pl;
    pl.ok = true;
    pl.ns = ns;
    pl.grid = grid;
    pl.warps = warps;
    pl.smem = off_ring + warps * ns * box_bytes;
    StreamParams& p = pl.p;
    p.W = a.W; p.X = a.X; p.Y = a.Y; p.gamma = a.gamma; p.err = env.err_word;
    p.M = mb; p.N = a.N; p.K = a.K; p.nb = nb; p.gpr = gpr; p.ns = ns;
    p.y_f32 = a.y_f32 ? 1 : 0; p.eps = a.eps;
    p.x_src_f16 = a.x_f32 ? 0 : 1;
    p.off_rowacc = off_rowacc; p.off_sx = off_sx; p.off_x = off_x; p.off_ring = off_ring;
    p.max_rows = max_rows;
    static const int dbg_skip = [] { const char* v = std::getenv("TC_GEMV_DBG_SKIP"); return v ? std::atoi(v) : 0; }();
    p.dbg_skip = dbg_skip;
    return pl;
}

template <typename KernelT>
cudaError_t launch_box(KernelT kernel, const StreamPlan& pl, const CUtensorMap& wmap, cudaStream_t st, bool pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(pl.warps * 32);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, pl.p, wmap);
}

template <int FMT>
cudaError_t launch_box_mb(int mb, const StreamPlan& pl, cudaStream_t st, bool pdl) {
    CUtensorMap wmap;
    // Q8_0 groups are 272 bytes: more than the 256 elements a box may have per dimension, so the
    // byte matrix is described in 4-byte elements there.
    constexpr int group_bytes = Fmt<FMT>::kGroupBytes;
    if (!encode_bytes_2d(&wmap, pl.p.W, static_cast<uint64_t>(pl.p.N),
                         static_cast<uint64_t>(pl.p.gpr) * group_bytes, group_bytes, 32,
                         FMT == FMT_Q4_0 ? 1 : 4))
        return cudaErrorNotSupported;
    switch (mb) {
        case 1: return launch_box(gemv_q_box_kernel<FMT, 1>, pl, wmap, st, pdl);
        case 2: return launch_box(gemv_q_box_kernel<FMT, 2>, pl, wmap, st, pdl);
        case 3: return launch_box(gemv_q_box_kernel<FMT, 3>, pl, wmap, st, pdl);
        default: return launch_box(gemv_q_box_kernel<FMT, 4>, pl, wmap, st, pdl);
    }
}

template <typename K>
cudaError_t set_smem(K kernel, int bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

cudaError_t init_decode_kernel(int smem_optin);

cudaError_t init_gemv_kernels(int smem_optin) {
    cudaError_t e = init_mma_kernels(smem_optin);
    if (e != cudaSuccess) return e;
    e = init_tc_kernels(smem_optin);
    if (e != cudaSuccess) return e;
    e = init_decode_kernel(smem_optin);
    if (e != cudaSuccess) return e;
#define TCB_SETB(FMT, MB)                                                         \
    e = set_smem(gemv_q_box_kernel<FMT, MB>, smem_optin);                         \
    if (e != cudaSuccess) return e;
    TCB_SETB(FMT_Q4_0, 1) TCB_SETB(FMT_Q4_0, 2) TCB_SETB(FMT_Q4_0, 3) TCB_SETB(FMT_Q4_0, 4)
    TCB_SETB(FMT_Q8_0, 1) TCB_SETB(FMT_Q8_0, 2) TCB_SETB(FMT_Q8_0, 3) TCB_SETB(FMT_Q8_0, 4)
#undef TCB_SETB
#define TCB_SET(FMT, XF, MB)                                                      \
    e = set_smem(gemv_q_stream_kernel<FMT, XF, MB>, smem_optin);                  \
    if (e != cudaSuccess) return e;
    TCB_SET(FMT_Q4_0, false, 1) TCB_SET(FMT_Q4_0, false, 2) TCB_SET(FMT_Q4_0, false, 3) TCB_SET(FMT_Q4_0, false, 4)
    TCB_SET(FMT_Q4_0, true, 1) TCB_SET(FMT_Q4_0, true, 2) TCB_SET(FMT_Q4_0, true, 3) TCB_SET(FMT_Q4_0, true, 4)
    TCB_SET(FMT_Q8_0, false, 1) TCB_SET(FMT_Q8_0, false, 2) TCB_SET(FMT_Q8_0, false, 3) TCB_SET(FMT_Q8_0, false, 4)
    TCB_SET(FMT_Q8_0, true, 1) TCB_SET(FMT_Q8_0, true, 2) TCB_SET(FMT_Q8_0, true, 3) TCB_SET(FMT_Q8_0, true, 4)
#undef TCB_SET
    return e;
}

cudaError_t launch_gemv_q(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                          int* launches, const char** name) {
    int count = 0;
    cudaError_t err = cudaSuccess;
    const char* used = "none";
    const size_t xsz = a.x_f32 ? 4 : 2, ysz = a.y_f32 ? 4 : 2;
    const bool fuse = a.gamma != nullptr;
    // The RMSNorm prologue keeps the normalised row in fp32, whatever the activation type.
    const bool stage_f32 = a.x_f32 || fuse;

    // Batched decode: the tcgen05 kernel reads the weights once for up to 32 activation rows.
    // It rounds dequantised weights to fp16, which only the fp16-activation bound allows.
    const bool want_tc = env.variant == VARIANT_TC ||
                         (env.variant == VARIANT_AUTO && a.M >= kTcMinBatch);
    if (want_tc && a.fmt == FMT_Q4_0 && !a.x_f32 && !fuse) {
        bool done = true;
        for (int m0 = 0; m0 < a.M; m0 += 32) {
            GemvQArgs s = a;
            s.M = (a.M - m0) < 32 ? (a.M - m0) : 32;
            s.X = static_cast<const uint8_t*>(a.X) + static_cast<size_t>(m0) * a.K * xsz;
            s.Y = static_cast<uint8_t*>(a.Y) + static_cast<size_t>(m0) * a.N * ysz;
            const cudaError_t te = launch_gemv_q4_tc(s, env, stream, &used);
            if (te == cudaErrorNotSupported && m0 == 0) { done = false; break; }
            if (te != cudaSuccess) { err = te; break; }
            ++count;
        }
        if (done) {
            if (launches) *launches += count;
            if (name) *name = used;
            return err;
        }
    }

    // The tensor-core dot kernel (two activation rows per launch) is selected explicitly.
    const bool try_mma = a.fmt == FMT_Q4_0 && env.variant == VARIANT_MMA;
    int step = kMaxMB;
    for (int m0 = 0; m0 < a.M && err == cudaSuccess; m0 += step) {
        if (try_mma) {
            GemvQArgs s2 = a;
            s2.M = (a.M - m0) < 2 ? (a.M - m0) : 2;
            s2.X = static_cast<const uint8_t*>(a.X) + static_cast<size_t>(m0) * a.K * xsz;
            s2.Y = static_cast<uint8_t*>(a.Y) + static_cast<size_t>(m0) * a.N * ysz;
            const cudaError_t me = launch_gemv_q4_mma(s2, env, stream, &used);
            if (me != cudaErrorNotSupported) {
                err = me;
                step = 2;
                ++count;
                continue;
            }
        }
        step = kMaxMB;
        const int mb = (a.M - m0) < kMaxMB ? (a.M - m0) : kMaxMB;
        GemvQArgs s = a;
        s.X = static_cast<const uint8_t*>(a.X) + static_cast<size_t>(m0) * a.K * xsz;
        s.Y = static_cast<uint8_t*>(a.Y) + static_cast<size_t>(m0) * a.N * ysz;
        s.M = mb;
        StreamPlan pl;
        static const bool use_box = [] { const char* v = std::getenv("TC_GEMV_BOX"); return !v || std::atoi(v) != 0; }();
        if (kActI16 && use_box && env.variant != VARIANT_GENERIC) {
            const StreamPlan pb = plan_box(s, mb, env);
            if (pb.ok) {
                const cudaError_t be = a.fmt == FMT_Q4_0 ? launch_box_mb<FMT_Q4_0>(mb, pb, stream, env.pdl)
                                                         : launch_box_mb<FMT_Q8_0>(mb, pb, stream, env.pdl);
                if (be != cudaErrorNotSupported) {
                    err = be;
                    used = a.fmt == FMT_Q4_0 ? "q4_0_gemv_box_sm100" : "q8_0_gemv_box_sm100";
                    ++count;
                    continue;
                }
            }
        }
        if (env.variant != VARIANT_GENERIC) pl = plan_stream(s, mb, stage_f32, env);
        if (pl.ok) {
            pl.p.x_src_f16 = a.x_f32 ? 0 : 1;
            if (a.fmt == FMT_Q4_0) {
                err = stage_f32 ? launch_stream_mb<FMT_Q4_0, true>(mb, pl, stream, env.pdl)
                                : launch_stream_mb<FMT_Q4_0, false>(mb, pl, stream, env.pdl);
                used = stage_f32 ? "q4_0_gemv_stream_f32x_sm100" : "q4_0_gemv_stream_sm100";
            } else {
                err = stage_f32 ? launch_stream_mb<FMT_Q8_0, true>(mb, pl, stream, env.pdl)
                                : launch_stream_mb<FMT_Q8_0, false>(mb, pl, stream, env.pdl);
                used = stage_f32 ? "q8_0_gemv_stream_f32x_sm100" : "q8_0_gemv_stream_sm100";
            }
        } else {
            GenericParams g;
            g.W = s.W; g.X = s.X; g.Y = s.Y; g.gamma = s.gamma;
            g.M = mb; g.N = s.N; g.K = s.K; g.nb = s.K / 32;
            g.fmt = s.fmt; g.x_f32 = s.x_f32; g.y_f32 = s.y_f32; g.eps = s.eps;
            int grid = (s.N + kWarps - 1) / kWarps;
            const int cap = env.sm_count > 0 ? env.sm_count * 8 : 1024;
            if (grid > cap) grid = cap;
            err = launch_with_attrs(gemv_q_generic_kernel, dim3(grid), dim3(kThreads), 0, stream,
                                    env.pdl, g);
            used = a.fmt == FMT_Q4_0 ? "q4_0_gemv_generic_sm100" : "q8_0_gemv_generic_sm100";
        }
        ++count;
    }
    if (launches) *launches += count;
    if (name) *name = used;
    return err;
}


cudaError_t init_decode_kernel(int smem_optin) {
    return cudaFuncSetAttribute(gemv_q4_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                smem_optin);
}

cudaError_t encode_decode_maps(const MegaOp* host_ops, int n_ops, void* host_maps) {
    static_assert(sizeof(CUtensorMap) == kDecodeMapBytes, "tensor map size");
    CUtensorMap* out = static_cast<CUtensorMap*>(host_maps);
    for (int i = 0; i < n_ops; ++i) {
        const MegaOp& op = host_ops[i];
        if (!encode_bytes_2d(&out[i], op.W, static_cast<uint64_t>(op.N),
                             static_cast<uint64_t>(op.K / 32) * 18u, 144u, 32u))
            return cudaErrorNotSupported;
    }
    return cudaSuccess;
}

cudaError_t launch_gemv_q4_decode(const MegaOp* host_ops, const MegaOp* dev_ops, const void* dev_maps,
                                  int n_ops, unsigned long long* counter, unsigned long long base,
                                  const LaunchEnv& env, cudaStream_t stream, int* barriers) {
    if (n_ops <= 0) return cudaErrorInvalidValue;
    int k_max = 0, n_max = 0, nbar = 0;
    for (int i = 0; i < n_ops; ++i)
        if (static_cast<unsigned long long>(host_ops[i].N) * static_cast<unsigned>(env.sm_count) >= (1ull << 32))
            return cudaErrorNotSupported;
    bool any_f32 = false;
    for (int i = 0; i < n_ops; ++i) {
        k_max = host_ops[i].K > k_max ? host_ops[i].K : k_max;
        n_max = host_ops[i].N > n_max ? host_ops[i].N : n_max;
        if (host_ops[i].flags & (MOP_X_F32 | MOP_FUSED)) any_f32 = true;
        if (host_ops[i].flags & MOP_BARRIER) ++nbar;
    }
    static const int want_warps = [] {
        const char* v = std::getenv("TC_MEGA_WARPS");
        const int n = v ? std::atoi(v) : 16;
        return (n == 8 || n == 16) ? n : 16;
    }();
    const int grid = env.sm_count;
    const int max_rows = (n_max + grid - 1) / grid + 1;
    const int optin = env.smem_optin > 0 ? env.smem_optin : 232448;
    MegaParams p;
    p.ops = dev_ops; p.maps = dev_maps; p.n_ops = n_ops; p.counter = counter; p.base = base; p.err = env.err_word;
    static const int dbg_skip = [] { const char* v = std::getenv("TC_GEMV_DBG_SKIP"); return v ? std::atoi(v) : 0; }();
    p.dbg_skip = dbg_skip;
    p.trace = nullptr;
#if TCB_MEGA_TRACE
    if (const char* s = std::getenv("TC_MEGA_TRACE")) p.trace = reinterpret_cast<long long*>(std::strtoull(s, nullptr, 0));
#endif
    int off = 8 * kMaxStreamWarps * 4 + 8 * kMaxStreamWarps + 16;   // barriers, scratch, abort flag
    off = align_up(off, 16);
    p.off_rowacc = off;
    {   // accumulators: the largest sum over a phase of the per-CTA rows, each rounded up to 32
        int worst = 0, run = 0, len = 0;
        for (int i = 0; i < n_ops; ++i) {
            const bool head = i == 0 || len >= kMaxPhaseOps ||
                              (host_ops[i].flags & (MOP_BARRIER | MOP_RESTAGE)) != 0;
            if (head) { run = 0; len = 0; }
            run += ((host_ops[i].N + grid - 1) / grid + 1 + 31) & ~31;
            ++len;
            worst = run > worst ? run : worst;
        }
        off += align_up(worst * 4, 16);
    }
    p.off_sx = off;
    off += align_up((k_max / 32) * 8, 16);
    p.off_x = off;
    off += align_up(k_max * 2, 128);
    p.off_ops = -1;
    if (n_ops * static_cast<int>(sizeof(MegaOp)) <= 32 * 1024) {
        p.off_ops = off;
        off += n_ops * static_cast<int>(sizeof(MegaOp));
    }
    p.off_ring = align_up(off, 128);
    off = p.off_ring;
    int warps = want_warps, ns = 0;
    for (; warps >= 8 && ns == 0; warps -= 8)
        for (int cand = 4; cand >= 2; --cand)
            if (off + warps * cand * 4608 <= optin - 1024) { ns = cand; break; }
    if (ns == 0) return cudaErrorNotSupported;
    warps += 8;   // undo the loop's last decrement
    p.ns = ns;
    const size_t smem = static_cast<size_t>(off) + static_cast<size_t>(warps) * ns * 4608;
    void* args[] = {&p};
    if (barriers) *barriers = nbar;
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(gemv_q4_decode_kernel),
                                       dim3(grid), dim3(warps * 32), args, smem, stream);
}


// ---------------------------------------------------------------------------------------
// Decode launch for callers that must not allocate.
//
// The persistent decode kernel needs two pieces of scratch in global memory: the operation table
// the CTAs walk and the arrival counter of its grid barrier.  The library normally keeps them in
// buffers it allocates on first use.  Some callers cannot have that: an inference server that
// has handed every byte of HBM to weights and KV cache at start-up, or a decode loop in which a
// cudaMalloc (which synchronises the whole device) is not acceptable at any point.  For them the
// same kernel is reachable with its scratch in the fixed array below, which is part of the
// library image on every GPU that loads it (48.25 KB: counter, table and tensor maps) and is never freed.
//
// Layout: bytes [0,256) arrival counter (first 8 bytes used), bytes [256, 256 + 256*64) the
// operation table, hence at most kStaticMaxOps operations per call.
// ---------------------------------------------------------------------------------------
constexpr int kStaticMaxOps = 256;
// counter (256 bytes) | operation table | tensor maps
constexpr size_t kStaticMapsOffset = 256 + kStaticMaxOps * sizeof(MegaOp);
static __device__ __align__(256) unsigned char
    g_decode_static_scratch[kStaticMapsOffset + kStaticMaxOps * kDecodeMapBytes];

namespace {
constexpr int kMaxDevices = 64;
unsigned char* g_static_scratch_addr[kMaxDevices] = {nullptr};

// The array's name is only a handle on the host; kernels need its device address, which differs
// per device and is looked up once per device with that device current.
cudaError_t static_scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (g_static_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_scratch_addr[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_scratch_addr[dev];
    return cudaSuccess;
}
}  // namespace

// ops: host array of n_ops operations in execution order (GemvQArgs with M == 1, Q4_0).  Builds
// the table on the stack (dependencies from pointer overlap, as the stream path does), copies it
// into the static scratch together with the operations' tensor maps, clears the arrival counter
// and launches.  No allocation of any kind.
cudaError_t launch_gemv_q4_decode_static(const GemvQArgs* ops, int n_ops, const LaunchEnv& env,
                                         cudaStream_t stream) {
    if (n_ops <= 0 || n_ops > kStaticMaxOps) return cudaErrorInvalidValue;
    MegaOp table[kStaticMaxOps];
    struct Span { uintptr_t lo, hi; };
    Span reads[3 * kStaticMaxOps], writes[kStaticMaxOps];
    int n_reads = 0, n_writes = 0;
    auto hit = [](const Span* v, int n, Span r) {
        for (int i = 0; i < n; ++i)
            if (r.lo < v[i].hi && v[i].lo < r.hi) return true;
        return false;
    };
    for (int i = 0; i < n_ops; ++i) {
        const GemvQArgs& a = ops[i];
        if (a.fmt != FMT_Q4_0 || a.M != 1 || a.N <= 0 || a.K <= 0 || a.K % 256 != 0 || !a.W || !a.X || !a.Y)
            return cudaErrorInvalidValue;
        if ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.X) |
             reinterpret_cast<uintptr_t>(a.gamma)) & 15u)
            return cudaErrorInvalidValue;
        const size_t xs = a.x_f32 ? 4 : 2, ys = a.y_f32 ? 4 : 2;
        const Span rx{reinterpret_cast<uintptr_t>(a.X), reinterpret_cast<uintptr_t>(a.X) + a.K * xs};
        const Span rg{reinterpret_cast<uintptr_t>(a.gamma),
                      reinterpret_cast<uintptr_t>(a.gamma) + (a.gamma ? a.K * xs : 0)};
        const Span rw{reinterpret_cast<uintptr_t>(a.W),
                      reinterpret_cast<uintptr_t>(a.W) + static_cast<size_t>(a.N) * (a.K / 32) * 18};
        const Span ry{reinterpret_cast<uintptr_t>(a.Y), reinterpret_cast<uintptr_t>(a.Y) + a.N * ys};
        bool barrier = i > 0 && (hit(writes, n_writes, rx) || hit(writes, n_writes, rg) ||
                                 hit(writes, n_writes, rw) || hit(writes, n_writes, ry) ||
                                 hit(reads, n_reads, ry));
        if (barrier) { n_reads = 0; n_writes = 0; }
        reads[n_reads++] = rx;
        if (a.gamma) reads[n_reads++] = rg;
        reads[n_reads++] = rw;
        writes[n_writes++] = ry;
        MegaOp& m = table[i];
        m.W = a.W; m.X = a.X; m.Y = a.Y; m.gamma = a.gamma; m.N = a.N; m.K = a.K; m.eps = a.eps;
        m.pad[0] = m.pad[1] = m.pad[2] = m.pad[3] = 0;
        m.flags = (barrier ? MOP_BARRIER : 0u) | (a.x_f32 ? MOP_X_F32 : 0u) |
                  (a.y_f32 ? MOP_Y_F32 : 0u) | (a.gamma ? MOP_FUSED : 0u);
        bool restage = true;
        if (i > 0 && !barrier) {
            const GemvQArgs& b = ops[i - 1];
            restage = !(b.X == a.X && b.gamma == a.gamma && b.K == a.K && b.x_f32 == a.x_f32);
        }
        if (restage) m.flags |= MOP_RESTAGE;
    }
    unsigned char* scratch = nullptr;
    cudaError_t e = static_scratch_for_current_device(&scratch);
    if (e != cudaSuccess) return e;
    // The array keeps whatever the previous call left: the counter must start from zero, the
    // table is overwritten.  (The host table lives on this stack frame: the copy from pageable
    // memory has consumed it when cudaMemcpyAsync returns.)
    e = cudaMemsetAsync(scratch, 0, 256, stream);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(scratch + 256, table, static_cast<size_t>(n_ops) * sizeof(MegaOp),
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
    // Tensor maps: encoded into a static host array and re-encoded only when the weights, shapes
    // or their order changed since the previous call (encoding costs about a microsecond each).
    alignas(64) static unsigned char maps[kStaticMaxOps * kDecodeMapBytes];
    static MegaOp maps_for[kStaticMaxOps];
    static int maps_n = 0;
    bool fresh = maps_n == n_ops;
    for (int i = 0; i < n_ops && fresh; ++i)
        fresh = maps_for[i].W == table[i].W && maps_for[i].N == table[i].N && maps_for[i].K == table[i].K;
    if (!fresh) {
        e = encode_decode_maps(table, n_ops, maps);
        if (e != cudaSuccess) return e;
        for (int i = 0; i < n_ops; ++i) maps_for[i] = table[i];
        maps_n = n_ops;
    }
    e = cudaMemcpyAsync(scratch + kStaticMapsOffset, maps, static_cast<size_t>(n_ops) * kDecodeMapBytes,
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
    return launch_gemv_q4_decode(table, reinterpret_cast<const MegaOp*>(scratch + 256),
                                 scratch + kStaticMapsOffset, n_ops,
                                 reinterpret_cast<unsigned long long*>(scratch), 0ULL, env, stream,
                                 nullptr);
}

}  // namespace tcb
