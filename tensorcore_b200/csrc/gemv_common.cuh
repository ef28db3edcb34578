// Device code shared by the quantized GEMV kernels (single-operation kernels in gemv_q.cu, the
// persistent decode kernel in decode_q4.cu): PTX wrappers for mbarriers, bulk copies and dp2a,
// the int16 activation staging with the fused RMSNorm prologue, and the integer dot product of
// one 8-block group.
#pragma once

#include "kernels.h"
#include "sm100_prims.cuh"

#include <cuda_fp16.h>

namespace tcb {
namespace {

constexpr int kWarps = 8;               // generic kernel
constexpr int kThreads = kWarps * 32;
constexpr int kMaxStreamWarps = 16;     // streaming kernel: 8 or 16 warps, chosen per launch
constexpr int kMaxStreamThreads = kMaxStreamWarps * 32;
constexpr int kGroupBlocks = 8;
constexpr int kMaxMB = 4;
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
    int x_acc = 0; // 0: X has the declared type; 1: X points at fp32 accumulators taken as they are;
                   // 2: fp32 accumulators whose values are rounded to fp16 first (the producer's
                   // result type) - gamma keeps the declared type in both cases
    // Persistent kernel only: the staging pass also stores elements [fin_lo, fin_hi) of the row it
    // has just loaded to fin_Y (fp16 when x_acc == 2, fp32 when x_acc == 1): the producer's result
    // buffer, which nothing has written yet.
    void* fin_Y = nullptr;
    int fin_lo = 0, fin_hi = 0;
    float eps;
    // shared-memory offsets (bytes)
    int off_rowacc, off_sx, off_x, off_ring;
    int max_rows;  // rows per CTA upper bound
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
// The same test, but the hardware may park the thread for up to `ns` nanoseconds while the phase is
// incomplete (it wakes as soon as the phase completes): a waiting warp then takes no issue slots
// from the warps that share its scheduler.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after about a second and reports false.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < 1000; ++i)
        if (mbar_try_wait_parked(bar, parity, 1000000u)) return true;     // up to a millisecond each
    return false;
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
__device__ __forceinline__ uint16_t lo16(uint32_t v) { return static_cast<uint16_t>(v); }
__device__ __forceinline__ uint16_t hi16(uint32_t v) { return static_cast<uint16_t>(v >> 16); }
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ uint32_t get4(const uint4& v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// ---------------------------------------------------------------------------------------
// Activation staging, chunk-transposed layout (streaming kernel: a lane per K group).  Element k
// of a staged int16 row sits at ((c*gpr + kg)*16 + (k&7)*2) with kg = k>>8, c = (k&255)>>3
// (32 chunks per group), so lanes holding consecutive groups kg read consecutive 16-byte chunks.
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

// COHERENT: the activations may have been written by other CTAs of the same (persistent)
// kernel, so they are read with L2-coherent loads instead of the read-only path.
template <bool COHERENT, typename T>
__device__ __forceinline__ T ld_act(const T* ptr) {
    return COHERENT ? __ldcg(ptr) : __ldg(ptr);
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

// Eight consecutive values starting at element elem0.  kind 0: fp16 array; 1: fp32 array;
// 2: fp32 array whose values are rounded to fp16 first (accumulators of an fp16 result).
template <bool COHERENT>
__device__ __forceinline__ void load8(const void* base, int kind, size_t elem0, float (&v)[8]) {
    if (kind == 0) {
        const uint4 t = ld_act<COHERENT>(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + elem0));
        v[0] = h2f(lo16(t.x)); v[1] = h2f(hi16(t.x)); v[2] = h2f(lo16(t.y)); v[3] = h2f(hi16(t.y));
        v[4] = h2f(lo16(t.z)); v[5] = h2f(hi16(t.z)); v[6] = h2f(lo16(t.w)); v[7] = h2f(hi16(t.w));
    } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem0);
        const float4 a = ld_act<COHERENT>(src), b = ld_act<COHERENT>(src + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (kind == 2) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __half2float(__float2half_rn(v[e]));
        }
    }
}

// Quantises one 8-value chunk (index i of row m) held in v[] and stores it; the four lanes of a
// quad hold the four chunks of a 32-element block and share its scale.  Every lane of the warp
// calls this (dead lanes with live = false and zeros) so the quad shuffles are among live lanes.
template <bool NATURAL>
__device__ __forceinline__ void quantise_chunk(const float (&v)[8], bool live, int i, int m, int zp,
                                               bool pow2, int gpr, int nb, uint4* dst, float2* sx2) {
    float amax = 0.f, bad = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        amax = fmaxf(amax, fabsf(v[e]));
        bad = fmaf(v[e], 0.f, bad);       // NaN as soon as one element is NaN or infinite
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    bad += __shfl_xor_sync(0xffffffffu, bad, 1);
    bad += __shfl_xor_sync(0xffffffffu, bad, 2);
    // fp16 sources get a power-of-two scale (block maximum mapped into [16384, 32768)): every
    // element within a factor 16 of the maximum is then represented exactly.
    float scale = amax * (1.0f / 32767.0f), inv = amax > 0.f ? 32767.0f / amax : 0.f;
    if (pow2 && amax > 0.f) {
        const uint32_t e = __float_as_uint(amax) & 0x7f800000u;
        scale = __uint_as_float(e - (14u << 23));
        inv = __uint_as_float((254u << 23) - (e - (14u << 23)));
    }
    // A block that holds a NaN or an infinity gets a NaN scale, so every result that uses the
    // block is NaN, as the reference's fp32 multiply-accumulate would make it non-finite
    // (lib/ops/quantized_cpu.cpp:193-228); fmaxf alone would drop a NaN silently.
    scale += bad;
    int q[8], isum = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        // round to nearest even without the conversion unit: adding 1.5 * 2^23 leaves the
        // integer in the low mantissa bits.  |v * inv| < 32767.5 by construction (the power-of-two
        // scale maps an fp16 maximum below 32753), so the result fits int16 without a clamp; a
        // block with a NaN or an infinity has arbitrary codes and a NaN scale.
        q[e] = __float_as_int(__fadd_rn(v[e] * inv, 12582912.0f)) - 0x4B400000;
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

// Stores those of the eight values v[] (elements 8*i .. 8*i+7 of a row) that lie in [lo, hi).
__device__ __forceinline__ void store8_range(void* Y, bool y_f32, int i, const float (&v)[8], int lo, int hi) {
    const int k0 = 8 * i;
    if (k0 + 8 <= lo || k0 >= hi) return;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int k = k0 + e;
        if (k >= lo && k < hi) {
            if (y_f32) static_cast<float*>(Y)[k] = v[e];
            else static_cast<__half*>(Y)[k] = __float2half_rn(v[e]);
        }
    }
}

// Stages MB rows as int16 + per-block scales.  With gamma the RMSNorm prologue runs first: sum of
// squares (fp32, pairwise: the relative error, about 1e-7, is far below what the int16 staging
// resolves, and fp64 arithmetic is slow on this part), rstd = 1/sqrtf(ss/K+eps),
// row = (x*rstd)*gamma in fp32 - the reference's order (lib/ops/quantized_cpu.cpp:276-284) - and
// that row is what gets quantised.  `zp` is the weight zero point (8 for
// Q4_0 codes taken as unsigned nibbles, 0 for Q8_0's signed bytes).
// NATURAL: the staged row and the scales keep the order of k (every lane of a warp then reads the
// same activations: one broadcast per load); otherwise the chunk-transposed layout above.
// DEFER (MB == 1): the block-wide reduction is taken off the critical path.  The row x*gamma is
// quantised (the per-block scales make the result independent of a common factor), every warp
// leaves its partial sum of squares in red_scratch[warp] (as float), and the caller multiplies
// its results by rstd_from_partials() instead.
// Rows of up to 4 chunks per thread (K <= 32 * blockDim) are loaded once, activations and gamma
// in the same round trip, and held in registers; longer rows are streamed.
__device__ __forceinline__ float sumsq8(const float (&v)[8]) {
    const float s01 = fmaf(v[0], v[0], v[1] * v[1]), s23 = fmaf(v[2], v[2], v[3] * v[3]);
    const float s45 = fmaf(v[4], v[4], v[5] * v[5]), s67 = fmaf(v[6], v[6], v[7] * v[7]);
    return (s01 + s23) + (s45 + s67);
}

// After a DEFER staging pass and its closing block barrier: 1/sqrt(mean square + eps), the same
// bits in every thread (each warp adds the per-warp partials in the same tree order).
__device__ __forceinline__ float rstd_from_partials(const double* red_scratch, int K, float eps) {
    const int nwarps = blockDim.x >> 5, l = threadIdx.x & 31;
    float t = l < nwarps ? reinterpret_cast<const float*>(red_scratch)[l] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return 1.0f / sqrtf(t / static_cast<float>(K) + eps);
}

template <int MB, bool COHERENT = false, bool NATURAL = false, bool DEFER = false>
__device__ void stage_activations_i16(const StreamParams& p, uint8_t* smem, int zp, double* red_scratch) {
    static_assert(!DEFER || MB == 1, "deferred normalisation keeps one partial sum per warp");
    const int K = p.K, gpr = p.gpr, nb = p.nb;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int nchunks = K >> 3;
    const bool f16 = p.x_src_f16 != 0;
    const int xkind = p.x_acc ? p.x_acc : (f16 ? 0 : 1), gkind = f16 ? 0 : 1;
    const bool fused = p.gamma != nullptr;
    const bool pow2 = (f16 || p.x_acc == 2) && !fused;
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
                    load8<COHERENT>(p.X, xkind, row0 + 8 * static_cast<size_t>(i), v[r]);
                    if (fused) load8<false>(p.gamma, gkind, 8 * static_cast<size_t>(i), g[r]);
                }
            }
            if (p.fin_Y != nullptr) {
#pragma unroll
                for (int r = 0; r < kHold; ++r) {
                    const int i = tid + r * nthreads;
                    if (i < nchunks) store8_range(p.fin_Y, p.x_acc == 1, i, v[r], p.fin_lo, p.fin_hi);
                }
            }
            float rstd = 1.0f;
            if (fused) {
                float ss = (sumsq8(v[0]) + sumsq8(v[1])) + (sumsq8(v[2]) + sumsq8(v[3]));
                if (DEFER) {
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if ((tid & 31) == 0) reinterpret_cast<float*>(red_scratch)[tid >> 5] = ss;
                } else {
                    ss = block_sum_f32(ss, reinterpret_cast<float*>(red_scratch));
                    rstd = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
                }
            }
#pragma unroll
            for (int r = 0; r < kHold; ++r) {
                const int i = tid + r * nthreads;
                if (r * nthreads >= nchunks) break;   // uniform: no lane has a chunk in this round
                if (fused) {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        v[r][e] = DEFER ? __fmul_rn(v[r][e], g[r][e]) : __fmul_rn(__fmul_rn(v[r][e], rstd), g[r][e]);
                }
                quantise_chunk<NATURAL>(v[r], i < nchunks, i, m, zp, pow2, gpr, nb, dst, sx2);
            }
        } else {
            float rstd = 1.0f, ss = 0.f;
            if (fused && !DEFER) {
                for (int i = tid; i < nchunks; i += nthreads) {
                    float v[8];
                    load8<COHERENT>(p.X, xkind, row0 + 8 * static_cast<size_t>(i), v);
                    ss += sumsq8(v);
                }
                ss = block_sum_f32(ss, reinterpret_cast<float*>(red_scratch));
                rstd = 1.0f / sqrtf(ss / static_cast<float>(K) + p.eps);
            }
            for (int base = 0; base < nchunks; base += nthreads) {
                const int i = base + tid;
                const bool live = i < nchunks;
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
                if (live) {
                    load8<COHERENT>(p.X, xkind, row0 + 8 * static_cast<size_t>(i), v);
                    if (p.fin_Y != nullptr) store8_range(p.fin_Y, p.x_acc == 1, i, v, p.fin_lo, p.fin_hi);
                    if (fused) {
                        float g[8];
                        load8<false>(p.gamma, gkind, 8 * static_cast<size_t>(i), g);
                        if (DEFER) ss += sumsq8(v);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            v[e] = DEFER ? __fmul_rn(v[e], g[e]) : __fmul_rn(__fmul_rn(v[e], rstd), g[e]);
                    }
                }
                quantise_chunk<NATURAL>(v, live, i, m, zp, pow2, gpr, nb, dst, sx2);
            }
            if (fused && DEFER) {
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if ((tid & 31) == 0) reinterpret_cast<float*>(red_scratch)[tid >> 5] = ss;
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

}  // namespace
}  // namespace tcb
