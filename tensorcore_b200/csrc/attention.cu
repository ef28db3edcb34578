// Scaled-dot-product attention forward for decode: few query rows against a long K/V cache.
//
// Interface replaced: tc_attention_forward (include/tensorcore/attention.h:24-60; arithmetic of
// lib/ops/attention_cpu.cpp:131-277): fp16 Q [B,H,Sq,D], K/V [B,Hkv,Sk,D], O [B,H,Sq,D], optional
// fp32 LSE [B,H,Sq]; softmax in fp32; causal mask (key index > query index), sliding window
// (query - key > window), ALiBi (score -= slope * (query - key)), grouped-query heads.
//
// One query row is a streaming pass over its head's K and V (2 * Sk * D * 2 bytes): HBM-bound.  A
// row's keys are cut into chunks so that B * H * Sq * chunks CTAs fill the GPU (a decode step has
// only B * H rows); every CTA keeps an online-softmax state (running maximum m, denominator l,
// unnormalised output o[D]) for its chunk:
//   scores    a lane takes a key: 32 keys per warp step, the key rows read with 16-byte loads,
//             fp32 dot products against the query row held in shared memory;
//   softmax   warp-wide maximum, p = exp(s - m), running rescale;
//   output    the lanes switch to a slice of D each and walk the step's 32 value rows (one
//             coalesced row per load), p broadcast by shuffle.
// The warps of a CTA are merged through shared memory; with one chunk the CTA writes O (and LSE)
// itself, otherwise it leaves (m, l, o) in scratch and a second small kernel merges the chunks.
// No tensor cores: with one to a few query rows the work is a matrix-vector product.
#include "kernels.h"

#include <cuda_fp16.h>
#include <cstdint>

namespace tcb {
namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnMaxD = 128;

struct AttnParams {
    const __half* Q;
    const __half* K;
    const __half* V;
    __half* O;
    float* LSE;           // may be null
    float* part;          // [rows][chunks][D + 2] when chunks > 1
    const float* slopes;  // device copy of the ALiBi slopes, or null
    int B, Hq, Hkv, Sq, Sk, D;
    int chunks, keys_per_chunk;
    float scale;
    int causal, window;
};

__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kAttnWarps * 32) attention_decode_kernel(const AttnParams p) {
    __shared__ float q_s[kAttnMaxD];
    __shared__ float o_s[kAttnWarps][kAttnMaxD];
    __shared__ float m_s[kAttnWarps], l_s[kAttnWarps];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.x, chunk = blockIdx.y;          // row = (b * Hq + h) * Sq + i
    const int i = row % p.Sq, bh = row / p.Sq, h = bh % p.Hq, b = bh / p.Hq;
    const int hkv = h / (p.Hq / p.Hkv);
    const int D = p.D;
    const __half* q = p.Q + static_cast<size_t>(row) * D;
    const __half* Kh = p.K + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    const __half* Vh = p.V + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    for (int d = tid; d < D; d += blockDim.x) q_s[d] = __half2float(q[d]);
    __syncthreads();
    const float slope = p.slopes ? p.slopes[h] : 0.f;
    const int k0 = chunk * p.keys_per_chunk, k1 = min(p.Sk, k0 + p.keys_per_chunk);

    // this lane's slice of the output: `per` consecutive elements when D is a multiple of 32 (one
    // vector load per value row), else elements lane, lane + 32, ...
    const int per = (D & 31) == 0 ? D >> 5 : 0;
    auto elem = [&](int t) { return per ? lane * per + t : lane + 32 * t; };
    float o[kAttnMaxD / 32];
#pragma unroll
    for (int t = 0; t < kAttnMaxD / 32; ++t) o[t] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j0 = k0 + warp * 32; j0 < k1; j0 += kAttnWarps * 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j < k1) {
            const __half* kr = Kh + static_cast<size_t>(j) * D;
            float acc = 0.f;
            if ((D & 7) == 0) {
                for (int d = 0; d < D; d += 8) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
                    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float2 f = __half22float2(h2[t]);
                        acc = fmaf(q_s[d + 2 * t], f.x, acc);
                        acc = fmaf(q_s[d + 2 * t + 1], f.y, acc);
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) acc = fmaf(q_s[d], __half2float(kr[d]), acc);
            }
            s = acc * p.scale;
            if (p.causal && j > i) s = -INFINITY;
            if (p.window > 0 && i - j > p.window) s = -INFINITY;
            if (p.slopes) s -= slope * static_cast<float>(i - j);
        }
        float m_new = fmaxf(m, warp_max(s));
        if (!(m_new > -INFINITY)) continue;                   // everything so far is masked
        const float keep = m > -INFINITY ? __expf(m - m_new) : 0.f;
        float pj = __expf(s - m_new);                         // 0 for masked keys
        if (!(s > -INFINITY)) pj = 0.f;
        l = l * keep + warp_sum(pj);
#pragma unroll
        for (int t = 0; t < kAttnMaxD / 32; ++t) o[t] *= keep;
        const int n = min(32, k1 - j0);
        for (int c = 0; c < n; ++c) {
            const float pc = __shfl_sync(0xffffffffu, pj, c);
            if (pc == 0.f) continue;                          // warp-uniform
            const __half* vr = Vh + static_cast<size_t>(j0 + c) * D;
            if (per == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(vr + 4 * lane);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 bq = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                o[0] = fmaf(pc, a.x, o[0]); o[1] = fmaf(pc, a.y, o[1]);
                o[2] = fmaf(pc, bq.x, o[2]); o[3] = fmaf(pc, bq.y, o[3]);
            } else if (per == 2) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(vr + 2 * lane));
                o[0] = fmaf(pc, a.x, o[0]); o[1] = fmaf(pc, a.y, o[1]);
            } else {
#pragma unroll
                for (int t = 0; t < kAttnMaxD / 32; ++t) {
                    const int d = elem(t);
                    if (d < D && (per == 0 || t < per)) o[t] = fmaf(pc, __half2float(vr[d]), o[t]);
                }
            }
        }
        m = m_new;
    }
    // merge the CTA's warps
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int t = 0; t < kAttnMaxD / 32; ++t) {
        const int d = elem(t);
        if (d < D && (per == 0 || t < per)) o_s[warp][d] = o[t];
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w]);
    float ll = 0.f;
    for (int w = 0; w < kAttnWarps; ++w) ll += m_s[w] > -INFINITY ? l_s[w] * __expf(m_s[w] - mm) : 0.f;
    for (int d = tid; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < kAttnWarps; ++w)
            if (m_s[w] > -INFINITY) acc += o_s[w][d] * __expf(m_s[w] - mm);
        if (p.chunks == 1) {
            p.O[static_cast<size_t>(row) * D + d] = __float2half_rn(ll != 0.f ? acc / ll : 0.f);
        } else {
            p.part[(static_cast<size_t>(row) * p.chunks + chunk) * (D + 2) + 2 + d] = acc;
        }
    }
    if (tid == 0) {
        if (p.chunks == 1) {
            if (p.LSE) p.LSE[row] = mm + logf(fmaxf(ll, 1e-30f));
        } else {
            float* dst = p.part + (static_cast<size_t>(row) * p.chunks + chunk) * (D + 2);
            dst[0] = mm;
            dst[1] = ll;
        }
    }
}

// Merges the chunks of a row: one warp per row.
__global__ void attention_merge_kernel(const AttnParams p, int rows) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int D = p.D;
    const float* base = p.part + static_cast<size_t>(row) * p.chunks * (D + 2);
    float mm = -INFINITY;
    for (int c = 0; c < p.chunks; ++c) mm = fmaxf(mm, base[static_cast<size_t>(c) * (D + 2)]);
    float ll = 0.f;
    for (int c = 0; c < p.chunks; ++c) {
        const float mc = base[static_cast<size_t>(c) * (D + 2)];
        if (mc > -INFINITY) ll += base[static_cast<size_t>(c) * (D + 2) + 1] * __expf(mc - mm);
    }
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int c = 0; c < p.chunks; ++c) {
            const float mc = base[static_cast<size_t>(c) * (D + 2)];
            if (mc > -INFINITY) acc += base[static_cast<size_t>(c) * (D + 2) + 2 + d] * __expf(mc - mm);
        }
        p.O[static_cast<size_t>(row) * D + d] = __float2half_rn(ll != 0.f ? acc / ll : 0.f);
    }
    if (lane == 0 && p.LSE) p.LSE[row] = mm + logf(fmaxf(ll, 1e-30f));
}

}  // namespace

size_t attention_scratch_floats(int rows, int Sk, int D, int sm_count, int* chunks_out) {
    // enough CTAs for two per SM, chunks of at least 256 keys
    int chunks = (2 * sm_count + rows - 1) / rows;
    const int most = (Sk + 255) / 256;
    if (chunks > most) chunks = most;
    if (chunks < 1) chunks = 1;
    if (chunks_out) *chunks_out = chunks;
    return chunks > 1 ? static_cast<size_t>(rows) * chunks * (D + 2) : 0;
}

cudaError_t launch_attention_forward(const void* Q, const void* K, const void* V, void* O, float* LSE,
                                     float* scratch, const float* slopes_dev, int B, int Hq, int Hkv, int Sq,
                                     int Sk, int D, float scale, bool causal, int window, int sm_count,
                                     cudaStream_t stream, int* launches) {
    if (D <= 0 || D > kAttnMaxD) return cudaErrorNotSupported;
    const long long rows_ll = static_cast<long long>(B) * Hq * Sq;
    if (rows_ll <= 0 || rows_ll > 0x7fffffffLL) return cudaErrorNotSupported;
    const int rows = static_cast<int>(rows_ll);
    AttnParams p;
    p.Q = static_cast<const __half*>(Q); p.K = static_cast<const __half*>(K); p.V = static_cast<const __half*>(V);
    p.O = static_cast<__half*>(O); p.LSE = LSE; p.part = scratch; p.slopes = slopes_dev;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk; p.D = D;
    int chunks = 1;
    (void)attention_scratch_floats(rows, Sk, D, sm_count, &chunks);
    if (chunks > 1 && !scratch) chunks = 1;
    if (chunks > 65535) chunks = 65535;
    p.chunks = chunks;
    p.keys_per_chunk = (Sk + chunks - 1) / chunks;
    p.scale = scale; p.causal = causal ? 1 : 0; p.window = window;
    attention_decode_kernel<<<dim3(rows, chunks), kAttnWarps * 32, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (chunks > 1) {
        attention_merge_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(p, rows);
        e = cudaGetLastError();
        if (e == cudaSuccess && launches) *launches += 1;
    }
    return e;
}

}  // namespace tcb
