// Scaled-dot-product attention forward for decode: few query rows against a long K/V cache.
//
// Interface replaced: tc_attention_forward (include/tensorcore/attention.h:24-60; arithmetic of
// lib/ops/attention_cpu.cpp:131-277): fp16 Q [B,H,Sq,D], K/V [B,Hkv,Sk,D], O [B,H,Sq,D], optional
// fp32 LSE [B,H,Sq]; softmax in fp32; causal mask (key index > query index), sliding window
// (query - key > window), ALiBi (score -= slope * (query - key)), grouped-query heads.
//
// One query row is a streaming pass over its head's K and V (2 * Sk * D * 2 bytes): HBM-bound.
//   * The query heads that share a K/V head (grouped-query attention) are handled by ONE CTA, so
//     the cache is read once per K/V head, not once per query head.
//   * A row's keys are cut into chunks so that about eight CTAs per SM are in flight (a decode step
//     has only B * Hkv * Sq groups); every CTA keeps an online-softmax state per query head (running
//     maximum m, denominator l, unnormalised output o[D]) for its chunk.
//   * head_dim 128 (attention_decode128_kernel): every load is a coalesced 512-byte piece of the
//     cache, 16 lanes per key; see the kernel.
//   * Other head_dims (attention_decode_kernel): a lane takes a key for the scores (D / 8
//     independent 16-byte loads, the query rows in shared memory), then the lanes switch to a
//     slice of D each and walk the step's 32 value rows, eight row loads in flight at a time, the
//     probabilities broadcast by shuffle.
// The warps of a CTA are merged through shared memory; with one chunk the CTA writes O (and LSE)
// itself, otherwise it leaves (m, l, o) in scratch and a second small kernel merges the chunks.
// head_dim 64 is compiled with fixed trip counts; any other head_dim <= 128 takes a generic
// instance of the same code.  No tensor cores: with one to a few query rows the work is a
// matrix-vector product.
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
    int group;            // query heads a CTA handles together (attention_group)
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

// DC: head_dim when it is 64 or 128 (fixed trip counts), 0 for the generic instance.  G: query heads
// per CTA.
template <int DC, int G>
__global__ void __launch_bounds__(kAttnWarps * 32) attention_decode_kernel(const AttnParams p) {
    // the merge kernel that follows may be set up now; it waits for this grid before it reads anything
    asm volatile("griddepcontrol.launch_dependents;");
    constexpr int kPer = DC ? DC / 32 : kAttnMaxD / 32;      // output elements per lane
    __shared__ float q_s[G][kAttnMaxD];
    __shared__ float o_s[kAttnWarps][G][kAttnMaxD];
    __shared__ float m_s[kAttnWarps][G], l_s[kAttnWarps][G];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = DC ? DC : p.D;
    // blockIdx.x = ((b * heads_per_grid) + hg) * Sq + i, where hg counts groups of G query heads
    const int groups = p.Hq / G;
    const int i = blockIdx.x % p.Sq, bg = blockIdx.x / p.Sq, hg = bg % groups, b = bg / groups;
    const int h0 = hg * G;                                   // first query head of the group
    const int hkv = h0 / (p.Hq / p.Hkv);
    const int chunk = blockIdx.y;
    const __half* Kh = p.K + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    const __half* Vh = p.V + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    for (int t = tid; t < G * D; t += blockDim.x) {
        const int g = t / D, d = t - g * D;
        q_s[g][d] = __half2float(p.Q[((static_cast<size_t>(b) * p.Hq + h0 + g) * p.Sq + i) * D + d]);
    }
    __syncthreads();
    float slope[G];
#pragma unroll
    for (int g = 0; g < G; ++g) slope[g] = p.slopes ? p.slopes[h0 + g] : 0.f;
    const int k0 = chunk * p.keys_per_chunk, k1 = min(p.Sk, k0 + p.keys_per_chunk);

    // this lane's slice of the output: `per` consecutive elements when D is a multiple of 32 (one
    // vector load per value row), else elements lane, lane + 32, ...
    const int per = (D & 31) == 0 ? D >> 5 : 0;
    auto elem = [&](int t) { return per ? lane * per + t : lane + 32 * t; };
    float o[G][kPer];
    float m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int t = 0; t < kPer; ++t) o[g][t] = 0.f;
    }
    for (int j0 = k0 + warp * 32; j0 < k1; j0 += kAttnWarps * 32) {
        const int j = j0 + lane;
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = -INFINITY;
        if (j < k1) {
            const __half* kr = Kh + static_cast<size_t>(j) * D;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.f;
            if (DC) {
                uint4 raw[DC ? DC / 8 : 1];
#pragma unroll
                for (int c = 0; c < DC / 8; ++c) raw[c] = __ldg(reinterpret_cast<const uint4*>(kr) + c);   // all in flight
#pragma unroll
                for (int c = 0; c < DC / 8; ++c) {
                    const __half2* h2 = reinterpret_cast<const __half2*>(&raw[c]);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float2 f = __half22float2(h2[t]);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            acc[g] = fmaf(q_s[g][8 * c + 2 * t], f.x, acc[g]);
                            acc[g] = fmaf(q_s[g][8 * c + 2 * t + 1], f.y, acc[g]);
                        }
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) {
                    const float kv = __half2float(kr[d]);
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g] = fmaf(q_s[g][d], kv, acc[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float sc = acc[g] * p.scale;
                if (p.causal && j > i) sc = -INFINITY;
                if (p.window > 0 && i - j > p.window) sc = -INFINITY;
                if (p.slopes) sc -= slope[g] * static_cast<float>(i - j);
                s[g] = sc;
            }
        }
        float pj[G];
        bool any = false;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float m_new = fmaxf(m[g], warp_max(s[g]));
            pj[g] = 0.f;
            if (m_new > -INFINITY) {                          // else everything so far is masked
                const float keep = m[g] > -INFINITY ? __expf(m[g] - m_new) : 0.f;
                if (s[g] > -INFINITY) pj[g] = __expf(s[g] - m_new);
                l[g] = l[g] * keep + warp_sum(pj[g]);
#pragma unroll
                for (int t = 0; t < kPer; ++t) o[g][t] *= keep;
                m[g] = m_new;
                any = true;
            }
        }
        if (!any) continue;                                   // warp-uniform
        const int n = min(32, k1 - j0);
        constexpr int kRows = 8;                              // value rows in flight
        for (int c0 = 0; c0 < n; c0 += kRows) {
            float v[kRows][kPer];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int c = c0 + r;
                const __half* vr = Vh + static_cast<size_t>(j0 + (c < n ? c : n - 1)) * D;
                if (DC == 128 || (!DC && per == 4)) {
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vr + 4 * lane));
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 bq = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    v[r][0] = a.x; v[r][1] = a.y; v[r][2] = bq.x; v[r][3] = bq.y;
                } else if (DC == 64 || (!DC && per == 2)) {
                    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(vr + 2 * lane));
                    v[r][0] = a.x; v[r][1] = a.y;
                } else {
#pragma unroll
                    for (int t = 0; t < kPer; ++t) {
                        const int d = elem(t);
                        v[r][t] = (d < D && (per == 0 || t < per)) ? __half2float(vr[d]) : 0.f;
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int c = c0 + r;
                if (c >= n) break;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pc = __shfl_sync(0xffffffffu, pj[g], c);
#pragma unroll
                    for (int t = 0; t < kPer; ++t) o[g][t] = fmaf(pc, v[r][t], o[g][t]);
                }
            }
        }
    }
    // merge the CTA's warps
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
#pragma unroll
        for (int t = 0; t < kPer; ++t) {
            const int d = elem(t);
            if (d < D && (per == 0 || t < per)) o_s[warp][g][d] = o[g][t];
        }
    }
    __syncthreads();
    for (int t = tid; t < G * D; t += blockDim.x) {
        const int g = t / D, d = t - g * D;
        float mm = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w][g]);
        float ll = 0.f, acc = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) {
            if (m_s[w][g] > -INFINITY) {
                const float e = __expf(m_s[w][g] - mm);
                ll += l_s[w][g] * e;
                acc += o_s[w][g][d] * e;
            }
        }
        const size_t row = (static_cast<size_t>(b) * p.Hq + h0 + g) * p.Sq + i;
        if (p.chunks == 1) {
            p.O[row * D + d] = __float2half_rn(ll != 0.f ? acc / ll : 0.f);
            if (d == 0 && p.LSE) p.LSE[row] = mm + logf(fmaxf(ll, 1e-30f));
        } else {
            float* dst = p.part + (row * p.chunks + chunk) * (D + 2);
            dst[2 + d] = acc;
            if (d == 0) { dst[0] = mm; dst[1] = ll; }
        }
    }
}

// Fast kernel for head_dim 128: every load is a coalesced 512-byte piece of the cache.
//
// K (and V) of a head are contiguous [Sk][128] fp16: 32 keys are 8 KB, which a warp reads with
// 16 instructions of 32 x 16 bytes.  Instruction c brings keys 2c (lanes 0-15) and 2c + 1 (lanes
// 16-31); a lane holds eight consecutive elements of its key - always elements 8 * (lane % 16)
// .. + 7, so its slice of every query row sits in registers.  A key's score is the sum of its 16
// lanes' partial dot products (four shuffles, after which all 16 lanes know it), so the half-warp
// that loads value row 2c (+1) already has that key's probability: no broadcast.  A lane
// accumulates its eight output elements over the keys of its half; the two halves are added at
// the end.  G query heads that share the K/V head are processed together (G <= 4).
// The kernel is bound by how many warps an SM keeps in flight (a step is a chain of round trips and
// shuffles), so the one- and two-head instances are held to 96 / 128 registers for five / four CTAs
// per SM at the price of a few spilled words (32 heads x 4096 keys: 36.9 -> 30.8 us; batch 8 x 2048
// keys: 99.5 -> 83.9 us); the four-head instance was slower that way (233 registers, two CTAs).
template <int G>
__global__ void __launch_bounds__(kAttnWarps * 32, G == 1 ? 5 : (G == 2 ? 4 : 1)) attention_decode128_kernel(const AttnParams p) {
    asm volatile("griddepcontrol.launch_dependents;");
    constexpr int D = 128;
    __shared__ float o_s[kAttnWarps][G][D];
    __shared__ float m_s[kAttnWarps][G], l_s[kAttnWarps][G];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hl = lane & 15, half = lane >> 4;
    const int groups = p.Hq / G;
    const int i = blockIdx.x % p.Sq, bg = blockIdx.x / p.Sq, hg = bg % groups, b = bg / groups;
    const int h0 = hg * G;
    const int hkv = h0 / (p.Hq / p.Hkv);
    const int chunk = blockIdx.y;
    const __half* Kh = p.K + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    const __half* Vh = p.V + (static_cast<size_t>(b) * p.Hkv + hkv) * p.Sk * D;
    float q[G][8], slope[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.Q + ((static_cast<size_t>(b) * p.Hq + h0 + g) * p.Sq + i) * D + 8 * hl);
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float2 f = __half22float2(h2[t]);
            q[g][2 * t] = f.x * p.scale;         // the scale folded into the query
            q[g][2 * t + 1] = f.y * p.scale;
        }
        slope[g] = p.slopes ? p.slopes[h0 + g] : 0.f;
    }
    const int k0 = chunk * p.keys_per_chunk, k1 = min(p.Sk, k0 + p.keys_per_chunk);
    float o[G][8], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int t = 0; t < 8; ++t) o[g][t] = 0.f;
    }
    for (int j0 = k0 + warp * 32; j0 < k1; j0 += kAttnWarps * 32) {
        // scores of the step's 32 keys: s[g][c] belongs to key j0 + 2c + half
        float s[G][16];
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {          // two batches of eight loads: 32 registers of raw keys
            uint4 raw[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int j = j0 + 2 * (8 * hb + c) + half;
                raw[c] = j < k1 ? __ldg(reinterpret_cast<const uint4*>(Kh + static_cast<size_t>(j) * D) + hl)
                                : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw[c]);
                float kf[8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 f = __half22float2(h2[t]);
                    kf[2 * t] = f.x; kf[2 * t + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float acc = 0.f;
#pragma unroll
                    for (int t = 0; t < 8; ++t) acc = fmaf(q[g][t], kf[t], acc);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 8);
                    const int j = j0 + 2 * (8 * hb + c) + half;
                    float sc = acc;
                    if (j >= k1) sc = -INFINITY;
                    if (p.causal && j > i) sc = -INFINITY;
                    if (p.window > 0 && i - j > p.window) sc = -INFINITY;
                    if (p.slopes) sc -= slope[g] * static_cast<float>(i - j);
                    s[g][8 * hb + c] = sc;
                }
            }
        }
        bool any = false;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mx = s[g][0];
#pragma unroll
            for (int c = 1; c < 16; ++c) mx = fmaxf(mx, s[g][c]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));       // the other half's keys
            const float m_new = fmaxf(m[g], mx);
            if (m_new > -INFINITY) {
                const float keep = m[g] > -INFINITY ? __expf(m[g] - m_new) : 0.f;
                float sum = 0.f;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    s[g][c] = s[g][c] > -INFINITY ? __expf(s[g][c] - m_new) : 0.f;    // now the probability
                    sum += s[g][c];
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 16);
                l[g] = l[g] * keep + sum;
#pragma unroll
                for (int t = 0; t < 8; ++t) o[g][t] *= keep;
                m[g] = m_new;
                any = true;
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c) s[g][c] = 0.f;
            }
        }
        if (!any) continue;                                   // warp-uniform
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            uint4 raw[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int j = j0 + 2 * (8 * hb + c) + half;
                raw[c] = j < k1 ? __ldg(reinterpret_cast<const uint4*>(Vh + static_cast<size_t>(j) * D) + hl)
                                : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&raw[c]);
                float vf[8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float2 f = __half22float2(h2[t]);
                    vf[2 * t] = f.x; vf[2 * t + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pc = s[g][8 * hb + c];
#pragma unroll
                    for (int t = 0; t < 8; ++t) o[g][t] = fmaf(pc, vf[t], o[g][t]);
                }
            }
        }
    }
    // the two halves of the warp hold the same output slice over different keys
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int t = 0; t < 8; ++t) o[g][t] += __shfl_xor_sync(0xffffffffu, o[g][t], 16);
        if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
        if (half == 0) {
#pragma unroll
            for (int t = 0; t < 8; ++t) o_s[warp][g][8 * hl + t] = o[g][t];
        }
    }
    __syncthreads();
    for (int t = tid; t < G * D; t += blockDim.x) {
        const int g = t / D, d = t - g * D;
        float mm = -INFINITY;
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w][g]);
        float ll = 0.f, acc = 0.f;
        for (int w = 0; w < kAttnWarps; ++w) {
            if (m_s[w][g] > -INFINITY) {
                const float e = __expf(m_s[w][g] - mm);
                ll += l_s[w][g] * e;
                acc += o_s[w][g][d] * e;
            }
        }
        const size_t row = (static_cast<size_t>(b) * p.Hq + h0 + g) * p.Sq + i;
        if (p.chunks == 1) {
            p.O[row * D + d] = __float2half_rn(ll != 0.f ? acc / ll : 0.f);
            if (d == 0 && p.LSE) p.LSE[row] = mm + logf(fmaxf(ll, 1e-30f));
        } else {
            float* dst = p.part + (row * p.chunks + chunk) * (D + 2);
            dst[2 + d] = acc;
            if (d == 0) { dst[0] = mm; dst[1] = ll; }
        }
    }
}

// Merges the chunks of a row: one CTA per row, a thread per chunk for the weights exp(m_c - m), then
// a thread per output element with the chunks' partial outputs as independent loads.
constexpr int kMergeMaxChunks = 128;
__global__ void __launch_bounds__(128) attention_merge_kernel(const AttnParams p) {
    __shared__ float e_s[kMergeMaxChunks];
    __shared__ float red_s[4];
    const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int D = p.D, chunks = p.chunks;
    // launched with programmatic stream serialisation: the grid that wrote the chunks is complete,
    // and its writes visible, once this returns (without that launch attribute it returns at once)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float* base = p.part + static_cast<size_t>(row) * chunks * (D + 2);
    float mc = -INFINITY, lc = 0.f;
    if (tid < chunks) {
        mc = base[static_cast<size_t>(tid) * (D + 2)];
        lc = base[static_cast<size_t>(tid) * (D + 2) + 1];
    }
    float mm = warp_max(mc);
    if (lane == 0) red_s[warp] = mm;
    __syncthreads();
    mm = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
    const float e = mc > -INFINITY ? __expf(mc - mm) : 0.f;
    if (tid < chunks) e_s[tid] = e;
    float ll = warp_sum(lc * e);
    __syncthreads();                    // red_s has been read by everyone
    if (lane == 0) red_s[warp] = ll;
    __syncthreads();
    ll = (red_s[0] + red_s[1]) + (red_s[2] + red_s[3]);
    for (int d = tid; d < D; d += 128) {
        float acc = 0.f;
#pragma unroll 8
        for (int c = 0; c < chunks; ++c) acc = fmaf(base[static_cast<size_t>(c) * (D + 2) + 2 + d], e_s[c], acc);
        p.O[static_cast<size_t>(row) * D + d] = __float2half_rn(ll != 0.f ? acc / ll : 0.f);
    }
    if (tid == 0 && p.LSE) p.LSE[row] = mm + logf(fmaxf(ll, 1e-30f));
}

template <int DC>
cudaError_t launch_group(int group, dim3 grid, cudaStream_t stream, const AttnParams& p) {
    switch (group) {
        case 1: attention_decode_kernel<DC, 1><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
        case 2: attention_decode_kernel<DC, 2><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
        case 4: attention_decode_kernel<DC, 4><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
        default: return cudaErrorNotSupported;
    }
    return cudaGetLastError();
}

// Query heads one CTA takes together: two of those that share a K/V head (the other pairs of the same
// K/V head run in other CTAs and find the cache in L2).  Four at a time was measured slower (64 heads on
// 8 K/V heads x 8192 keys: 47.3 against 41.3 us): the four-head instance needs 233 registers, two CTAs
// per SM; one at a time re-reads the cache eight times (73.5 us).
int attention_group(int Hq, int Hkv) {
    const int per = Hq / Hkv;
    return per % 2 == 0 ? 2 : 1;
}

}  // namespace

size_t attention_scratch_floats(int B, int Hq, int Hkv, int Sq, int Sk, int D, int sm_count, int* chunks_out) {
    // Enough CTAs for eight per SM, chunks of at least 128 keys (one step of 32 keys per warp): a
    // step is a few dependent round trips to memory, so the bandwidth comes from many warps in
    // flight, not from long chunks.
    const long long ctas = static_cast<long long>(B) * (Hq / attention_group(Hq, Hkv)) * Sq;
    int chunks = static_cast<int>((8LL * sm_count + ctas - 1) / ctas);
    const int most = (Sk + 127) / 128;
    if (chunks > most) chunks = most;
    if (chunks < 1) chunks = 1;
    if (chunks > kMergeMaxChunks) chunks = kMergeMaxChunks;
    if (chunks_out) *chunks_out = chunks;
    const size_t rows = static_cast<size_t>(B) * Hq * Sq;
    return chunks > 1 ? rows * chunks * (D + 2) : 0;
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
    p.group = attention_group(Hq, Hkv);
    int chunks = 1;
    (void)attention_scratch_floats(B, Hq, Hkv, Sq, Sk, D, sm_count, &chunks);
    if (chunks > 1 && !scratch) chunks = 1;
    p.chunks = chunks;
    p.keys_per_chunk = (Sk + chunks - 1) / chunks;
    p.scale = scale; p.causal = causal ? 1 : 0; p.window = window;
    const dim3 grid(static_cast<unsigned>(rows / p.group), static_cast<unsigned>(chunks));
    cudaError_t e;
    const bool aligned = ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V)) & 15u) == 0;
    if (D == 128 && aligned) {
        switch (p.group) {
            case 4: attention_decode128_kernel<4><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
            case 2: attention_decode128_kernel<2><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
            default: attention_decode128_kernel<1><<<grid, kAttnWarps * 32, 0, stream>>>(p); break;
        }
        e = cudaGetLastError();
    } else {
        e = D == 64 ? launch_group<64>(p.group, grid, stream, p) : launch_group<0>(p.group, grid, stream, p);
    }
    if (e != cudaSuccess) return e;
    if (launches) *launches += 1;
    if (chunks > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(rows));
        cfg.blockDim = dim3(128);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, attention_merge_kernel, p);
        if (e == cudaSuccess && launches) *launches += 1;
    }
    return e;
}

}  // namespace tcb
