// Batched-decode GEMV for Q4_0 weights on the sm_100a tensor cores (tcgen05, accumulators and the
// weight operand in tensor memory).
//
//   Y[m][n] = sum_k X[m][k] * dequant(W)[n][k],   fp16 X, 5 <= M <= 32 activation rows.
//
// The reference computes this case as M independent dequant-dots per output row
// (lib/ops/quantized/gemv_dispatch.cpp:52-90 with the kernels of metal_quant_kernels.h); a GPU
// pays the weight stream M times that way.  Here the weight stream is read once:
//
//   * A CTA owns 256 weight rows and a K range (a cluster of `split` CTAs shares one row tile
//     along K).  Its weight rows arrive in shared memory as raw Q4_0 bytes, one 144-byte group
//     (8 blocks, 256 weights) per row per stage, by bulk copies.
//   * 16 dequantising warps: one thread per weight row turns a group into fp16
//     (q - 8) * d - one rounding, |relative error| <= 2^-11 per weight - and stores it with
//     tcgen05.st into its own TMEM lane: the MMA's A operand (128 lanes = 128 rows) never
//     touches shared memory.
//   * 2 warps stage the activations for the same K range as the B operand in shared memory
//     (canonical no-swizzle K-major core matrices), batch padded with zeros to 16 or 32 columns.
//   * One thread issues tcgen05.mma (M128 x N16|32 x K16, kind::f16, fp32 accumulate); there are
//     two accumulators (rows 0-127 and 128-255) of 16|32 TMEM columns each.  No per-block
//     fix-up is needed because the scale is already folded into A.
//   * Epilogue: tcgen05.ld, then either a direct store or, when K is split, a deterministic
//     reduction over the cluster through distributed shared memory.
//
// Within a 32-weight block the dequantiser emits K in the order that is cheapest to unpack
// (see `unpack_word`), and the activation stager applies the same permutation, so the MMA sees
// matching K indices on both operands.
//
// Accuracy: products are exact in fp32 inside the MMA, accumulation is fp32; the only extra
// rounding against the reference's fp32 dequant-dot is the fp16 rounding of (q-8)*d, a scaled
// RMS error of about 2e-4 - inside the 2e-3 bound that applies to fp16 activations, outside the
// 1e-4 bound of fp32 activations, which therefore never take this path.
#include "kernels.h"
#include "sm100_prims.cuh"

#include <cuda_fp16.h>

#include <cstdlib>

namespace tcb {
namespace {

using namespace sm100;

constexpr int kTileRows = 256;                 // weight rows per CTA (two 128-lane accumulators)
constexpr int kSets = 2;                       // dequantiser thread sets; set s takes stages s, s+2..
constexpr int kDqWarps = 8 * kSets;
constexpr int kProducerWarp = kDqWarps;
constexpr int kMmaWarp = kDqWarps + 1;
constexpr int kXWarp0 = kDqWarps + 2;
constexpr int kXWarps = 2;
constexpr int kTcThreads = (kDqWarps + 2 + kXWarps) * 32;
constexpr int kRawStages = 3;
constexpr int kXStages = 3;
constexpr int kASlots = 3;                     // per accumulator half; 64 TMEM columns each
constexpr int kGroupBytes = 144;               // 8 Q4_0 blocks
constexpr int kRawStageBytes = kTileRows * kGroupBytes;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColA = 64;                 // accumulators live in columns [0, 64)
constexpr int kMaxBatch = 32;

struct TcParams {
    const uint8_t* W;
    const __half* X;
    void* Y;
    uint32_t* err;
    int M, N, K;
    int y_f32;
    int nbatch;      // MMA N extent: 16 or 32
    int groups;      // K / 256
    int split;       // CTAs per row tile = cluster size
    int off_raw, off_x;
};

struct Ring {
    int idx;
    uint32_t phase;
    __device__ __forceinline__ void set(int pos, int size) {
        idx = pos % size;
        phase = static_cast<uint32_t>(pos / size) & 1u;
    }
    __device__ __forceinline__ void advance(int n, int size) {
        idx += n;
        while (idx >= size) { idx -= size; phase ^= 1u; }
    }
};

// Barrier block at the start of dynamic shared memory.
struct Barriers {
    uint64_t raw_full[kRawStages];
    uint64_t raw_empty[kRawStages];
    uint64_t x_full[kXStages];
    uint64_t x_empty[kXStages];
    uint64_t a_full[2][kASlots];
    uint64_t a_empty[2][kASlots];
    uint64_t d_full;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int kBarrierBytes = 512;
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// Four bytes of quants (k = 4t .. 4t+3 in the low nibbles, k = 16+4t .. in the high nibbles)
// become four fp16 pairs, already scaled:
//   out[0] = (k0, k0+2)   out[1] = (k0+16, k0+18)   out[2] = (k0+1, k0+3)   out[3] = (k0+17, k0+19)
// A nibble ORed into the mantissa of 1024.0 (bits 0-3) or of 64.0 (bits 4-7) is that constant
// plus the nibble exactly; subtracting 1032 or 72 leaves q - 8.
__device__ __forceinline__ void unpack_word(uint32_t w, __half2 d2, uint32_t* out) {
    const uint32_t ws = w >> 8;
    const __half2 c_lo = bits_h2(0x64086408u);   // 1032
    const __half2 c_hi = bits_h2(0x54805480u);   // 72
    const uint32_t r0 = (w & 0x000F000Fu) | 0x64006400u;
    const uint32_t r1 = (w & 0x00F000F0u) | 0x54005400u;
    const uint32_t r2 = (ws & 0x000F000Fu) | 0x64006400u;
    const uint32_t r3 = (ws & 0x00F000F0u) | 0x54005400u;
    out[0] = h2_bits(__hmul2(__hsub2(bits_h2(r0), c_lo), d2));
    out[1] = h2_bits(__hmul2(__hsub2(bits_h2(r1), c_hi), d2));
    out[2] = h2_bits(__hmul2(__hsub2(bits_h2(r2), c_lo), d2));
    out[3] = h2_bits(__hmul2(__hsub2(bits_h2(r3), c_hi), d2));
}

// Block B (0..7) of a 144-byte group held as 36 words: 16 packed fp16 pairs.
template <int B>
__device__ __forceinline__ void dequant_block(const uint32_t (&g)[36], uint32_t (&out)[16]) {
    constexpr int byte0 = 18 * B;
    constexpr int w0 = byte0 / 4;
    uint32_t dd;
    if constexpr ((B & 1) == 0) {
        dd = __byte_perm(g[w0], 0, 0x1010);       // scale in the low half of word w0
    } else {
        dd = __byte_perm(g[w0], 0, 0x3232);       // scale in the high half
    }
    const __half2 d2 = bits_h2(dd);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        uint32_t w;
        if constexpr ((B & 1) == 0) {
            w = __byte_perm(g[w0 + t], g[w0 + t + 1], 0x5432);  // quants start 2 bytes into w0
        } else {
            w = g[w0 + 1 + t];
        }
        unpack_word(w, d2, &out[4 * t]);
    }
}

__global__ void __launch_bounds__(kTcThreads, 1) gemv_q4_tc_kernel(const TcParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    Barriers* bars = reinterpret_cast<Barriers*>(smem);
    volatile int* abort_flag = &bars->abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int split = p.split;
    const int tile = blockIdx.x / split;
    const int crank = static_cast<int>(cluster_ctarank());
    const int g0 = p.groups * crank / split;
    const int g1 = p.groups * (crank + 1) / split;
    const int ng = g1 - g0;
    const int row0 = tile * kTileRows;
    const int valid_rows = min(kTileRows, p.N - row0);
    const int nb = p.nbatch;
    const uint32_t lbo = static_cast<uint32_t>(nb) * 16u;        // bytes between K core matrices
    const uint32_t x_stage_bytes = static_cast<uint32_t>(nb) * 512u;
    const uint32_t raw_base = s_u32(smem + p.off_raw);
    const uint32_t x_base = s_u32(smem + p.off_x);

    if (tid == 0) {
        for (int i = 0; i < kRawStages; ++i) {
            bar_init(&bars->raw_full[i], 1);
            bar_init(&bars->raw_empty[i], 8);       // the 8 warps of the set that read the stage
        }
        for (int i = 0; i < kXStages; ++i) {
            bar_init(&bars->x_full[i], kXWarps);
            bar_init(&bars->x_empty[i], 1);
        }
        for (int h = 0; h < 2; ++h)
            for (int i = 0; i < kASlots; ++i) {
                bar_init(&bars->a_full[h][i], 4);   // the 4 warps that own this half's lanes
                bar_init(&bars->a_empty[h][i], 1);
            }
        bar_init(&bars->d_full, 1);
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;

    bool failed = false;

    if (warp < kDqWarps) {
        // ---------------- dequantisers: one thread per weight row --------------------------------
        const int set = warp >> 3, wl = warp & 7, h = wl >> 2, q = wl & 3;
        const int row_local = h * 128 + q * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        Ring raw, slot;
        raw.set(set, kRawStages);
        slot.set(2 * set, kASlots);
        for (int i = set; i < ng && !failed; i += kSets) {
            if (!bar_wait(&bars->raw_full[raw.idx], raw.phase, abort_flag)) { failed = true; break; }
            const uint32_t src = raw_base + raw.idx * kRawStageBytes + row_local * kGroupBytes;
            uint32_t g[36];
#pragma unroll
            for (int v = 0; v < 9; ++v) {
                const uint4 t4 = lds128(src + 16 * v);
                g[4 * v] = t4.x; g[4 * v + 1] = t4.y; g[4 * v + 2] = t4.z; g[4 * v + 3] = t4.w;
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&bars->raw_empty[raw.idx]);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (failed) break;
                if (!bar_wait(&bars->a_empty[h][slot.idx], slot.phase ^ 1u, abort_flag)) {
                    failed = true;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t col = lane_base + kColA + static_cast<uint32_t>((h * kASlots + slot.idx) * 64);
                uint32_t out[16];
                if (half == 0) {
                    dequant_block<0>(g, out); tmem_st16(col, out);
                    dequant_block<1>(g, out); tmem_st16(col + 16, out);
                    dequant_block<2>(g, out); tmem_st16(col + 32, out);
                    dequant_block<3>(g, out); tmem_st16(col + 48, out);
                } else {
                    dequant_block<4>(g, out); tmem_st16(col, out);
                    dequant_block<5>(g, out); tmem_st16(col + 16, out);
                    dequant_block<6>(g, out); tmem_st16(col + 32, out);
                    dequant_block<7>(g, out); tmem_st16(col + 48, out);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) bar_arrive(&bars->a_full[h][slot.idx]);
                slot.advance(half == 0 ? 1 : 2 * kSets - 1, kASlots);
            }
            raw.advance(kSets, kRawStages);
        }
    } else if (warp == kProducerWarp) {
        // ---------------- weight producer: 144 bytes per row per stage ---------------------------
        const size_t row_bytes = static_cast<size_t>(p.groups) * kGroupBytes;
        const uint8_t* wbase = p.W + static_cast<size_t>(row0) * row_bytes + static_cast<size_t>(g0) * kGroupBytes;
        Ring raw;
        raw.set(0, kRawStages);
        int issued = 0;
        for (int i = 0; i < ng; ++i) {
            if (!bar_wait(&bars->raw_empty[raw.idx], raw.phase ^ 1u, abort_flag)) { failed = true; break; }
            if (lane == 0) bar_expect_tx(&bars->raw_full[raw.idx], static_cast<uint32_t>(valid_rows) * kGroupBytes);
            __syncwarp();
            uint8_t* dst = smem + p.off_raw + raw.idx * kRawStageBytes;
            for (int r = lane; r < valid_rows; r += 32)
                bulk_load(dst + r * kGroupBytes, wbase + r * row_bytes + static_cast<size_t>(i) * kGroupBytes,
                          kGroupBytes, &bars->raw_full[raw.idx]);
            ++issued;
            raw.advance(1, kRawStages);
        }
        if (failed || *abort_flag) {
            // Let copies already in flight land before the CTA's shared memory is released.
            const int first = issued > kRawStages ? issued - kRawStages : 0;
            for (int s = first; s < issued; ++s) {
                Ring r;
                r.set(s, kRawStages);
                bar_wait(&bars->raw_full[r.idx], r.phase, nullptr, 100000000LL);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issue ----------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_f16_f32(128, nb);
            Ring xs, slot;
            xs.set(0, kXStages);
            slot.set(0, kASlots);
            for (int i = 0; i < ng && !failed; ++i) {
                if (!bar_wait(&bars->x_full[xs.idx], xs.phase, abort_flag)) { failed = true; break; }
                const uint32_t xs_addr = x_base + xs.idx * x_stage_bytes;
                for (int half = 0; half < 2 && !failed; ++half) {
                    for (int h = 0; h < 2; ++h) {
                        if (!bar_wait(&bars->a_full[h][slot.idx], slot.phase, abort_flag)) { failed = true; break; }
                        tc_fence_after_sync();
                        const uint32_t a_col = tmem_base + kColA + static_cast<uint32_t>((h * kASlots + slot.idx) * 64);
                        const uint32_t d_col = tmem_base + static_cast<uint32_t>(h * kMaxBatch);
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) {
                            const int kstep = half * 8 + jj;
                            const uint64_t bdesc = smem_desc_kmajor(xs_addr + 2u * kstep * lbo, lbo, 128u);
                            mma_f16_ts(d_col, a_col + 8u * jj, bdesc, idesc, (i | half | jj) != 0 ? 1u : 0u);
                        }
                        mma_commit(&bars->a_empty[h][slot.idx]);
                    }
                    slot.advance(1, kASlots);
                }
                if (!failed) mma_commit(&bars->x_empty[xs.idx]);
                xs.advance(1, kXStages);
            }
            mma_commit(&bars->d_full);
            if (failed || *abort_flag) bar_wait(&bars->d_full, 0, nullptr, 100000000LL);
        }
    } else {
        // ---------------- activation stager ----------------------------------------------------------
        const int tx = tid - kXWarp0 * 32;
        const int chunks = 32 * nb;   // 16-byte chunks per stage
        Ring xs;
        xs.set(0, kXStages);
        for (int i = 0; i < ng; ++i) {
            if (!bar_wait(&bars->x_empty[xs.idx], xs.phase ^ 1u, abort_flag)) { failed = true; break; }
            const uint32_t dst0 = x_base + xs.idx * x_stage_bytes;
            const size_t kg = static_cast<size_t>(g0 + i) * 256;
            for (int c = tx; c < chunks; c += kXWarps * 32) {
                const int n_lo = c & 7, kc = (c >> 3) & 31, n_hi = c >> 8;
                const int n = n_hi * 8 + n_lo;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (n < p.M) {
                    const __half* xr = p.X + static_cast<size_t>(n) * p.K + kg + (kc >> 2) * 32 + (kc & 3) * 4;
                    const uint2 a = *reinterpret_cast<const uint2*>(xr);        // k0 .. k0+3
                    const uint2 b = *reinterpret_cast<const uint2*>(xr + 16);   // k0+16 .. k0+19
                    v.x = __byte_perm(a.x, a.y, 0x5410);   // (k0,   k0+2)
                    v.y = __byte_perm(b.x, b.y, 0x5410);   // (k0+16, k0+18)
                    v.z = __byte_perm(a.x, a.y, 0x7632);   // (k0+1, k0+3)
                    v.w = __byte_perm(b.x, b.y, 0x7632);   // (k0+17, k0+19)
                }
                sts128(dst0 + static_cast<uint32_t>(kc) * lbo + n_hi * 128 + n_lo * 16, v);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) bar_arrive(&bars->x_full[xs.idx]);
            xs.advance(1, kXStages);
        }
    }

    if (failed) {
        *abort_flag = 1;
        if (p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
    }
    __syncwarp();

    // ---------------- epilogue: set 0's warps read the accumulators ---------------------------------
    float* red = reinterpret_cast<float*>(smem + p.off_raw);   // [nbatch][256], split-K partials
    if (warp < 8) {
        const int h = warp >> 2, q = warp & 3;
        const int row_local = h * 128 + q * 32 + lane;
        const bool ok = bar_wait(&bars->d_full, 0, abort_flag) && !*abort_flag;
        if (!ok && !*abort_flag) {
            *abort_flag = 1;
            if (p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
        }
        tc_fence_after_sync();
        if (ok) {
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(h * kMaxBatch);
            const int row = row0 + row_local;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u * 16 >= nb) break;
                uint32_t v[16];
                tmem_ld16(taddr + 16u * u, v);
                tmem_wait_ld();
                if (split == 1) {
                    if (row < p.N) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int m = u * 16 + e;
                            if (m < p.M) {
                                const float f = __uint_as_float(v[e]);
                                if (p.y_f32) static_cast<float*>(p.Y)[static_cast<size_t>(m) * p.N + row] = f;
                                else static_cast<__half*>(p.Y)[static_cast<size_t>(m) * p.N + row] = __float2half_rn(f);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        red[(u * 16 + e) * kTileRows + row_local] = __uint_as_float(v[e]);
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();

    if (split > 1) {
        cluster_sync_all();
        if (!*abort_flag) {
            const int r_lo = kTileRows * crank / split, r_hi = kTileRows * (crank + 1) / split;
            const int rows_c = r_hi - r_lo;
            const uint32_t red_addr = s_u32(red);
            for (int e = tid; e < p.M * rows_c; e += kTcThreads) {
                const int m = e / rows_c, r = r_lo + e % rows_c;
                const int row = row0 + r;
                if (row >= p.N) continue;
                float acc = 0.f;
                for (int c = 0; c < split; ++c)
                    acc += ld_cluster_f32(red_addr + static_cast<uint32_t>(m * kTileRows + r) * 4u, c);
                if (p.y_f32) static_cast<float*>(p.Y)[static_cast<size_t>(m) * p.N + row] = acc;
                else static_cast<__half*>(p.Y)[static_cast<size_t>(m) * p.N + row] = __float2half_rn(acc);
            }
        }
        cluster_sync_all();   // peers may still be reading this CTA's partials
    }

    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

cudaError_t init_tc_kernels(int smem_optin) {
    return cudaFuncSetAttribute(gemv_q4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                smem_optin);
}

// cudaErrorNotSupported when the operation is outside this kernel's domain.
cudaError_t launch_gemv_q4_tc(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                              const char** name) {
    if (a.fmt != FMT_Q4_0 || a.x_f32 || a.gamma != nullptr) return cudaErrorNotSupported;
    if (a.M < 1 || a.M > kMaxBatch || a.K <= 0 || a.K % 256 != 0 || a.N <= 0) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(a.W) & 15u) || (reinterpret_cast<uintptr_t>(a.X) & 7u))
        return cudaErrorNotSupported;

    TcParams p{};
    p.W = a.W;
    p.X = static_cast<const __half*>(a.X);
    p.Y = a.Y;
    p.err = env.err_word;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.y_f32 = a.y_f32 ? 1 : 0;
    p.nbatch = a.M <= 16 ? 16 : 32;
    p.groups = a.K / 256;
    const int tiles = (a.N + kTileRows - 1) / kTileRows;
    int split = env.sm_count > 0 ? env.sm_count / tiles : 1;
    if (const char* s = std::getenv("TC_TC_SPLIT")) split = std::atoi(s);
    if (split > 8) split = 8;
    if (split > p.groups) split = p.groups;
    if (split < 1) split = 1;
    p.split = split;
    p.off_raw = kBarrierBytes;
    p.off_x = p.off_raw + kRawStages * kRawStageBytes;
    const int smem = p.off_x + kXStages * p.nbatch * 512;
    if (smem > env.smem_optin) return cudaErrorNotSupported;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * split);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (name) *name = "q4_0_gemv_tcgen05_sm100";
    return cudaLaunchKernelEx(&cfg, gemv_q4_tc_kernel, p);
}

}  // namespace tcb
