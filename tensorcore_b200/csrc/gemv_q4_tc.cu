// Batched-decode GEMV for Q4_0 weights on the sm_100a tensor cores (tcgen05, accumulators and the
// weight operand in tensor memory).
//
//   Y[m][n] = sum_k X[m][k] * dequant(W)[n][k],   fp16 X, 5 <= M <= 32 activation rows.
//
// The reference computes this case as M independent dequant-dots per output row, re-reading the
// weights for every activation row (lib/ops/quantized_cpu.cpp:193-228); a GPU pays the weight
// stream M times that way.  Here the weight stream is read once:
//
//   * A CTA owns 256 weight rows and a K range (a cluster of `split` CTAs shares one row tile
//     along K).  Its weight rows arrive in shared memory as raw Q4_0 bytes, one 144-byte group
//     (8 blocks, 256 weights) per row per stage: a single tiled TMA copy of a 256 x 144-byte box
//     (per-row bulk copies of 144 bytes cost ~30 ns each in the copy engine and were 10x slower).
//   * 16 dequantising warps in two sets that alternate stages: one thread per weight row turns a
//     group into fp16 (q - 8) * d - one rounding, |relative error| <= 2^-11 per weight - and
//     stores it with tcgen05.st into its own TMEM lane: the MMA's A operand (128 lanes = 128
//     rows) never touches shared memory.
//   * The same threads stage the activations of their stage as the B operand in shared memory
//     (canonical no-swizzle K-major core matrices, batch padded with zeros to 16 or 32 columns);
//     the global loads for a set's next stage are in flight while it dequantises.
//   * Two threads, one per 128-row half, issue tcgen05.mma (M128 x N16|32 x K16, kind::f16, fp32
//     accumulate) into that half's accumulator of 16|32 TMEM columns.  No per-block fix-up is
//     needed because the scale is already folded into A.
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
// 1e-4 bound of fp32 activations, which therefore never take this path.  The fused RMSNorm form
// reaches this kernel with its rows already normalised and rounded to fp16 by a separate pass
// (one more rounding of the same size, same bound).
#include "kernels.h"
#include "sm100_prims.cuh"
#include "tensor_map.h"

#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>

namespace tcb {
namespace {

using namespace sm100;

constexpr int kTileRows = 256;                 // weight rows per CTA (two 128-lane accumulators)
constexpr int kSets = 2;                       // dequantiser thread sets; set s takes stages s, s+2..
constexpr int kSetThreads = 256;
constexpr int kDqWarps = 8 * kSets;
constexpr int kProducerWarp = kDqWarps;
constexpr int kMmaWarp = kDqWarps + 1;
constexpr int kTcThreads = (kDqWarps + 3) * 32;   // + producer + one MMA issuer per half
constexpr int kRawStages = 4;
constexpr int kXStages = 3;
constexpr int kASlots = 3;                     // per accumulator half; 64 TMEM columns each
constexpr int kGroupBytes = 144;               // 8 Q4_0 blocks
constexpr int kRawStageBytes = kTileRows * kGroupBytes;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColA = 64;                 // accumulators live in columns [0, 64)
constexpr int kMaxBatch = 32;
constexpr int kXPer = kMaxBatch * 32 / kSetThreads;   // activation chunks per thread per stage

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
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t bits) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(bits));
    return r;
}
__device__ __forceinline__ void unpack_word(uint32_t w, __half2 d2, uint32_t* out) {
    const uint32_t ws = w >> 8;
    const __half2 c_lo = bits_h2(0x64086408u);   // 1032
    const __half2 c_hi = bits_h2(0x54805480u);   // 72
    const uint32_t r0 = and_or(w, 0x000F000Fu, 0x64006400u);
    const uint32_t r1 = and_or(w, 0x00F000F0u, 0x54005400u);
    const uint32_t r2 = and_or(ws, 0x000F000Fu, 0x64006400u);
    const uint32_t r3 = and_or(ws, 0x00F000F0u, 0x54005400u);
    out[0] = h2_bits(__hmul2(__hsub2(bits_h2(r0), c_lo), d2));
    out[1] = h2_bits(__hmul2(__hsub2(bits_h2(r1), c_hi), d2));
    out[2] = h2_bits(__hmul2(__hsub2(bits_h2(r2), c_lo), d2));
    out[3] = h2_bits(__hmul2(__hsub2(bits_h2(r3), c_hi), d2));
}

// Block B (0..7) of a 144-byte group, of which the caller holds words W0 .. W0+19: 16 packed
// fp16 pairs.  Block B starts at byte 18*B: its scale sits in the low or high half of a word and
// its quants are word-aligned (odd B) or straddle words by two bytes (even B).
template <int B, int W0>
__device__ __forceinline__ void dequant_block(const uint32_t (&g)[20], uint32_t (&out)[16]) {
    constexpr int w0 = (18 * B) / 4 - W0;
    static_assert(w0 >= 0 && w0 + 5 <= 20, "block outside the held words");
    const uint32_t dd = __byte_perm(g[w0], 0, (B & 1) == 0 ? 0x1010 : 0x3232);
    const __half2 d2 = bits_h2(dd);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        uint32_t w;
        if constexpr ((B & 1) == 0) {
            w = __byte_perm(g[w0 + t], g[w0 + t + 1], 0x5432);
        } else {
            w = g[w0 + 1 + t];
        }
        unpack_word(w, d2, &out[4 * t]);
    }
}

// Activation chunk loads of one stage for one thread: chunk c = tl + 256 * u covers activation
// row n = 8 * u + (tl & 7) and the 8 K values {k0..k0+3, k0+16..k0+19}, k0 from kc = tl >> 3.
struct XRegs {
    uint2 a[kXPer], b[kXPer];
};
__device__ __forceinline__ void x_load(const TcParams& p, int group, int tl, int nb, XRegs& r) {
    const int n_lo = tl & 7, kc = tl >> 3;
    const __half* base = p.X + static_cast<size_t>(group) * 256 + (kc >> 2) * 32 + (kc & 3) * 4;
#pragma unroll
    for (int u = 0; u < kXPer; ++u) {
        const int n = u * 8 + n_lo;
        r.a[u] = make_uint2(0u, 0u);
        r.b[u] = make_uint2(0u, 0u);
        if (u * 8 < nb && n < p.M) {
            const __half* xr = base + static_cast<size_t>(n) * p.K;
            r.a[u] = *reinterpret_cast<const uint2*>(xr);        // k0 .. k0+3
            r.b[u] = *reinterpret_cast<const uint2*>(xr + 16);   // k0+16 .. k0+19
        }
    }
}
// Writes the chunks in the dequantiser's K order as no-swizzle K-major core matrices:
// chunk (n, kc) at kc * lbo + (n / 8) * 128 + (n % 8) * 16.
__device__ __forceinline__ void x_store(uint32_t dst0, uint32_t lbo, int tl, int nb, const XRegs& r) {
    const int n_lo = tl & 7, kc = tl >> 3;
    const uint32_t dst = dst0 + static_cast<uint32_t>(kc) * lbo + n_lo * 16;
#pragma unroll
    for (int u = 0; u < kXPer; ++u) {
        if (u * 8 >= nb) break;
        uint4 v;
        v.x = __byte_perm(r.a[u].x, r.a[u].y, 0x5410);   // (k0,   k0+2)
        v.y = __byte_perm(r.b[u].x, r.b[u].y, 0x5410);   // (k0+16, k0+18)
        v.z = __byte_perm(r.a[u].x, r.a[u].y, 0x7632);   // (k0+1, k0+3)
        v.w = __byte_perm(r.b[u].x, r.b[u].y, 0x7632);   // (k0+17, k0+19)
        sts128(dst + u * 128, v);
    }
}

__global__ void __launch_bounds__(kTcThreads, 1)
gemv_q4_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap wmap) {
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
    const int nb = p.nbatch;
    const uint32_t lbo = static_cast<uint32_t>(nb) * 16u;        // bytes between K core matrices
    const uint32_t x_stage_bytes = static_cast<uint32_t>(nb) * 512u;
    const uint32_t raw_base = s_u32(smem + p.off_raw);
    const uint32_t x_base = s_u32(smem + p.off_x);

    // The next kernel on the stream may start its own prologue and weight copies now; what it
    // reads of this kernel's output it reads behind its own dependency wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == kProducerWarp * 32) prefetch_tensormap(&wmap);
    if (tid == 0) {
        for (int i = 0; i < kRawStages; ++i) {
            bar_init(&bars->raw_full[i], 1);
            bar_init(&bars->raw_empty[i], 8);       // the 8 warps of the set that read the stage
        }
        for (int i = 0; i < kXStages; ++i) {
            bar_init(&bars->x_full[i], 8);          // the 8 warps of the set that staged it
            bar_init(&bars->x_empty[i], 2);         // one commit per MMA issuer
        }
        for (int h = 0; h < 2; ++h)
            for (int i = 0; i < kASlots; ++i) {
                bar_init(&bars->a_full[h][i], 128); // every thread that owns one of this half's lanes
                bar_init(&bars->a_empty[h][i], 1);
            }
        bar_init(&bars->d_full, 2);
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    if (warp < 8) {
        // Zero both accumulators: warp w owns lanes 32 * (w % 4) of accumulator w / 4.
        uint32_t z[16] = {};
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>((warp >> 2) * kMaxBatch);
        tmem_st16(taddr, z);
        tmem_st16(taddr + 16, z);
        tmem_wait_st();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    bool failed = false;

    if (warp < kDqWarps) {
        // ---------------- dequantisers: one thread per weight row; they also stage activations ----
        const int set = warp >> 3, wl = warp & 7, h = wl >> 2, q = wl & 3;
        const int tl = tid & (kSetThreads - 1);
        const int row_local = h * 128 + q * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        Ring raw, slot, xs;
        raw.set(set, kRawStages);
        xs.set(set, kXStages);
        slot.set(2 * set, kASlots);
        XRegs xr;
        // Activations and outputs belong to the stream's order: wait for the kernel before this one
        // here, with the weight copies (which no kernel of a decode step writes) already in flight.
        // These warps also write the outputs.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (set < ng) x_load(p, g0 + set, tl, nb, xr);
        for (int i = set; i < ng && !failed; i += kSets) {
            // Activations of this stage: loaded a stage ago, now permuted into shared memory.
            if (!bar_wait_warp(&bars->x_empty[xs.idx], xs.phase ^ 1u, abort_flag)) { failed = true; break; }
            x_store(x_base + xs.idx * x_stage_bytes, lbo, tl, nb, xr);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) bar_arrive(&bars->x_full[xs.idx]);
            if (i + kSets < ng) x_load(p, g0 + i + kSets, tl, nb, xr);

            if (!bar_wait_warp(&bars->raw_full[raw.idx], raw.phase, abort_flag)) { failed = true; break; }
            const uint32_t src = raw_base + raw.idx * kRawStageBytes + row_local * kGroupBytes;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (failed) break;
                // Blocks 0-3 live in bytes [0,72) of the group, blocks 4-7 in [72,144): five
                // 16-byte loads from byte 0 or byte 64 cover either half.
                uint32_t g[20];
#pragma unroll
                for (int v = 0; v < 5; ++v) {
                    const uint4 t4 = lds128(src + 64 * half + 16 * v);
                    g[4 * v] = t4.x; g[4 * v + 1] = t4.y; g[4 * v + 2] = t4.z; g[4 * v + 3] = t4.w;
                }
                if (!bar_wait_warp(&bars->a_empty[h][slot.idx], slot.phase ^ 1u, abort_flag)) {
                    failed = true;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t col = lane_base + kColA + static_cast<uint32_t>((h * kASlots + slot.idx) * 64);
                uint32_t out[16];
                if (half == 0) {
                    dequant_block<0, 0>(g, out); tmem_st16(col, out);
                    dequant_block<1, 0>(g, out); tmem_st16(col + 16, out);
                    dequant_block<2, 0>(g, out); tmem_st16(col + 32, out);
                    dequant_block<3, 0>(g, out); tmem_st16(col + 48, out);
                } else {
                    dequant_block<4, 16>(g, out); tmem_st16(col, out);
                    dequant_block<5, 16>(g, out); tmem_st16(col + 16, out);
                    dequant_block<6, 16>(g, out); tmem_st16(col + 32, out);
                    dequant_block<7, 16>(g, out); tmem_st16(col + 48, out);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                bar_arrive(&bars->a_full[h][slot.idx]);
                if (half == 1) {
                    // The raw stage is released only here, after every value loaded from it has
                    // been consumed by a tcgen05.st that has completed.  Releasing it right after
                    // the loads were issued let the next tiled copy overwrite rows whose loads the
                    // scheduler had deferred (seen as a block holding the data of 4 stages later).
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) bar_arrive(&bars->raw_empty[raw.idx]);
                }
                slot.advance(half == 0 ? 1 : 2 * kSets - 1, kASlots);
            }
            raw.advance(kSets, kRawStages);
            xs.advance(kSets, kXStages);
        }
    } else if (warp == kProducerWarp) {
        // ---------------- weight producer: one 256-row x 144-byte box per stage ------------------
        // The weights are a 2-D byte tensor [N][K/32*18]; rows past N read as zeros.
        Ring raw;
        raw.set(0, kRawStages);
        int issued = 0;
        if (lane == 0) {
            for (int i = 0; i < ng; ++i) {
                if (!bar_wait(&bars->raw_empty[raw.idx], raw.phase ^ 1u, abort_flag)) { failed = true; break; }
                bar_expect_tx(&bars->raw_full[raw.idx], kRawStageBytes);
                tensor_load_2d(smem + p.off_raw + raw.idx * kRawStageBytes, &wmap,
                               (g0 + i) * kGroupBytes, row0, &bars->raw_full[raw.idx]);
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
        }
    } else {
        // ---------------- MMA issue: one thread per accumulator half -------------------------------
        // The MMAs are tiny (M128 x N<=32 x K16) and the issuing thread is on the critical path, so
        // each half has its own issuer on its own scheduler, all operands are computed before the
        // wait, and every MMA accumulates (the accumulators were zeroed at start-up).
        if (lane == 0) {
            const int h = warp - kMmaWarp;
            const uint32_t idesc = idesc_f16_f32(128, nb);
            const uint32_t desc_step = (2u * lbo) >> 4;
            const uint32_t d_col = tmem_base + static_cast<uint32_t>(h * kMaxBatch);
            Ring xs, slot;
            xs.set(0, kXStages);
            slot.set(0, kASlots);
            for (int i = 0; i < ng && !failed; ++i) {
                // Descriptor of the stage's first K step; each further step starts 2 * lbo bytes on.
                const uint64_t desc0 = smem_desc_kmajor(x_base + xs.idx * x_stage_bytes, lbo, 128u);
                if (!bar_wait(&bars->x_full[xs.idx], xs.phase, abort_flag)) { failed = true; break; }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t a_col = tmem_base + kColA + static_cast<uint32_t>((h * kASlots + slot.idx) * 64);
                    uint64_t bdesc[8];
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) bdesc[jj] = desc0 + static_cast<uint64_t>((half * 8 + jj) * desc_step);
                    if (!bar_wait(&bars->a_full[h][slot.idx], slot.phase, abort_flag)) { failed = true; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) mma_f16_ts_acc(d_col, a_col + 8u * jj, bdesc[jj], idesc);
                    mma_commit(&bars->a_empty[h][slot.idx]);
                    slot.advance(1, kASlots);
                }
                if (!failed) mma_commit(&bars->x_empty[xs.idx]);
                xs.advance(1, kXStages);
            }
            mma_commit(&bars->d_full);
            if (failed || *abort_flag) bar_wait(&bars->d_full, 0, nullptr, 100000000LL);
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
        const bool ok = bar_wait_warp(&bars->d_full, 0, abort_flag) && __all_sync(0xffffffffu, !*abort_flag);
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

// How many clusters of `size` CTAs of this kernel the device can hold at once; cached per size
// and shared-memory footprint (the two batch widths).  0 when the query fails.
int max_active_clusters(int size, int smem) {
    static int cache[2][9] = {};
    static bool known[2][9] = {};
    const int w = smem > kBarrierBytes + kRawStages * kRawStageBytes + kXStages * 16 * 512 ? 1 : 0;
    if (!known[w][size]) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(size * 64);
        cfg.blockDim = dim3(kTcThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemv_q4_tc_kernel, &cfg) != cudaSuccess) {
            n = 0;
            (void)cudaGetLastError();
        }
        cache[w][size] = n;
        known[w][size] = true;
    }
    return cache[w][size];
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
    p.off_raw = kBarrierBytes;
    p.off_x = p.off_raw + kRawStages * kRawStageBytes;
    const int smem = p.off_x + kXStages * p.nbatch * 512;
    if (smem > env.smem_optin) return cudaErrorNotSupported;
    // K is split over a cluster when there are fewer row tiles than SMs: the largest cluster size
    // whose clusters can all be resident at once (one wave), so that the split shortens the
    // per-CTA K loop instead of queueing clusters.
    int split = 1;
    for (int s = 8; s > 1; --s) {
        if (s > p.groups || tiles * s > env.sm_count) continue;
        if (tiles <= max_active_clusters(s, smem)) { split = s; break; }
    }
    if (const char* s = std::getenv("TC_TC_SPLIT")) split = std::atoi(s);
    if (split > 8) split = 8;
    if (split > p.groups) split = p.groups;
    if (split < 1) split = 1;
    p.split = split;

    CUtensorMap wmap;
    // The weights as a 2-D byte tensor: dimension 0 = the bytes of a row, box = one 8-block group
    // (144 bytes) of 256 rows.
    if (!encode_bytes_2d(&wmap, a.W, a.N, static_cast<size_t>(p.groups) * kGroupBytes, kGroupBytes, kTileRows))
        return cudaErrorNotSupported;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * split);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (env.pdl) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    if (name) *name = "q4_0_gemv_tcgen05_sm100";
    return cudaLaunchKernelEx(&cfg, gemv_q4_tc_kernel, p, wmap);
}

}  // namespace tcb
