// Q4_0 GEMV for decode (M = 1 or 2) on sm_100a with the dot products on the warp-level
// tensor-core instruction (mma.sync m16n8k16, fp16 x fp16 -> fp32).
//
// Why tensor cores for a GEMV: the kernel is HBM-bound only if the SM can unpack 4-bit codes
// fast enough.  A CUDA-core dot costs one FMA per weight on top of the unpacking (measured:
// 3.2 issued instructions per weight, issue-bound at ~55 % of HBM rate).  Here the multiply-
// adds leave the instruction stream: a masked code word IS a pair of fp16 operands (a code c in
// the low mantissa bits of a binary16 is the subnormal c * 2^-24, in bits 4..7 it is c * 2^-20),
// so unpacking is 5 integer instructions per 8 weights and nothing else is per-weight.
//
// Mapping.  The 8 columns of the MMA are not batch columns but 8 consecutive blocks of the same
// 16 weight rows: MMA k-slot (2t, 2t+1) carries two codes of block 2t and slot (2t+8, 2t+9) two
// codes of block 2t+1 (t = lane % 4), and the activation operand B[k][n] is non-zero only where
// slot k belongs to block n.  Sixteen MMAs walk the 32 elements of the blocks, after which lane
// (g, t) holds in its four accumulator registers the raw dot products of rows g and g+8 with
// blocks 2t and 2t+1 - exactly the blocks whose bytes (and therefore fp16 scales) it loaded
// itself.  The per-block fix-up (scale, zero point) is then 3 instructions per block per row
// with no redundancy between lanes.
//
// Data movement.  A CTA owns a contiguous range of rows.  It walks them in panels of 16 rows;
// a producer warp streams each panel in chunks of up to 64 blocks per row with one 1-D bulk
// async copy (TMA) per row into a ring of shared-memory stages whose row pitch is padded so that
// the 32 lanes' 32-bit loads (8 rows x 4 block pairs) hit 32 different banks.  Eight consumer
// warps each take one 8-block group of a stage.  Full/empty mbarriers order the ring; every wait
// is bounded and abortable.  With programmatic dependent launch the weight stream starts before
// the previous kernel in the stream has finished; activations are staged after the dependency
// wait, pre-permuted into MMA operand order (and pre-divided by 16 for high-nibble slots).
//
// fp32 activations (and the RMSNorm-fused form, whose normalised row is fp32) run the MMAs twice,
// on the fp16 head and the fp16 remainder of each activation (x = hi + lo to 2^-22 relative).
#include "kernels.h"

#include <cuda_fp16.h>

#include <cstdlib>

namespace tcb {
namespace {

#ifndef TCB_MMA_WARPS
#define TCB_MMA_WARPS 16
#endif
constexpr int kConsumerWarps = TCB_MMA_WARPS;   // one 8-block group of a stage per warp
constexpr int kMaxKc = kConsumerWarps * 8;      // blocks per row per stage
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kMmaThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kPanelRows = 16;
constexpr int kMaxStages = 6;

struct MmaParams {
    const uint8_t* W;
    const void* X;
    void* Y;
    const void* gamma;
    uint32_t* err;
    int M, N, K;
    int nb;            // blocks per row
    int kc;            // blocks per chunk (multiple of 8, <= kMaxKc)
    int chunks;        // chunks per panel = ceil(nb / kc)
    int pitch;         // bytes between rows of a stage
    int ns;            // ring stages
    uint32_t ns_magic; // floor(2^32 / ns) + 1: s / ns == umulhi(s, ns_magic) for small s
    int x_f32;         // activations are fp32 in global memory
    int y_f32;
    int split;         // 1: two-pass hi/lo activations (fp32 x or fused norm)
    float eps;
    int off_red, off_sx, off_zero, off_xfrag, off_ring;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void bar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_u32(bar)),
                 "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(s_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded, abortable wait: false when `*abort_flag` is raised or ~1 s of clocks has passed.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (bar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!bar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) return false;
    }
    return true;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(s_u32(dst)), "l"(src), "r"(bytes), "r"(s_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Shared-memory loads by 32-bit window address (constant offsets fold into the instruction).
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float hbits2f(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<uint16_t>(h16)));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(a))) |
           (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(b))) << 16);
}

__device__ double csum_f64(double v, double* scratch) {  // consumer threads only
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    consumer_sync();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    consumer_sync();
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) t += scratch[i];
    return t;
}

// Operand order of one block's activations.  MMA j = 4*i + v (i = code word 0..3, v = variant)
// multiplies the code pair extracted from word i by variant v:
//   v=0: low nibbles of bytes 4i, 4i+2   -> elements 4i,      4i+2
//   v=1: high nibbles of the same bytes  -> elements 16+4i,   16+4i+2   (codes carry x16)
//   v=2: low nibbles of bytes 4i+1, 4i+3 -> elements 4i+1,    4i+3
//   v=3: high nibbles of those           -> elements 16+4i+1, 16+4i+3   (x16)
__device__ __forceinline__ void frag_elems(int j, int& e0, int& e1, float& sc) {
    const int i = j >> 2, v = j & 3;
    const int base = 4 * i + ((v & 2) ? 1 : 0) + ((v & 1) ? 16 : 0);
    e0 = base;
    e1 = base + 2;
    sc = (v & 1) ? 0.0625f : 1.0f;
}

// Loads the 32 activations of block b of row m into registers as fp32 (128-bit loads).
__device__ __forceinline__ void load_block(const MmaParams& p, int m, int b, float (&x)[32]) {
    if (p.x_f32) {
        const float4* src = reinterpret_cast<const float4*>(
            static_cast<const float*>(p.X) + static_cast<size_t>(m) * p.K + b * 32);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 v = __ldg(src + q);
            x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
        }
    } else {
        const uint4* src = reinterpret_cast<const uint4*>(
            static_cast<const __half*>(p.X) + static_cast<size_t>(m) * p.K + b * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = __ldg(src + q);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[8 * q + 2 * e] = hbits2f(u[e] & 0xffffu);
                x[8 * q + 2 * e + 1] = hbits2f(u[e] >> 16);
            }
        }
    }
}
__device__ __forceinline__ void load_gamma_block(const MmaParams& p, int b, float (&gm)[32]) {
    if (p.x_f32) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.gamma) + b * 32);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 v = __ldg(src + q);
            gm[4 * q] = v.x; gm[4 * q + 1] = v.y; gm[4 * q + 2] = v.z; gm[4 * q + 3] = v.w;
        }
    } else {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __half*>(p.gamma) + b * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = __ldg(src + q);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                gm[8 * q + 2 * e] = hbits2f(u[e] & 0xffffu);
                gm[8 * q + 2 * e + 1] = hbits2f(u[e] >> 16);
            }
        }
    }
}

// Stages the activations of MB rows: xfrag[pass][block][16] (32-bit operand registers) and
// sxs[m][block] = 8 * 2^-24 * (sum of the block's activations); pass = m*(split?2:1) + part.
// One thread handles one block: it loads the 32 values with 128-bit loads, applies the RMSNorm
// prologue if gamma is given (sum of squares in double over the CTA, rstd = 1/sqrtf(float(ss/K)
// + eps), value = (x*rstd)*gamma in fp32), and writes the block's 16 operand registers.
template <int MB>
__device__ void stage_x(const MmaParams& p, uint8_t* smem, double* scratch) {
    const int tid = threadIdx.x;  // consumer thread 0..255
    const int nb = p.nb;
    uint4* xfrag = reinterpret_cast<uint4*>(smem + p.off_xfrag);
    float* sxs = reinterpret_cast<float*>(smem + p.off_sx);
    const int npass = p.split ? 2 : 1;
    for (int m = 0; m < MB; ++m) {
        float rstd = 1.f;
        if (p.gamma != nullptr) {
            double ss = 0.0;
            for (int b = tid; b < nb; b += kConsumerThreads) {
                float x[32];
                load_block(p, m, b, x);
#pragma unroll
                for (int e = 0; e < 32; ++e) ss += static_cast<double>(x[e]) * static_cast<double>(x[e]);
            }
            ss = csum_f64(ss, scratch);
            rstd = 1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(p.K)) + p.eps);
        }
        for (int b = tid; b < nb; b += kConsumerThreads) {
            float x[32];
            load_block(p, m, b, x);
            if (p.gamma != nullptr) {
                float gm[32];
                load_gamma_block(p, b, gm);
#pragma unroll
                for (int e = 0; e < 32; ++e) x[e] = __fmul_rn(__fmul_rn(x[e], rstd), gm[e]);
            }
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 32; ++e) s += x[e];
            sxs[m * nb + b] = s * (8.0f / 16777216.0f);
            uint32_t hi[16], lo[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                int e0, e1; float sc;
                frag_elems(j, e0, e1, sc);
                if (!p.split) {
                    hi[j] = pack_h2(x[e0] * sc, x[e1] * sc);
                } else {
                    const float h0 = __half2float(__float2half_rn(x[e0]));
                    const float h1 = __half2float(__float2half_rn(x[e1]));
                    hi[j] = pack_h2(h0 * sc, h1 * sc);
                    lo[j] = pack_h2((x[e0] - h0) * sc, (x[e1] - h1) * sc);
                }
            }
            uint4* dst = xfrag + (static_cast<size_t>(m * npass) * nb + b) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_uint4(hi[4 * q], hi[4 * q + 1], hi[4 * q + 2], hi[4 * q + 3]);
            if (p.split) {
                uint4* dl = xfrag + (static_cast<size_t>(m * npass + 1) * nb + b) * 4;
#pragma unroll
                for (int q = 0; q < 4; ++q) dl[q] = make_uint4(lo[4 * q], lo[4 * q + 1], lo[4 * q + 2], lo[4 * q + 3]);
            }
        }
    }
    consumer_sync();
}

template <int MB, int NPASS>
__global__ void __maxnreg__(kConsumerWarps > 8 ? 96 : 112) gemv_q4_mma_kernel(const MmaParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);            // [kMaxStages]
    uint64_t* empty = full + kMaxStages;                           // [kMaxStages]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 16 * kMaxStages);
    double* scratch = reinterpret_cast<double*>(smem + 16 * kMaxStages + 16);  // kConsumerWarps doubles
    float* red = reinterpret_cast<float*>(smem + p.off_red);       // [2][8 warps][16 rows][MB]
    uint8_t* ring = smem + p.off_ring;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = static_cast<int>(static_cast<long long>(p.N) * blockIdx.x / gridDim.x);
    const int r1 = static_cast<int>(static_cast<long long>(p.N) * (blockIdx.x + 1) / gridDim.x);
    const int rows = r1 - r0;
    const int panels = (rows + kPanelRows - 1) / kPanelRows;
    const int ips = p.kc >> 3;                        // items (8-block groups) per full stage
    const int ipp = p.nb >> 3;                        // items per panel
    const int total_stages = panels * p.chunks;
    const int stage_bytes = kPanelRows * p.pitch;
    const size_t row_bytes = static_cast<size_t>(p.nb) * 18;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        for (int i = 0; i < p.ns; ++i) { bar_init(&full[i], 1); bar_init(&empty[i], ips); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer warp ----------------
        for (int s = 0; s < total_stages; ++s) {
            const int slot = s % p.ns, use = s / p.ns;
            if (use > 0 && !bar_wait(&empty[slot], static_cast<uint32_t>((use - 1) & 1), abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicOr(p.err, ERR_WAIT_TIMEOUT); }
                break;
            }
            const int panel = s / p.chunks, chunk = s - panel * p.chunks;
            const int prow0 = r0 + panel * kPanelRows;
            const int nrows = min(kPanelRows, r1 - prow0);
            const int cblocks = min(p.kc, p.nb - chunk * p.kc);
            const uint32_t bytes = static_cast<uint32_t>(cblocks) * 18u;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (lane == 0) {
                bar_expect_tx(&full[slot], bytes * static_cast<uint32_t>(nrows));
                // a short last chunk holds fewer items than the barrier counts: arrive for them
                for (int i = cblocks >> 3; i < ips; ++i) bar_arrive(&empty[slot]);
            }
            __syncwarp();
            if (lane < nrows) {
                bulk_load(ring + static_cast<size_t>(slot) * stage_bytes + static_cast<size_t>(lane) * p.pitch,
                          p.W + static_cast<size_t>(prow0 + lane) * row_bytes +
                              static_cast<size_t>(chunk) * p.kc * 18,
                          bytes, &full[slot]);
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    if (tid < 16) reinterpret_cast<uint32_t*>(smem + p.off_zero)[tid] = 0u;   // B operand of idle lanes
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stage_x<MB>(p, smem, scratch);

    const int g = lane >> 2, t = lane & 3;
    const float* sxs = reinterpret_cast<const float*>(smem + p.off_sx);
    // 32-bit shared-window addresses: every load below is [register + immediate].
    const uint32_t ring32 = s_u32(ring);
    const uint32_t lane_off = static_cast<uint32_t>(g * p.pitch + t * 36);
    const uint32_t hi_row_off = static_cast<uint32_t>(8 * p.pitch);
    // This lane feeds operand B only for the column (= block of the group) it matches; all
    // other lanes read a zeroed 64-byte region.
    const bool feeds_even = (g == 2 * t), feeds_odd = (g == 2 * t + 1);
    const uint32_t base_e = feeds_even ? s_u32(smem + p.off_xfrag) : s_u32(smem + p.off_zero);
    const uint32_t base_o = feeds_odd ? s_u32(smem + p.off_xfrag) + 64u : s_u32(smem + p.off_zero);
    const uint32_t mask_e = feeds_even ? 0xffffffffu : 0u, mask_o = feeds_odd ? 0xffffffffu : 0u;
    const uint32_t pass_stride = static_cast<uint32_t>(p.nb) * 64u;
    const bool fast_items = (ips == kConsumerWarps);

    for (int panel = 0; panel < panels; ++panel) {
        float acc[MB][2];
#pragma unroll
        for (int m = 0; m < MB; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
        const int first = panel * ipp;
        // item ids of this panel that belong to this warp: id = warp (mod 8)
        int id = first + ((warp - first % kConsumerWarps) + kConsumerWarps) % kConsumerWarps;
        for (; id < first + ipp; id += kConsumerWarps) {
            const int rem = id - first;
            const int chunk = fast_items ? (rem / kConsumerWarps) : (rem / ips);
            const int bgl = fast_items ? (rem % kConsumerWarps) : (rem - chunk * ips);
            const uint32_t s = static_cast<uint32_t>(panel * p.chunks + chunk);
            const uint32_t use = __umulhi(s, p.ns_magic);          // s / ns
            const uint32_t slot = s - use * static_cast<uint32_t>(p.ns);
            if (*abort_flag) continue;
            if (!bar_wait(&full[slot], use & 1u, abort_flag)) {
                if (lane == 0) { *abort_flag = 1; atomicOr(p.err, ERR_WAIT_TIMEOUT); }
                continue;
            }
            const uint32_t wa_addr = ring32 + slot * static_cast<uint32_t>(stage_bytes) + lane_off +
                                     static_cast<uint32_t>(bgl) * 144u;
            const uint32_t wb_addr = wa_addr + hi_row_off;
            uint32_t wa[9], wb[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) { wa[i] = lds32(wa_addr + 4 * i); wb[i] = lds32(wb_addr + 4 * i); }

            // code words: the even block of the pair straddles word boundaries by 2 bytes
            uint32_t ea[4], eb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ea[i] = __funnelshift_r(wa[i], wa[i + 1], 16);
                eb[i] = __funnelshift_r(wb[i], wb[i + 1], 16);
            }
            const int blk = chunk * p.kc + bgl * 8 + 2 * t;      // even block index in the row
            const uint32_t xoff = static_cast<uint32_t>(blk) * 64u;
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                // two independent accumulation chains hide the MMA latency
                float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ps = 0; ps < NPASS; ++ps) {
                    const uint32_t off = xoff + static_cast<uint32_t>(m * NPASS + ps) * pass_stride;
                    const uint32_t pe = base_e + (off & mask_e), po = base_o + (off & mask_o);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 be = lds128(pe + 16 * i);
                        const uint4 bo = lds128(po + 16 * i);
                        const uint32_t sa = ea[i] >> 8, sb = eb[i] >> 8;
                        const uint32_t oa = wa[5 + i], ob = wb[5 + i];
                        const uint32_t ta = oa >> 8, tb = ob >> 8;
                        mma16816(c, ea[i] & 0x000f000fu, eb[i] & 0x000f000fu, oa & 0x000f000fu,
                                 ob & 0x000f000fu, be.x, bo.x);
                        mma16816(d, ea[i] & 0x00f000f0u, eb[i] & 0x00f000f0u, oa & 0x00f000f0u,
                                 ob & 0x00f000f0u, be.y, bo.y);
                        mma16816(c, sa & 0x000f000fu, sb & 0x000f000fu, ta & 0x000f000fu,
                                 tb & 0x000f000fu, be.z, bo.z);
                        mma16816(d, sa & 0x00f000f0u, sb & 0x00f000f0u, ta & 0x00f000f0u,
                                 tb & 0x00f000f0u, be.w, bo.w);
                    }
                }
                // c[0]+d[0]: row g x even block, [1]: row g x odd block, [2]/[3]: row g+8.
                const float2 zs = *reinterpret_cast<const float2*>(&sxs[m * p.nb + blk]);
                const float de_a = hbits2f(wa[0] & 0xffffu), do_a = hbits2f(wa[4] >> 16);
                const float de_b = hbits2f(wb[0] & 0xffffu), do_b = hbits2f(wb[4] >> 16);
                acc[m][0] = fmaf(de_a, (c[0] - zs.x) + d[0], fmaf(do_a, (c[1] - zs.y) + d[1], acc[m][0]));
                acc[m][1] = fmaf(de_b, (c[2] - zs.x) + d[2], fmaf(do_b, (c[3] - zs.y) + d[3], acc[m][1]));
            }
            // Released only after every word loaded from the slot has been used: a release placed
            // right after issuing the loads does not stop them from being scheduled later, after
            // the producer's next copy has landed.
            __syncwarp();
            if (lane == 0) bar_arrive(&empty[slot]);
        }
        // combine the four block-pair lanes of each row, then the eight warps
        float* rbuf = red + static_cast<size_t>(panel & 1) * kConsumerWarps * kPanelRows * MB;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = acc[m][h];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if (t == 0) rbuf[(warp * kPanelRows + g + 8 * h) * MB + m] = v;
            }
        }
        consumer_sync();
        if (tid < kPanelRows * MB) {
            const int r = tid / MB, m = tid - r * MB;
            const int row = r0 + panel * kPanelRows + r;
            if (row < r1) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) v += rbuf[(w * kPanelRows + r) * MB + m];
                v *= 16777216.0f;
                const size_t o = static_cast<size_t>(m) * p.N + row;
                if (p.y_f32) static_cast<float*>(p.Y)[o] = v;
                else static_cast<__half*>(p.Y)[o] = __float2half_rn(v);
            }
        }
    }
    if (*abort_flag) {
        // let copies that are still in flight land before the CTA's shared memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
}

inline int up(int v, int a) { return (v + a - 1) / a * a; }

}  // namespace

cudaError_t init_mma_kernels(int smem_optin) {
    cudaError_t e = cudaSuccess;
#define TCB_MMA_SET(MB, NP)                                                                  \
    e = cudaFuncSetAttribute(gemv_q4_mma_kernel<MB, NP>,                                     \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);       \
    if (e != cudaSuccess) return e;
    TCB_MMA_SET(1, 1) TCB_MMA_SET(1, 2) TCB_MMA_SET(2, 1) TCB_MMA_SET(2, 2)
#undef TCB_MMA_SET
    return e;
}

// Returns cudaErrorNotSupported when the shape / alignment is outside this kernel's domain
// (the caller then uses another variant).
cudaError_t launch_gemv_q4_mma(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                               const char** name) {
    if (a.fmt != FMT_Q4_0 || a.M < 1 || a.M > 2 || a.K % 256 != 0) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(a.W) & 15u) != 0) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(a.X) & 15u) != 0) return cudaErrorNotSupported;
    if (a.gamma && (reinterpret_cast<uintptr_t>(a.gamma) & 15u) != 0) return cudaErrorNotSupported;
    const int nb = a.K / 32;
    const bool split = a.x_f32 || a.gamma != nullptr;
    MmaParams p;
    p.W = a.W; p.X = a.X; p.Y = a.Y; p.gamma = a.gamma; p.err = env.err_word;
    p.M = a.M; p.N = a.N; p.K = a.K; p.nb = nb;
    p.kc = nb < kMaxKc ? nb : kMaxKc;
    p.chunks = (nb + p.kc - 1) / p.kc;
    const int m8 = p.kc / 8;
    p.pitch = p.kc * 18 + ((m8 & 1) ? 32 : 16);   // pitch / 16 odd: conflict-free row stride
    p.x_f32 = a.x_f32 ? 1 : 0;
    p.y_f32 = a.y_f32 ? 1 : 0;
    p.split = split ? 1 : 0;
    p.eps = a.eps;
    int off = 16 * kMaxStages + 16 + 8 * kConsumerWarps;
    off = up(off, 16);
    p.off_red = off;
    off += up(2 * kConsumerWarps * kPanelRows * a.M * 4, 16);
    p.off_sx = off;
    off += up(a.M * nb * 4, 16);
    p.off_zero = off;
    off += 64;
    p.off_xfrag = off;
    off += up(a.M * (split ? 2 : 1) * nb * 64, 128);
    p.off_ring = off;
    const int stage_bytes = kPanelRows * p.pitch;
    const int optin = env.smem_optin > 0 ? env.smem_optin : 232448;
    // 17 warps at 112 registers fill the register file: no second CTA fits, use all shared memory
    const int half_budget = kConsumerWarps > 8 ? optin - 2048 : optin / 2 - 1024;
    int ns = (half_budget - off) / stage_bytes;
    if (ns < 2) ns = (optin - off) / stage_bytes;       // one CTA per SM
    if (ns < 2) return cudaErrorNotSupported;
    if (ns > kMaxStages) ns = kMaxStages;
    p.ns = ns;
    p.ns_magic = static_cast<uint32_t>(0xFFFFFFFFu / static_cast<uint32_t>(ns)) + 1u;
    const int smem = off + ns * stage_bytes;

    static const int ctas_per_sm = [] {
        const char* v = std::getenv("TC_GEMV_CTAS_PER_SM");
        const int n = v ? std::atoi(v) : 1;
        return n >= 1 && n <= 4 ? n : 1;
    }();
    const int max_groups = (a.N + kPanelRows - 1) / kPanelRows;
    int grid = env.sm_count * ctas_per_sm;
    if (grid > max_groups) grid = max_groups;
    if (grid < 1) grid = 1;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (env.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (name) *name = split ? "q4_0_gemv_mma_split_sm100" : "q4_0_gemv_mma_sm100";
    if (a.M == 1)
        return split ? cudaLaunchKernelEx(&cfg, gemv_q4_mma_kernel<1, 2>, p)
                     : cudaLaunchKernelEx(&cfg, gemv_q4_mma_kernel<1, 1>, p);
    return split ? cudaLaunchKernelEx(&cfg, gemv_q4_mma_kernel<2, 2>, p)
                 : cudaLaunchKernelEx(&cfg, gemv_q4_mma_kernel<2, 1>, p);
}

}  // namespace tcb
