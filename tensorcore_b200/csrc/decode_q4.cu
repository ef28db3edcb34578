// Persistent decode kernel for sm_100a: a whole recorded list of Q4_0, M = 1 GEMVs - one decode
// token - in ONE cooperative launch, one CTA per SM; tensor parallel: one such launch per rank.
//
// Work.  An operation Y[N] = dequant(W[N,K]) . x[K] is cut into boxes of 32 weight rows x one
// 8-block group (144 bytes per row, 256 weights per row), each fetched by one tiled TMA copy
// through a per-operation tensor map.  Operations that share their input and need no ordering
// between them (q/k/v, gate/up) form a phase.  The boxes of a phase are numbered band-major - a
// band is four consecutive groups, i.e. 1024 input elements and 576 contiguous bytes of every
// row - then by row block, then by group inside the band, and dealt evenly to the CTAs (CTA c
// owns boxes [U*c/G, U*(c+1)/G)).  So every SM streams the same number of bytes whatever N is, and
// a CTA needs only the one or two bands of the input that its boxes touch.
//
// Three kinds of warps.  Producer warps walk the CTA's box sequence over all phases and keep a ring
// of boxes in shared memory full (weights do not depend on activations: the ring refills while the
// consumers are between two phases).  Consumer warps take a box each: a lane owns one ROW of the
// box, all lanes read the same int16 activations from shared memory (one broadcast per load), and
// the lane adds its partial dot product, together with a count of one, to the operation's
// accumulator pair in global memory with ONE vector reduction (L2 atomics; the K split of a row
// over boxes, warps, CTAs and - tensor parallel - GPUs all ends in the same pair).  Housekeeping
// warps follow behind: result buffers, clearing, and an arrival counter that nobody waits at.
//
// Epochs without barriers.  Operations that read what an earlier one wrote belong to different
// epochs.  A CTA that starts an epoch stages ITS bands of the input straight from the producer's
// accumulator pairs (L2-coherent loads, scaled and rounded to the producer's result type),
// quantised to int16 with one scale per 32 elements, and simply repeats the load until every
// pair's count says that all of the row's partial sums have arrived.  RMSNorm prologue: the row
// x*gamma is quantised without the 1/rms factor, which needs the whole row; instead the CTAs that
// stage a band leave the band's sum of squares, with a flag, in a slot beside the accumulators,
// and whoever reads the accumulators next (the next staging pass, or the housekeeping warp that
// writes the result buffer) multiplies by 1/sqrt(mean square + eps) computed from the slots.  The
// accumulators come from a pool in twelve generations (epoch mod 12) and are all zero again when
// the kernel ends.
//
// Every wait is bounded (about a second), sets an error bit and lets the kernel end.
#include "gemv_common.cuh"
#include "tensor_map.h"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

namespace tcb {
namespace {

constexpr int kMaxPhaseOps = 4;        // operations merged into one phase
constexpr int kBoxBytes = 32 * 144;
constexpr int kBandGroups = 4;         // groups per band
constexpr int kMaxBands = 32;          // slots per staged row: K <= 32 * 1024
constexpr uint32_t MOP_NO_STORE = 256u;  // internal: a later operation overwrites this result before anyone reads it
constexpr int kPhaseLenShift = 16;     // MegaOp::flags bits 16..18: operations in the phase that starts here
constexpr int kDecodeMaxSlots = 64;    // ring slots: 16 consumer warps x 4 stages at most
constexpr int kProducerWarps = 4;     // one per warp scheduler
constexpr int kFlowGenerations = 12;  // accumulator generations of the one-GPU kernel (epoch mod 12)
constexpr int kKeeperWarps = 4;       // housekeeping warps: they take the epochs in turn
constexpr int kAuxWarps = kProducerWarps + kKeeperWarps;
constexpr int kDecodeMaxThreads = (kMaxStreamWarps + kProducerWarps + kKeeperWarps) * 32;   // consumer, producer and housekeeping warps

__device__ __forceinline__ void arrive_gpu(unsigned long long* p) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(1ULL) : "memory");
}
__device__ __forceinline__ void arrive_relaxed_sys(unsigned long long* p) {
    asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(1ULL) : "memory");
}
__device__ __forceinline__ unsigned long long poll_gpu(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long poll_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// floor(x / gridDim) without a division: x * ceil(2^32 / gridDim) >> 32.  For x below 2^32 the
// result is the exact quotient or one more; every partition below takes both of its ends from this
// same function (clamped to the total), so the pieces still tile the range exactly.
__device__ __forceinline__ uint32_t grid_share(uint32_t total, uint32_t c, uint32_t inv_grid) {
    const uint32_t q = __umulhi(total * c, inv_grid);
    return q < total ? q : total;
}

// a / b for b > 0 and a < 2^31 without the integer division sequence: a float quotient (which can be
// off by one either way) corrected with one multiply.
__device__ __forceinline__ uint32_t div_u32(uint32_t a, uint32_t b) {
    uint32_t q = __float2uint_rz(__fdividef(__uint2float_rz(a), __uint2float_ru(b)));
    if (q * b > a) --q;
    uint32_t r = a - q * b;
    while (r >= b) { r -= b; ++q; }
    return q;
}

// What a CTA needs to know about one phase, worked out once at kernel start and kept in shared
// memory: its share of the phase's boxes and where they sit in the CTA's box sequence.
struct PhaseRec {
    uint32_t s0;              // sequence number (over the whole launch) of this CTA's first box of the phase
    uint32_t n;               // this CTA's boxes in the phase
    uint32_t c0;              // number of its first box within the phase
    uint32_t R;               // row blocks of the phase's operations together
    uint32_t rb[3];           // first row block of the phase's 2nd, 3rd, 4th operation (~0u when absent)
    uint16_t o;               // first operation
    uint8_t len, band_lo;     // operations in the phase; first band this CTA touches ...
    uint16_t gpr;             // groups per row
    uint8_t band_hi, pad;     // ... and the last
    uint32_t pad2;
};
static_assert(sizeof(PhaseRec) == 40, "phase records are read in 8-byte pieces");

// Position of box u of a phase: band-major, then row block, then group inside the band.  Full
// bands hold 4R boxes (R row blocks), a last narrower band R * (gpr % 4).
__device__ __forceinline__ void box_position(uint32_t R, uint32_t gpr, uint32_t u, uint32_t& kg, uint32_t& r) {
    const uint32_t full = gpr / kBandGroups, per = R * kBandGroups;
    uint32_t band = div_u32(u, per), kgi;
    if (band >= full) {
        band = full;
        const uint32_t w = gpr % kBandGroups, off = u - full * per;   // callers keep u below R * gpr, so w > 0 here
        r = w == 3 ? div_u32(off, 3) : (w == 2 ? off >> 1 : off);
        kgi = off - r * w;
    } else {
        const uint32_t off = u - band * per;
        r = off / kBandGroups;
        kgi = off % kBandGroups;
    }
    kg = band * kBandGroups + kgi;
}

// This CTA's share of a vector of n rows.
__device__ __forceinline__ void cta_slice(uint32_t n, uint32_t inv_grid, uint32_t& lo, uint32_t& hi) {
    lo = grid_share(n, blockIdx.x, inv_grid);          // plan_decode keeps n below 2^24: no overflow
    hi = blockIdx.x + 1 == gridDim.x ? n : grid_share(n, blockIdx.x + 1, inv_grid);
}

// Barrier among the consumer warps only (the other warps never join it).
__device__ __forceinline__ void consumer_sync(int nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One atomic operation adds a partial sum to an accumulator and counts the addition beside it.
__device__ __forceinline__ void red_add_pair(float2* p, float v) {
    asm volatile("red.relaxed.gpu.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v), "f"(1.0f) : "memory");
}
__device__ __forceinline__ void red_add_pair_sys(float2* p, float v) {     // into another GPU's pool as well
    asm volatile("red.relaxed.sys.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(v), "f"(1.0f) : "memory");
}
// Two accumulators with their counts, straight from L2.  `sys`: other GPUs add to them too.
__device__ __forceinline__ float4 ld_pairs(const float2* p, bool sys) {
    float4 v;
    if (sys)
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    else
        asm volatile("ld.relaxed.gpu.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_pair(const float2* p, bool sys = false) {
    float2 v;
    if (sys) asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}
constexpr long long kWaitClocks = 2000000000LL;    // about a second: every wait gives up after this

// 1 / sqrt(mean square + eps) of a row of K elements from the per-band sums of squares its staging
// pass left in the pool, each stored together with a flag; waits (bounded) until all are there.
// Called by whole warps; every reader runs the same arithmetic, so they all get the same bits.
__device__ __forceinline__ float rstd_from_flagged_slots(const float2* slots, int K, float eps, volatile int* abort_s) {
    const int nbands = ((K >> 8) + kBandGroups - 1) / kBandGroups, l = threadIdx.x & 31;
    float t = 0.f;
    if (l < nbands) {
        float2 v = ld_pair(slots + l);
        if (v.y != 1.0f) {
            const long long t0 = clock64();
            while ((v = ld_pair(slots + l)).y != 1.0f) {
                if (*abort_s || clock64() - t0 > kWaitClocks) { *abort_s = 1; break; }
            }
        }
        t = v.x;
    }
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return rsqrtf(t / static_cast<float>(K) + eps);
}

// Stages bands [band_lo, band_hi] of the input of `op` (the head of a phase) as int16 with one
// scale per 32 elements, at their natural positions in the shared-memory row.  Four warps take
// one band (32 chunks of 8 elements each per group), so up to four bands are staged at a time.
// Input from the accumulators of the epoch before: a thread reads its eight sums together with
// their counts and repeats the read until every count says that all partial sums have arrived -
// the completed value and the knowledge that it is complete come in the same load, no barrier in
// between.  Fused RMSNorm: quantises x * gamma and leaves each band's sum of squares, with a flag,
// in its slot.
template <bool SYS>
__device__ void stage_bands_flow(const MegaOp& op, const DecodeParams& p, uint8_t* smem, float* scratch,
                                 uint32_t band_lo, uint32_t band_hi, int nthreads, volatile int* abort_s) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;     // the consumers are the CTA's first warps
    const int nwarps = nthreads >> 5;
    const uint32_t flags = op.flags;
    const bool fused = (flags & MOP_FUSED) != 0, f16 = !(flags & MOP_X_F32);
    const bool from_acc = op.xacc_off >= 0, round16 = (flags & MOP_XACC_F16) != 0;
    const int K = op.K, nb = K >> 5, gpr = K >> 8;
    const bool pow2 = (from_acc ? round16 : f16) && !fused;
    const int xkind = f16 ? 0 : 1, gkind = f16 ? 0 : 1;
    float2* pool2 = reinterpret_cast<float2*>(p.pool);
    uint4* dst = reinterpret_cast<uint4*>(smem + p.off_x);
    float2* sx2 = reinterpret_cast<float2*>(smem + p.off_sx);
    const float want = static_cast<float>(op.xexpect);
    const uint32_t per_pass = static_cast<uint32_t>(nwarps) / 4;
    for (uint32_t b0 = band_lo; b0 <= band_hi; b0 += per_pass) {
        const uint32_t band = b0 + static_cast<uint32_t>(warp >> 2);
        const bool mine = band <= band_hi;
        const int g0 = static_cast<int>(band) * kBandGroups;
        const int width = mine ? min(kBandGroups, gpr - g0) : 0;          // groups in this band
        float ssq = 0.f;
        for (int c = (warp & 3) * 32 + lane; c - lane < width * 32; c += 128) {   // warp-uniform trip count
            const bool live = c < width * 32;
            const int i = g0 * 32 + c;                                    // chunk index in the row
            float v[8], g[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { v[e] = 0.f; g[e] = 1.f; }
            if (live && fused) load8<false>(op.gamma, gkind, 8 * static_cast<size_t>(i), g);
            if (from_acc) {
                if (live) {
                    const float2* src = pool2 + op.xacc_off + 8 * static_cast<size_t>(i);
                    float4 a[4];
                    bool done = false;
                    const long long t0 = clock64();
                    while (!done) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) a[e] = ld_pairs(src + 2 * e, SYS);
                        done = true;
#pragma unroll
                        for (int e = 0; e < 4; ++e) done = done && a[e].y == want && a[e].w == want;
                        if (!done && (*abort_s || clock64() - t0 > kWaitClocks)) { *abort_s = 1; break; }
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) { v[2 * e] = a[e].x; v[2 * e + 1] = a[e].z; }
                }
                // what the producer's result buffer will hold: the accumulator scaled by the
                // producer's own 1/rms (when its prologue was fused) and rounded to its type
                const float xs = op.xss_off >= 0
                                     ? rstd_from_flagged_slots(pool2 + op.xss_off, op.xss_k, op.xss_eps, abort_s) : 1.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    v[e] *= xs;
                    if (round16) v[e] = __half2float(__float2half_rn(v[e]));
                }
            } else if (live) {
                load8<true>(op.X, xkind, 8 * static_cast<size_t>(i), v);
            }
            if (fused) {
                ssq += sumsq8(v);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], g[e]);
            }
            quantise_chunk<true>(v, live, i, 0, 8, pow2, gpr, nb, dst, sx2);
        }
        if (fused) {
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) scratch[warp] = ssq;
        }
        consumer_sync(nthreads);
        if (fused && tid < static_cast<int>(per_pass) && b0 + tid <= band_hi) {
            const float* s4 = scratch + 4 * tid;
            pool2[op.ss_off + b0 + tid] = make_float2((s4[0] + s4[1]) + (s4[2] + s4[3]), 1.0f);
        }
        if (b0 + per_pass <= band_hi) consumer_sync(nthreads);    // the partial sums are reused by the next pass
    }
}

// ---------------------------------------------------------------------------------------
// The producer warps.  Producer pi feeds consumer warps pi, pi + np, ...: it walks their part of
// this CTA's box sequence - all phases, in order - 32 boxes at a time, one lane per box: finds the
// box's phase, its position in the phase, its operation and row block.  Then, a few boxes at a
// time, it waits for the ring slot to be free, leaves a descriptor for the consumer (accumulator
// index of the box's row 0, group, valid rows) and starts the tiled copy.  Weights do not depend
// on activations: the producers never wait for data, so the ring is full again while the
// consumers are still between two phases.  Every ring slot has exactly one producer, which fills
// it in order - so a wait on a slot's barriers is always for their current phase.  (A wait by
// parity for a phase further ahead would be answered by an older one.)
// ---------------------------------------------------------------------------------------
struct BoxRef { int x, y; uint32_t opi, d0, d1; };

__device__ __forceinline__ bool locate_box(const PhaseRec* phases, int n_phases, const MegaOp* ops, uint32_t s,
                                           int& ph, BoxRef& b) {
    while (ph < n_phases && s >= phases[ph].s0 + phases[ph].n) ++ph;
    if (ph >= n_phases) return false;
    const PhaseRec& r = phases[ph];
    uint32_t kg, rblk;
    box_position(r.R, r.gpr, r.c0 + (s - r.s0), kg, rblk);
    uint32_t k = 0, base = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j)
        if (rblk >= r.rb[j]) { k = j + 1; base = r.rb[j]; }
    const uint32_t rb = rblk - base;
    b.opi = r.o + k;
    const MegaOp& op = ops[b.opi];
    b.x = static_cast<int>(kg * 144u);
    b.y = static_cast<int>(rb * 32u);
    const uint32_t left = static_cast<uint32_t>(op.N) - rb * 32u;
    b.d0 = op.acc_off + op.y_row0 + rb * 32u;
    b.d1 = kg | ((left < 32u ? left : 32u) << 16) | ((op.flags & MOP_PEERS) ? (1u << 24) : 0u);
    return true;
}

__device__ void produce_boxes(const DecodeParams& p, const MegaOp* ops, const PhaseRec* phases, int n_phases,
                              uint64_t* full, uint64_t* empty, uint2* desc, uint8_t* ring, volatile int* abort_s,
                              int nwc, int pi, int np) {
    const int lane = threadIdx.x & 31;
    const uint32_t ns = static_cast<uint32_t>(p.ns);
    const uint32_t wp = static_cast<uint32_t>(nwc / np);         // consumer warps per producer
    const uint32_t rpc = 32u / wp;                               // rounds of the consumer warps per 32 boxes
    const uint32_t my_w = static_cast<uint32_t>(pi) + static_cast<uint32_t>(np) * (static_cast<uint32_t>(lane) % wp);
    const uint32_t my_r = static_cast<uint32_t>(lane) / wp;
    const uint8_t* maps = static_cast<const uint8_t*>(p.maps);   // one 128-byte tensor map per operation
    const uint32_t total = n_phases > 0 ? phases[n_phases - 1].s0 + phases[n_phases - 1].n : 0u;
    const uint32_t rounds = (total + static_cast<uint32_t>(nwc) - 1u) / static_cast<uint32_t>(nwc);
    uint32_t kb = 0;                 // next round to issue (a round = one box per consumer warp)
    int ph_s = 0;                    // a phase at or before the one of the first box of that round
    bool ok = true;
    while (kb < rounds && ok) {
        int ph = ph_s;
        BoxRef b;
        const uint32_t k = kb + my_r, q = k * static_cast<uint32_t>(nwc) + my_w;
        const bool live = locate_box(phases, n_phases, ops, q, ph, b);
        const uint32_t slot = my_w + static_cast<uint32_t>(nwc) * (k % ns), use = k / ns;
        // Lanes issue their boxes a few at a time, in order, so that the ring refills as it drains.
        constexpr int kBatch = 4;
        for (int sub = 0; sub < 32 && ok; sub += kBatch) {
            bool good = true;
            if (live && lane >= sub && lane < sub + kBatch) {
                if (use > 0) {
                    // the consumer has copied the slot's previous box into registers
                    const uint32_t par = (use - 1u) & 1u;
                    if (!mbar_try_wait(&empty[slot], par)) {
                        int tries = 0;
                        while (!mbar_try_wait_parked(&empty[slot], par, 1000000u)) {      // up to a millisecond each
                            if (*abort_s || ++tries > 1000) { good = false; break; }
                        }
                    }
                }
                if (good) {
                    desc[slot] = make_uint2(b.d0, b.d1);
                    mbar_expect_tx(&full[slot], kBoxBytes);
                    sm100::tensor_load_2d(ring + static_cast<size_t>(slot) * kBoxBytes,
                                          maps + static_cast<size_t>(b.opi) * kDecodeMapBytes, b.x, b.y, &full[slot]);
                }
            }
            ok = __all_sync(0xffffffffu, good);
        }
        ph = __shfl_sync(0xffffffffu, ph, 0);
        ph_s = ph < n_phases ? ph : ph_s;
        kb += rpc;
    }
    if (!ok && lane == 0) { *abort_s = 1; atomicOr(p.err, ERR_WAIT_TIMEOUT); }
    // Nothing may still be on its way into this CTA's shared memory when the CTA ends: wait (bounded)
    // for the last copy into each of this warp's slots.  Only the LAST use of a slot can be waited
    // for by parity.  (After a failure a slot whose copy was never started runs into the bound.)
    if (my_r < ns && total > my_w) {
        const uint32_t k_max = (total - 1u - my_w) / static_cast<uint32_t>(nwc);   // last round of consumer warp my_w
        if (k_max >= my_r) {
            const uint32_t k = k_max - (k_max - my_r) % ns;                        // its last round in stage my_r
            (void)mbar_wait_bounded(&full[my_w + static_cast<uint32_t>(nwc) * my_r], (k / ns) & 1u);
        }
    }
}

// ---------------------------------------------------------------------------------------
// The housekeeping warps.  Everything that is not on the path from one operation's last partial
// sum to the next operation's first box happens here, behind the consumers.  Four warps take the
// epochs in turn, each with an arrival counter of its own, so that one iteration may last four
// epochs.  An iteration, for epoch e, once the CTA's consumers have finished e:
//     1. this CTA's slice of the results of epoch e - 1 goes to the result buffers: the counts
//        say when a row is complete, the 1/rms factors of fused operations come from their sums
//        of squares;
//     2. the CTA arrives on the warp's arrival counter (release: publishes step 1 and the
//        clearing of the iteration before) and
//     3. waits until every CTA has arrived for epoch e: then nobody reads the accumulators of
//        epoch e - 1 any more (they were read while staging epoch e), nor its sums of squares
//        (staging, and step 1);
//     4. it zeroes its slice of those accumulators, and the sums of squares;
//     5. it notes that iteration e is done.
// The accumulators come from a pool in G generations.  Those that epoch t uses were last used by
// epoch t - G, cleared in iteration t - G + 1 and published by the same warp's next arrival, in
// iteration t - G + 5: a consumer starts epoch t when that iteration is done (with G = 12 that
// iteration began seven epochs earlier).  A phase whose input is a result buffer written by this
// launch in epoch s (three epochs earlier or more; anything closer reads the accumulators) waits
// for iteration s + 1 instead, which stored and published it.
// So the counters are grid barriers that nobody waits at: they trail the computation.
// ---------------------------------------------------------------------------------------
__device__ void epoch_scales(const MegaOp* ops, int b, int e, const float2* pool2, float* jscale, int cap,
                             volatile int* abort_s) {
    const int lane = threadIdx.x & 31;
    constexpr int kOpsAtOnce = 4;
    for (int kb = b; kb < e; kb += kOpsAtOnce) {
        float2 sl[kOpsAtOnce];
#pragma unroll
        for (int j = 0; j < kOpsAtOnce; ++j) {      // all loads first, then the (rarely needed) waits
            sl[j] = make_float2(0.f, 1.0f);
            if (kb + j < e) {
                const MegaOp& op = ops[kb + j];
                const int nbands = ((op.K >> 8) + kBandGroups - 1) / kBandGroups;
                if ((op.flags & MOP_FUSED) && !(op.flags & MOP_NO_STORE) && lane < nbands) sl[j] = ld_pair(pool2 + op.ss_off + lane);
            }
        }
#pragma unroll
        for (int j = 0; j < kOpsAtOnce; ++j) {
            if (kb + j >= e) break;
            const MegaOp& op = ops[kb + j];
            float sc = 1.0f;
            if ((op.flags & MOP_FUSED) && !(op.flags & MOP_NO_STORE)) {
                if (sl[j].y != 1.0f) {
                    const long long t0 = clock64();
                    while ((sl[j] = ld_pair(pool2 + op.ss_off + lane)).y != 1.0f) {
                        if (*abort_s || clock64() - t0 > kWaitClocks) { *abort_s = 1; break; }
                    }
                }
                float t = sl[j].x;      // the same arithmetic as rstd_from_flagged_slots
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                sc = rsqrtf(t / static_cast<float>(op.K) + op.eps);
            }
            if (lane == 0 && kb + j - b < cap) jscale[kb + j - b] = sc;
        }
    }
    __syncwarp();
}

__device__ void epoch_results(const MegaOp* ops, int b, int e, const float2* pool2, uint32_t inv_grid,
                              const float* jscale, int cap, volatile int* abort_s, bool sys) {
    const int lane = threadIdx.x & 31;
    constexpr int kRowsAtOnce = 8;
    for (int k = b; k < e; ++k) {
        const MegaOp& op = ops[k];
        const uint32_t flags = op.flags;
        if (flags & MOP_NO_STORE) continue;
        uint32_t lo, hi;
        cta_slice(op.y_rows, inv_grid, lo, hi);
        const float2* acc = pool2 + op.acc_off;
        const float want = static_cast<float>(op.expect);
        const float scale = k - b < cap ? jscale[k - b]
                                        : ((flags & MOP_FUSED) ? rstd_from_flagged_slots(pool2 + op.ss_off, op.K, op.eps, abort_s) : 1.0f);
        const uint32_t r0 = op.y_row0, r1 = op.y_row0 + static_cast<uint32_t>(op.N);
        const bool all_rows = sys && (flags & MOP_PEERS);
        void* Y = op.Y;
        for (uint32_t i0 = lo + lane; i0 < hi; i0 += 32u * kRowsAtOnce) {
            float2 v[kRowsAtOnce];
#pragma unroll
            for (int u = 0; u < kRowsAtOnce; ++u) {
                const uint32_t i = i0 + 32u * u;
                if (i < hi) v[u] = ld_pair(acc + i, sys);
            }
#pragma unroll
            for (int u = 0; u < kRowsAtOnce; ++u) {
                const uint32_t i = i0 + 32u * u;
                if (i >= hi) break;
                // rows outside this operation's part get nothing - unless the other ranks fill them
                const float need = (all_rows || (i >= r0 && i < r1)) ? want : 0.f;
                if (v[u].y != need) {
                    const long long t0 = clock64();
                    while ((v[u] = ld_pair(acc + i)).y != need) {
                        if (*abort_s || clock64() - t0 > kWaitClocks) { *abort_s = 1; break; }
                    }
                }
                const float y = v[u].x * scale;
                if (flags & MOP_Y_F32) static_cast<float*>(Y)[i] = y;
                else static_cast<__half*>(Y)[i] = __float2half_rn(y);
            }
        }
    }
}
__device__ void zero_epoch(const MegaOp* ops, int b, int e, float2* pool2, uint32_t inv_grid) {
    const int lane = threadIdx.x & 31;
    for (int k = b; k < e; ++k) {
        const MegaOp& op = ops[k];
        uint32_t lo, hi;
        cta_slice(op.y_rows, inv_grid, lo, hi);
        float2* acc = pool2 + op.acc_off;
        for (uint32_t i = lo + lane; i < hi; i += 32) acc[i] = make_float2(0.f, 0.f);
        // the slots are few: every CTA clears them all (they all do it after the same wait)
        if ((op.flags & MOP_FUSED) && (op.flags & MOP_RESTAGE)) pool2[op.ss_off + lane] = make_float2(0.f, 0.f);
    }
}

template <bool MULTI>
__device__ void keep_house(const DecodeParams& p, const MegaOp* ops, const uint16_t* ep_op, int n_epochs,
                           volatile int* ctl, float* jscale, int jp) {
    const int lane = threadIdx.x & 31;
    float2* pool2 = reinterpret_cast<float2*>(p.pool);
    constexpr bool multi = MULTI;
    unsigned long long* counter = p.counter + 4 * jp;    // each housekeeping warp has its own, 32 bytes apart
    unsigned long long target = p.base;
    const unsigned long long per_round = static_cast<unsigned long long>(gridDim.x) * (multi ? p.n_ranks : 1);
    // Tensor parallel: a CTA arrives on the counter of every rank, so a round is complete when the
    // CTAs of all ranks have arrived - other ranks add into this rank's accumulators, and must not
    // before it has cleared them.
    auto arrive = [&]() {
        if (multi) {
            // one fence for all ranks' counters (a release per counter would wait for the system-wide
            // fence once per rank)
            __threadfence_system();
            for (int r = 0; r < p.n_ranks; ++r) arrive_relaxed_sys(p.peer_counter[r] + 4 * jp);
        } else {
            arrive_gpu(counter);
        }
    };
    // One more iteration than there are epochs: the last one finishes the last epoch.  Every warp
    // arrives equally often per launch (the host advances one base for all counters): a warp with
    // an iteration less makes up for it with a bare arrival.
    const int rounds = (n_epochs + kKeeperWarps) / kKeeperWarps;
    for (int it = 0; it < rounds; ++it) {
        const int e = jp + it * kKeeperWarps;
        if (e > n_epochs) {
            if (lane == 0) arrive();
            target += per_round;
            break;
        }
        if (e < n_epochs && lane == 0) {
            const long long t0 = clock64();
            while (ctl[2] < e + 1) {                   // the consumers have finished epoch e
                if (ctl[0] || clock64() - t0 > kWaitClocks) { ctl[0] = 1; break; }
                __nanosleep(200);                      // leave the issue slots to the consumers
            }
        }
        __syncwarp();
        const int b = e > 0 ? ep_op[e - 1] : 0, en = e > 0 ? ep_op[e] : 0;     // operations of epoch e - 1
        epoch_scales(ops, b, en, pool2, jscale, p.jscale_cap, &ctl[0]);
        epoch_results(ops, b, en, pool2, p.inv_grid, jscale, p.jscale_cap, &ctl[0], multi);
        target += per_round;
        __syncwarp();
        if (lane == 0) {
            arrive();
            const long long t0 = clock64();
            while ((multi ? poll_sys(counter) : poll_gpu(counter)) < target) {
                if (ctl[0] || clock64() - t0 > kWaitClocks) { ctl[0] = 1; break; }
            }
        }
        __syncwarp();
        if (ctl[0]) break;
        zero_epoch(ops, b, en, pool2, p.inv_grid);
        __syncwarp();
        if (lane == 0) ctl[8 + jp] = e;
    }
    if (multi && !ctl[0]) {
        // Another rank may start its next launch, and add into this rank's accumulators, as soon as
        // it leaves this kernel: nobody leaves before everyone has cleared everything.
        target += per_round;
        __syncwarp();
        if (lane == 0) {
            arrive();
            const long long t0 = clock64();
            while (poll_sys(counter) < target) {
                if (ctl[0] || clock64() - t0 > kWaitClocks) { ctl[0] = 1; break; }
            }
        }
        __syncwarp();
    }
    if (ctl[0] && lane == 0) atomicOr(p.err, ERR_WAIT_TIMEOUT);
}

// MULTI: tensor parallel (results may be added into other ranks' accumulators, system-scope loads and
// arrival rounds); the one-GPU instance carries none of that in its loops.
template <bool MULTI>
__global__ void __launch_bounds__(kDecodeMaxThreads, 1) decode_q4_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                      // [kDecodeMaxSlots]
    uint64_t* empty = full + kDecodeMaxSlots;                                // [kDecodeMaxSlots]
    float* scratch = reinterpret_cast<float*>(smem + 16 * kDecodeMaxSlots);  // [32]
    // [0] abort, [1] phases found, [2] epochs the consumers have finished, [4] the consumers' common
    // view of [0], [8 + j] last iteration housekeeping warp j has completed
    volatile int* ctl = reinterpret_cast<volatile int*>(smem + 16 * kDecodeMaxSlots + 128);
    uint2* desc = reinterpret_cast<uint2*>(smem + p.off_desc);               // [kDecodeMaxSlots]
    PhaseRec* phases = reinterpret_cast<PhaseRec*>(smem + p.off_phases);
    uint16_t* ep_op = reinterpret_cast<uint16_t*>(smem + p.off_epochs);      // first operation of every epoch
    uint8_t* ring = smem + p.off_ring;
    const uint8_t* xs = smem + p.off_x;
    const float2* sx2 = reinterpret_cast<const float2*>(smem + p.off_sx);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwc = (blockDim.x >> 5) - kProducerWarps - kKeeperWarps, nct = nwc * 32;   // consumer warps / threads
    const int ns = p.ns, n_ops = p.n_ops;
    const uint32_t inv_grid = p.inv_grid;

    if (tid == 0) {
        for (int i = 0; i < nwc * ns; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        ctl[0] = 0; ctl[2] = 0;
        for (int j = 0; j < kKeeperWarps; ++j) ctl[8 + j] = -1;
        fence_barrier_init();
    }
    // The operation table is read at every hand-over: keep it in shared memory when it fits (a
    // global read costs an L2 round trip).
    const MegaOp* ops = p.ops;
    if (p.off_ops >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(smem + p.off_ops);
        const uint4* src = reinterpret_cast<const uint4*>(p.ops);
        for (int i = tid; i < n_ops * static_cast<int>(sizeof(MegaOp) / 16); i += blockDim.x) dst[i] = src[i];
        ops = reinterpret_cast<const MegaOp*>(smem + p.off_ops);
    }
    __syncthreads();
    // Phase records and epochs.  Warp 0 lists the phase heads in order (plan_decode leaves the
    // length of the phase in the head's flags) and the first operation of every epoch (a head with
    // a barrier in front starts a new epoch, after as many empty ones as it asks for); every thread
    // then fills in the records of some phases, and warp 0 turns the CTA's box counts into running
    // sums.
    if (warp == 0) {
        int nph = 0;
        for (int base = 0; base < n_ops; base += 32) {
            const int i = base + lane;
            const uint32_t len = i < n_ops ? ((ops[i].flags >> kPhaseLenShift) & 7u) : 0u;
            const uint32_t heads = __ballot_sync(0xffffffffu, len != 0);
            const int at = nph + __popc(heads & ((1u << lane) - 1u));
            if (len != 0 && at < p.n_phases) { phases[at].o = static_cast<uint16_t>(i); phases[at].len = static_cast<uint8_t>(len); }
            nph += __popc(heads);
        }
        if (lane == 0) {
            ctl[1] = nph;
            int ne = 0;
            ep_op[ne++] = 0;
            for (int i = 1; i < n_ops && ne <= p.n_epochs; ++i) {
                const uint32_t f = ops[i].flags;
                if (!(f & MOP_BARRIER)) continue;
                const int extra = ((f & MOP_BARRIER2) ? 1 : 0);
                for (int x = 0; x <= extra && ne <= p.n_epochs; ++x) ep_op[ne++] = static_cast<uint16_t>(i);
            }
            if (ne != p.n_epochs) ctl[1] = -1;
            ep_op[p.n_epochs] = static_cast<uint16_t>(n_ops);
        }
    }
    __syncthreads();
    const int n_phases = ctl[1];
    if (n_phases != p.n_phases) {      // the host counted differently: the table is not what it planned
        if (tid == 0) atomicOr(p.err, ERR_BAD_SHAPE);
        return;
    }
    for (int t = tid; t < n_phases; t += blockDim.x) {
        PhaseRec& r = phases[t];
        const int o = r.o, len = r.len;
        uint32_t rows = 0;
        for (int k = 0; k < kMaxPhaseOps; ++k) {
            if (k > 0) r.rb[k - 1] = k < len ? rows : ~0u;
            if (k < len) rows += static_cast<uint32_t>((ops[o + k].N + 31) >> 5);
        }
        r.R = rows;
        const uint32_t gpr = static_cast<uint32_t>(ops[o].K) >> 8;
        r.gpr = static_cast<uint16_t>(gpr);
        const uint32_t u = rows * gpr;   // the launcher refuses lists with u * gridDim >= 2^32
        const uint32_t c0 = grid_share(u, blockIdx.x, inv_grid);
        const uint32_t c1 = blockIdx.x + 1 == gridDim.x ? u : grid_share(u, blockIdx.x + 1, inv_grid);
        r.c0 = c0;
        r.n = c1 - c0;
        r.s0 = 0;
        r.band_lo = r.band_hi = 0;
        if (c1 > c0) {
            const uint32_t full_bands = gpr / kBandGroups, per = rows * kBandGroups;
            const uint32_t b0 = div_u32(c0, per), b1 = div_u32(c1 - 1, per);
            r.band_lo = static_cast<uint8_t>(b0 < full_bands ? b0 : full_bands);
            r.band_hi = static_cast<uint8_t>(b1 < full_bands ? b1 : full_bands);
        }
    }
    __syncthreads();
    if (warp == 0) {
        uint32_t run = 0;
        for (int base = 0; base < n_phases; base += 32) {
            const int i = base + lane;
            const uint32_t n = i < n_phases ? phases[i].n : 0u;
            uint32_t incl = n;
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (i < n_phases) phases[i].s0 = run + incl - n;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();

    if (warp >= nwc + kProducerWarps) {
        const int jp = warp - nwc - kProducerWarps;
        keep_house<MULTI>(p, ops, ep_op, p.n_epochs, ctl, reinterpret_cast<float*>(smem + p.off_jscale) + jp * p.jscale_cap, jp);
        return;
    }
    if (warp >= nwc) {
        produce_boxes(p, ops, phases, n_phases, full, empty, desc, ring, &ctl[0], nwc, warp - nwc, kProducerWarps);
        return;
    }

    // ---- consumer warps ----
    const int ctid = tid, cw = warp;     // the consumers are the CTA's first warps
    float2* pool2 = reinterpret_cast<float2*>(p.pool);
    bool failed = false;                            // this warp gave up on a wait
    int epoch = 0;                                  // the epoch of the current phase
    uint32_t s = static_cast<uint32_t>(cw);       // this warp's next box in the CTA's sequence
    int cj = 0;                                     // its ring stage
    uint32_t cpar = 0;                              // parity of that stage's current use
    for (int ph = 0; ph < n_phases; ++ph) {
        const PhaseRec& rec = phases[ph];
        const int o = rec.o;
        const uint32_t flags = ops[o].flags;
        const int rounds = ph > 0 && (flags & MOP_BARRIER) ? ((flags & MOP_BARRIER2) ? 2 : 1) : 0;
        // Everyone in the CTA is done with the previous phase: its staged activations may be replaced.
        // (Thread 0 samples the abort flag before the barrier, everyone reads the sample after it: the
        // flag can be raised at any moment, and the consumers must all leave at the same point.)
        if (ctid == 0) ctl[4] = ctl[0];
        consumer_sync(nct);
        if (ctl[4]) break;
        if (rounds > 0) {
            epoch += rounds;
            if (ctid == 0) ctl[2] = epoch;    // the housekeeping warp takes over epochs < epoch
            // The accumulators and the slots of this epoch belong to a generation that epoch - G
            // used: wait until the housekeeping warp that cleared it has seen every CTA's clearing
            // published (it has, unless it lags epochs behind).  No fence: the clearing was performed
            // before that warp could see the arrivals, and nothing below is issued before this loop
            // ends.
            const int need = epoch - kFlowGenerations + 1 + kKeeperWarps;
            if (need >= 0) {
                volatile int* done = &ctl[8 + need % kKeeperWarps];
                if (*done < need) {
                    const long long t0 = clock64();
                    while (*done < need) {
                        if (ctl[0] || clock64() - t0 > kWaitClocks) { ctl[0] = 1; break; }
                    }
                }
            }
        }
        if (ops[o].x_epoch) {
            // The input is a result buffer that epoch x_epoch - 1 of this launch wrote: wait for the
            // iteration that stored and published it.
            const int need = static_cast<int>(ops[o].x_epoch);
            volatile int* done = &ctl[8 + need % kKeeperWarps];
            if (*done < need) {
                const long long t0 = clock64();
                while (*done < need) {
                    if (ctl[0] || clock64() - t0 > kWaitClocks) { ctl[0] = 1; break; }
                }
            }
        }
        if (rec.n) {
            stage_bands_flow<MULTI>(ops[o], p, smem, scratch, rec.band_lo, rec.band_hi, nct, &ctl[0]);
        } else {
            consumer_sync(nct);   // keeps the barrier count of stage_bands (one per phase at least)
        }
        const uint32_t send = rec.s0 + rec.n;
        while (s < send && !failed) {
            const int slot = cw + nwc * cj;
            if (!mbar_wait_bounded(&full[slot], cpar)) { failed = true; break; }
            const uint2 d = desc[slot];
            uint32_t w[36];
            {
                const uint4* src = reinterpret_cast<const uint4*>(
                    ring + static_cast<size_t>(slot) * kBoxBytes + static_cast<size_t>(lane) * 144);
#pragma unroll
                for (int v = 0; v < 9; ++v) {
                    const uint4 t = src[v];
                    w[4 * v + 0] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);      // the producer may refill the slot
            if (++cj == ns) { cj = 0; cpar ^= 1u; }
            s += static_cast<uint32_t>(nwc);
            float out[1] = {0.f};
            group_dot_i16<FMT_Q4_0, 1, true>(w, xs, sx2, static_cast<int>(d.y & 0xffffu), 0, 0, 0, out);
            if (static_cast<uint32_t>(lane) < ((d.y >> 16) & 63u)) {
                if (MULTI && (d.y >> 24)) {     // tensor parallel: into every rank's accumulators
                    for (int r = 0; r < p.n_ranks; ++r)
                        red_add_pair_sys(reinterpret_cast<float2*>(p.peer_pool[r]) + d.x + lane, out[0]);
                } else {
                    red_add_pair(pool2 + d.x + lane, out[0]);
                }
            }
        }
        if (__any_sync(0xffffffffu, failed)) {
            failed = true;
            if (lane == 0) { ctl[0] = 1; atomicOr(p.err, ERR_WAIT_TIMEOUT); }
        }
    }
    // all boxes done: hand the last epoch to the housekeeping warp
    consumer_sync(nct);
    if (ctid == 0) ctl[2] = p.n_epochs;
}

inline int align_up(int v, int a) { return (v + a - 1) / a * a; }
inline bool spans_overlap(DecodeSpan a, DecodeSpan b) { return a.lo < b.hi && b.lo < a.hi; }
inline bool span_hits(const DecodeSpan* v, int n, DecodeSpan r) {
    for (int i = 0; i < n; ++i)
        if (spans_overlap(v[i], r)) return true;
    return false;
}

}  // namespace

cudaError_t init_decode_kernel(int smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(decode_q4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_q4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
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

cudaError_t plan_decode(const GemvQArgs* ops, const DecodeTpOp* tp, int n_ops, DecodeSpan* work,
                        MegaOp* table, DecodePlan* plan, size_t pool_capacity_floats, int n_ranks) {
    if (!ops || !work || !table || !plan || n_ops <= 0) return cudaErrorInvalidValue;
    DecodeSpan* reads = work;                 // inputs read since the last barrier (x, gamma, W)
    DecodeSpan* writes = work + 3 * n_ops;    // results written since the last barrier
    DecodeSpan* epoch_of = work + 4 * n_ops;  // .lo = epoch of an operation
    int nr = 0, nw = 0;
    DecodeSpan y_box{~static_cast<uintptr_t>(0), 0};   // bounding interval of every result so far
    auto y_span = [&](int j) {
        const GemvQArgs& b = ops[j];
        const size_t rows = tp && tp[j].y_rows ? static_cast<size_t>(tp[j].y_rows) : static_cast<size_t>(b.N);
        const uintptr_t lo = reinterpret_cast<uintptr_t>(b.Y);
        return DecodeSpan{lo, lo + rows * (b.y_f32 ? 4 : 2)};
    };
    // Pass 1: barriers and epochs, accumulator offsets inside an epoch, hand-over of results.
    // Timing of a result of epoch p: accumulators complete after the barrier that ends p; read
    // from there by operations of epoch p + 1; result buffer written during the wait at the
    // barrier that ends p + 1, hence visible from epoch p + 3; accumulators zeroed at the end of
    // p + 2.  So a reader of the buffer in epoch p + 2, or another writer in epoch p + 1, gets
    // one more (empty) epoch in front of it.
    int epoch = 0;
    size_t in_epoch = 0, worst = 0;         // accumulators of the current epoch, and the largest epoch
    size_t ss_epoch = 0, ss_worst = 0;      // the same for the sums of squares, which get a region of their own
    uint32_t ss_cur = 0;
    for (int i = 0; i < n_ops; ++i) {
        const GemvQArgs& a = ops[i];
        if (a.fmt != FMT_Q4_0 || a.M != 1 || a.N <= 0 || a.K <= 0 || a.K % 256 != 0 || !a.W || !a.X || !a.Y)
            return cudaErrorNotSupported;
        if (a.K / 256 > kBandGroups * kMaxBands) return cudaErrorNotSupported;
        if ((reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.X) |
             reinterpret_cast<uintptr_t>(a.gamma)) & 15u)
            return cudaErrorNotSupported;
        if (reinterpret_cast<uintptr_t>(a.Y) & (a.y_f32 ? 3u : 1u)) return cudaErrorNotSupported;
        const size_t xs = a.x_f32 ? 4 : 2;
        const uintptr_t xl = reinterpret_cast<uintptr_t>(a.X), gl = reinterpret_cast<uintptr_t>(a.gamma);
        const uintptr_t wl = reinterpret_cast<uintptr_t>(a.W);
        const DecodeSpan rx{xl, xl + a.K * xs};
        const DecodeSpan rg{gl, gl + (a.gamma ? a.K * xs : 0)};
        const DecodeSpan rw{wl, wl + static_cast<size_t>(a.N) * (a.K / 32) * 18};
        const DecodeSpan ry = y_span(i);
        const uint32_t y_rows = tp && tp[i].y_rows ? static_cast<uint32_t>(tp[i].y_rows) : static_cast<uint32_t>(a.N);
        const uint32_t y_row0 = tp ? static_cast<uint32_t>(tp[i].y_row0) : 0u;
        if (static_cast<unsigned long long>(y_row0) + a.N > y_rows) return cudaErrorInvalidValue;
        if (y_rows >= (1u << 24)) return cudaErrorNotSupported;
        // Weights are fetched ahead of every barrier, and gamma is read while earlier results may
        // still be on their way to their buffers: neither may be an earlier result.
        if (spans_overlap(rw, y_box) || (a.gamma && spans_overlap(rg, y_box))) {
            for (int j = 0; j < i; ++j) {
                const DecodeSpan yj = y_span(j);
                if (spans_overlap(rw, yj) || (a.gamma && spans_overlap(rg, yj))) return cudaErrorNotSupported;
            }
        }
        // A result that is overwritten - same buffer, same extent - before anything reads it never
        // needs to reach its buffer: the earlier operation is computed but not stored, and the two
        // need no barrier between them (a benchmark loop that sends every projection of every
        // layer to one scratch vector is the common case).
        auto same_span = [](DecodeSpan a, DecodeSpan b) { return a.lo == b.lo && a.hi == b.hi; };
        auto dead_until = [&](int j) {      // nothing in (j, i) reads operation j's result
            const DecodeSpan yj = y_span(j);
            for (int t = j + 1; t < i; ++t) {
                const uintptr_t tl = reinterpret_cast<uintptr_t>(ops[t].X);
                if (spans_overlap(DecodeSpan{tl, tl + ops[t].K * static_cast<size_t>(ops[t].x_f32 ? 4 : 2)}, yj)) return false;
            }
            return !spans_overlap(rx, yj);
        };
        bool waw_only = i > 0 && !span_hits(writes, nw, rx) && !span_hits(reads, nr, ry);
        if (waw_only) {
            for (int w = 0; w < nw && waw_only; ++w)
                if (spans_overlap(writes[w], ry) &&
                    !(same_span(writes[w], ry) && ops[i - nw + w].y_f32 == a.y_f32 && dead_until(i - nw + w)))
                    waw_only = false;
        }
        int nbar = (i > 0 && !waw_only &&
                    (span_hits(writes, nw, rx) || span_hits(writes, nw, ry) || span_hits(reads, nr, ry))) ? 1 : 0;
        if (waw_only)
            for (int w = 0; w < nw; ++w)
                if (spans_overlap(writes[w], ry)) table[i - nw + w].flags |= MOP_NO_STORE;
        int producer = -1;
        if (i > 0 && (spans_overlap(rx, y_box) || spans_overlap(ry, y_box))) {
            for (int round = 0; round < 3; ++round) {
                const int e_i = epoch + nbar;
                bool bump = false, seen_x = false, seen_y = false;
                producer = -1;
                for (int j = i - 1; j >= 0 && !(seen_x && seen_y); --j) {
                    const int d = e_i - static_cast<int>(epoch_of[j].lo);
                    if (d > 2) break;
                    const DecodeSpan yj = y_span(j);
                    if (!seen_x && spans_overlap(rx, yj)) {        // latest writer of what this one reads
                        seen_x = true;
                        if (d == 2) bump = true;
                        else if (d == 1) producer = j;
                    }
                    if (!seen_y && spans_overlap(ry, yj)) {        // latest writer of what this one writes
                        seen_y = true;
                        if (d == 1) {
                            if (same_span(ry, yj) && ops[j].y_f32 == a.y_f32 && dead_until(j)) table[j].flags |= MOP_NO_STORE;
                            else bump = true;
                        }
                    }
                }
                if (!bump) break;
                ++nbar;
            }
        }
        if (nbar > 2) return cudaErrorNotSupported;
        if (nbar > 0) {
            nr = nw = 0;
            epoch += nbar;
            in_epoch = 0;
            ss_epoch = 0;
        }
        reads[nr++] = rx;
        if (a.gamma) reads[nr++] = rg;
        reads[nr++] = rw;
        writes[nw++] = ry;
        y_box.lo = ry.lo < y_box.lo ? ry.lo : y_box.lo;
        y_box.hi = ry.hi > y_box.hi ? ry.hi : y_box.hi;
        epoch_of[i].lo = static_cast<uintptr_t>(epoch);
        MegaOp& m = table[i];
        m.W = a.W; m.X = a.X; m.Y = a.Y; m.gamma = a.gamma; m.N = a.N; m.K = a.K; m.eps = a.eps;
        m.flags = (nbar > 0 ? MOP_BARRIER : 0u) | (nbar > 1 ? MOP_BARRIER2 : 0u) | (a.x_f32 ? MOP_X_F32 : 0u) |
                  (a.y_f32 ? MOP_Y_F32 : 0u) | (a.gamma ? MOP_FUSED : 0u) | (tp && tp[i].peers ? MOP_PEERS : 0u);
        bool restage = true;
        if (i > 0 && nbar == 0) {
            const GemvQArgs& b = ops[i - 1];
            restage = !(b.X == a.X && b.gamma == a.gamma && b.K == a.K && b.x_f32 == a.x_f32);
        }
        if (restage) m.flags |= MOP_RESTAGE;
        m.y_row0 = y_row0;
        m.y_rows = y_rows;
        m.acc_off = static_cast<uint32_t>(in_epoch);
        const size_t layout = tp && tp[i].layout_rows > static_cast<int>(y_rows) ? static_cast<size_t>(tp[i].layout_rows) : y_rows;
        in_epoch += (layout + 31) & ~static_cast<size_t>(31);
        m.ss_off = 0;
        if (a.gamma) {
            if (restage) {      // operations that share a staged row share its sums of squares
                ss_cur = static_cast<uint32_t>(ss_epoch);
                ss_epoch += kMaxBands;
            }
            m.ss_off = ss_cur;
        }
        m.xacc_off = -1;
        m.xss_off = -1;
        m.xss_k = 0;
        m.xss_eps = 0.f;
        m.x_epoch = 0;
        m.pad = 0;
        if (producer < 0 && i > 0 && spans_overlap(rx, y_box)) {
            // the input comes from memory that this list wrote earlier (three epochs ago or more)
            for (int j = i - 1; j >= 0; --j)
                if (spans_overlap(rx, y_span(j))) { m.x_epoch = static_cast<uint32_t>(epoch_of[j].lo) + 1u; break; }
        }
        if (producer >= 0) {
            // the result of the epoch before: taken from its accumulators, if it lies cleanly inside
            const GemvQArgs& b = ops[producer];
            const DecodeSpan yj = y_span(producer);
            const size_t es = b.y_f32 ? 4 : 2;
            const bool contained = rx.lo >= yj.lo && rx.hi <= yj.hi && b.y_f32 == a.x_f32 &&
                                   (rx.lo - yj.lo) % (4 * es) == 0;
            if (!contained) return cudaErrorNotSupported;
            m.xacc_off = producer;                                         // resolved in pass 2
            m.xss_k = static_cast<int32_t>((rx.lo - yj.lo) / es);         // first element, for now
            if (!b.y_f32) m.flags |= MOP_XACC_F16;
        }
        worst = in_epoch > worst ? in_epoch : worst;
        ss_worst = ss_epoch > ss_worst ? ss_epoch : ss_worst;
        if (worst + ss_worst > (1u << 28)) return cudaErrorNotSupported;
    }
    // A generation: accumulators first, then the sums of squares.  The two never share an
    // address: accumulators are zeroed before reuse, the sums are simply overwritten.
    const size_t gen = worst + ss_worst;
    // The accumulators of an epoch are cleared by a warp that trails the computation, and the
    // clearing is confirmed some epochs after that; more generations than that needs let the
    // trailing warps lag without holding anybody up.  Every accumulator is a pair (sum, number of
    // partial sums added).
    const size_t gens = kFlowGenerations;
    const size_t per_acc = 2;
    if (pool_capacity_floats && gens * gen * per_acc > pool_capacity_floats) return cudaErrorNotSupported;
    // Pass 2: place the accumulators and the sums of squares (generation = epoch mod 3).
    int barriers = 1;   // the trailing one
    int run_ops = 0, max_epoch_ops = 0;
    for (int i = 0; i < n_ops; ++i) {
        MegaOp& m = table[i];
        const uint32_t base = static_cast<uint32_t>((epoch_of[i].lo % gens) * gen);
        m.acc_off += base;
        if (m.flags & MOP_FUSED) m.ss_off += base + static_cast<uint32_t>(worst);
        // partial sums per row: one per box; summed over the ranks when they split K among them
        m.expect = tp && tp[i].expect > 0 ? static_cast<uint32_t>(tp[i].expect) : static_cast<uint32_t>(m.K / 256);
        m.xexpect = 0;
        if (m.xacc_off >= 0) {
            const MegaOp& pr = table[m.xacc_off];      // earlier in the list: already placed
            m.xexpect = pr.expect;
            m.xacc_off = static_cast<int32_t>(pr.acc_off + static_cast<uint32_t>(m.xss_k));
            m.xss_k = 0;
            if (pr.flags & MOP_FUSED) {
                m.xss_off = static_cast<int32_t>(pr.ss_off);
                m.xss_k = pr.K;
                m.xss_eps = pr.eps;
            }
        }
        if (m.flags & MOP_BARRIER) { barriers += (m.flags & MOP_BARRIER2) ? 2 : 1; run_ops = 0; }
        ++run_ops;
        max_epoch_ops = run_ops > max_epoch_ops ? run_ops : max_epoch_ops;
    }
    plan->max_epoch_ops = max_epoch_ops;
    for (int i = 0; i < n_ops;) {          // phases: runs that share their staged input, at most kMaxPhaseOps long
        int e = i + 1;
        while (e < n_ops && e - i < kMaxPhaseOps && !(table[e].flags & (MOP_BARRIER | MOP_RESTAGE))) ++e;
        table[i].flags |= static_cast<uint32_t>(e - i) << kPhaseLenShift;
        i = e;
    }
    plan->n_ops = n_ops;
    plan->epochs = barriers;
    // each of a CTA's housekeeping warps arrives on its own counter for every kKeeperWarps-th epoch and
    // once more at the end; tensor parallel: and a last time, so that no rank leaves early
    plan->barriers = (barriers + kKeeperWarps) / kKeeperWarps + (n_ranks > 1 ? 1 : 0);
    plan->pool_floats = gens * gen * per_acc;
    return cudaSuccess;
}

cudaError_t launch_decode(const MegaOp* host_ops, const DecodePlan& plan, const DecodeDevice& dev,
                          const LaunchEnv& env, cudaStream_t stream) {
    const int n_ops = plan.n_ops;
    if (n_ops <= 0 || !dev.ops || !dev.maps || !dev.pool || !dev.counter) return cudaErrorInvalidValue;
    if (dev.n_ranks < 1 || dev.n_ranks > kDecodeMaxRanks) return cudaErrorInvalidValue;
    static const int want_warps = [] {
        const char* v = std::getenv("TC_DECODE_WARPS");
        const int n = v ? std::atoi(v) : 16;
        return (n == 8 || n == 16) ? n : 16;
    }();
    const int grid = env.sm_count;
    if (n_ops >= 65536) return cudaErrorNotSupported;
    int k_max = 0, n_phases = 0;
    {   // box numbering is 32-bit: the boxes of a phase times the grid must stay below 2^32
        unsigned long long run = 0;
        for (int i = 0; i < n_ops; ++i) {
            const bool head = ((host_ops[i].flags >> kPhaseLenShift) & 7u) != 0;
            if (head) { run = 0; ++n_phases; }
            run += static_cast<unsigned long long>((host_ops[i].N + 31) / 32) * (host_ops[i].K / 256);
            if (run * static_cast<unsigned>(grid) >= (1ull << 32)) return cudaErrorNotSupported;
            if (host_ops[i].K / 256 >= 65536) return cudaErrorNotSupported;
            k_max = host_ops[i].K > k_max ? host_ops[i].K : k_max;
        }
    }
    const int optin = env.smem_optin > 0 ? env.smem_optin : 232448;
    DecodeParams p;
    std::memset(&p, 0, sizeof(p));
    p.ops = dev.ops; p.maps = dev.maps; p.n_ops = n_ops; p.pool = dev.pool;
    p.counter = dev.counter; p.base = dev.base; p.err = env.err_word;
    p.n_ranks = dev.n_ranks; p.rank = dev.rank;
    p.n_phases = n_phases;
    p.n_epochs = plan.epochs;
    p.inv_grid = static_cast<uint32_t>(((1ull << 32) + grid - 1) / grid);
    for (int r = 0; r < dev.n_ranks; ++r) { p.peer_pool[r] = dev.peer_pool[r]; p.peer_counter[r] = dev.peer_counter[r]; }
    int off = 16 * kDecodeMaxSlots + 128 + 64;   // full / empty barriers, scratch, control words (16 ints)
    p.off_desc = off;
    off += 8 * kDecodeMaxSlots;
    p.off_phases = off;
    off += align_up(n_phases * static_cast<int>(sizeof(PhaseRec)), 16);
    p.off_epochs = off;
    off += align_up((plan.epochs + 1) * 2, 16);
    p.off_jscale = off;
    p.jscale_cap = plan.max_epoch_ops < 256 ? plan.max_epoch_ops : 256;
    off += align_up(kKeeperWarps * p.jscale_cap * 4, 16);
    p.off_sx = off;
    off += align_up((k_max / 32) * 8, 16);
    off = align_up(off, 128);
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
            if (off + warps * cand * kBoxBytes <= optin - 1024) { ns = cand; break; }
    if (ns == 0) return cudaErrorNotSupported;
    warps += 8;   // undo the loop's last decrement
    p.ns = ns;
    const size_t smem = static_cast<size_t>(off) + static_cast<size_t>(warps) * ns * kBoxBytes;
    void* args[] = {&p};
    // `warps` consumer warps, the producer warps and the housekeeping warps
    const void* kernel = dev.n_ranks > 1 ? reinterpret_cast<const void*>(decode_q4_kernel<true>)
                                         : reinterpret_cast<const void*>(decode_q4_kernel<false>);
    return cudaLaunchCooperativeKernel(kernel, dim3(grid),
                                       dim3((warps + kProducerWarps + kKeeperWarps) * 32), args, smem, stream);
}

// ---------------------------------------------------------------------------------------
// Decode launch for callers that must not allocate.
//
// The persistent decode kernel needs scratch in global memory: the operation table the CTAs walk,
// one tensor map per operation, the arrival counter of its grid barrier and the fp32 accumulators
// its results are summed in.  The library normally keeps them in buffers it allocates on first
// use.  Some callers cannot have that: an inference server that has handed every byte of HBM to
// weights and KV cache at start-up, or a decode loop in which a cudaMalloc (which synchronises the
// whole device) is not acceptable at any point.  For them the same kernel is reachable with its
// scratch in the fixed array below, which is part of the library image on every GPU that loads it
// and is never freed.
//
// Layout: [0,256) arrival counter (first 8 bytes used) | operation table | tensor maps |
// accumulators.  Hence at most kDecodeStaticMaxOps operations per call and
// kDecodeStaticPoolFloats accumulators.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticTableOffset = 256;
constexpr size_t kStaticMapsOffset = kStaticTableOffset + kDecodeStaticMaxOps * sizeof(MegaOp);
constexpr size_t kStaticPoolOffset = kStaticMapsOffset + kDecodeStaticMaxOps * kDecodeMapBytes;
constexpr size_t kStaticBytes = kStaticPoolOffset + kDecodeStaticPoolFloats * sizeof(float);
static_assert(kStaticPoolOffset % 256 == 0, "accumulators start on a 256-byte boundary");
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticBytes];

namespace {
constexpr int kMaxDevices = 64;
// Host-side state of the static launch site, one per device: the array's device address and the
// tensor maps encoded for the previous call (re-encoded only when weights, shapes or their order
// change; encoding costs about a microsecond each).  Guarded by one mutex: calls from several
// host threads are serialised here, whatever device they target.
struct StaticSite {
    unsigned char* addr = nullptr;
    int maps_n = 0;
    MegaOp maps_for[kDecodeStaticMaxOps];
    alignas(64) unsigned char maps[kDecodeStaticMaxOps * kDecodeMapBytes];
};
std::mutex g_static_mutex;
StaticSite* g_static_site[kMaxDevices] = {nullptr};
StaticSite g_static_first;     // device 0 (or whichever comes first) needs no host allocation

// The array's name is only a handle on the host; kernels need its device address, which differs
// per device and is looked up once per device with that device current.
cudaError_t static_site_for_current_device(StaticSite** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (g_static_site[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
        if (e != cudaSuccess) return e;
        // host bookkeeping (plain new, no device allocation) for the second and later devices
        StaticSite* s = g_static_first.addr == nullptr ? &g_static_first : new (std::nothrow) StaticSite();
        if (!s) return cudaErrorMemoryAllocation;
        s->addr = static_cast<unsigned char*>(ptr);
        g_static_site[dev] = s;
    }
    *out = g_static_site[dev];
    return cudaSuccess;
}
}  // namespace

// ops: host array of n_ops operations in execution order (GemvQArgs with M == 1, Q4_0).  Plans the
// table on the stack, copies it into the static scratch together with the operations' tensor
// maps, clears the arrival counter and the accumulators the table uses, and launches.  No device
// allocation of any kind.
cudaError_t launch_gemv_q4_decode_static(const GemvQArgs* ops, int n_ops, const LaunchEnv& env,
                                         cudaStream_t stream) {
    if (n_ops <= 0 || n_ops > kDecodeStaticMaxOps) return cudaErrorNotSupported;
    MegaOp table[kDecodeStaticMaxOps];
    DecodeSpan work[5 * kDecodeStaticMaxOps];
    DecodePlan plan;
    cudaError_t e = plan_decode(ops, nullptr, n_ops, work, table, &plan, kDecodeStaticPoolFloats);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSite* site = nullptr;
    e = static_site_for_current_device(&site);
    if (e != cudaSuccess) return e;
    unsigned char* scratch = site->addr;
    // The array keeps whatever the previous call left.  The counter must start from zero; the
    // accumulators are all zero after a call that ran to its end, but not after one that gave up
    // on a bounded wait, so the part this table uses is cleared as well; the table and the maps
    // are overwritten.  (The host table lives on this stack frame: the copy from pageable memory
    // has consumed it when cudaMemcpyAsync returns.)
    e = cudaMemsetAsync(scratch, 0, 256, stream);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(scratch + kStaticPoolOffset, 0, plan.pool_floats * sizeof(float), stream);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(scratch + kStaticTableOffset, table, static_cast<size_t>(n_ops) * sizeof(MegaOp),
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
    bool fresh = site->maps_n == n_ops;
    for (int i = 0; i < n_ops && fresh; ++i)
        fresh = site->maps_for[i].W == table[i].W && site->maps_for[i].N == table[i].N &&
                site->maps_for[i].K == table[i].K;
    if (!fresh) {
        e = encode_decode_maps(table, n_ops, site->maps);
        if (e != cudaSuccess) { site->maps_n = 0; return e; }
        for (int i = 0; i < n_ops; ++i) site->maps_for[i] = table[i];
        site->maps_n = n_ops;
    }
    e = cudaMemcpyAsync(scratch + kStaticMapsOffset, site->maps, static_cast<size_t>(n_ops) * kDecodeMapBytes,
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
    DecodeDevice dev;
    dev.ops = reinterpret_cast<const MegaOp*>(scratch + kStaticTableOffset);
    dev.maps = scratch + kStaticMapsOffset;
    dev.pool = reinterpret_cast<float*>(scratch + kStaticPoolOffset);
    dev.counter = reinterpret_cast<unsigned long long*>(scratch);
    dev.base = 0;
    return launch_decode(table, plan, dev, env, stream);
}

}  // namespace tcb
