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
// Arithmetic (gemv_common.cuh): activations are staged once per CTA as int16 with one fp32
// scale per 32-element block; a block's dot product is exact integer arithmetic on the dp2a unit
// and one fused multiply-add applies d_w * s_x, with the zero point (-8 for Q4_0's unsigned
// nibbles) removed through the block's precomputed activation sum.
//
// Two geometries.  Streaming kernel: a lane per K group; activations (M <= 4 rows per pass) live
// in shared memory in a chunk-transposed layout so that the 32 lanes of a warp, which work on 32
// consecutive groups, read consecutive 16-byte chunks; per-lane partial sums are combined with a
// segmented warp-shuffle reduction (a warp's 32 groups may span several weight rows) and added to
// per-row accumulators in shared memory.  Box kernel (default): a lane per weight row of a
// 32-row x one-group box fetched by a tiled TMA copy, activations read by broadcast.
//
// With programmatic dependent launch the kernel starts its weight stream before waiting for
// the previous kernel in the stream, so consecutive GEMVs of a decode step overlap their
// fill/drain phases.  Every mbarrier wait is bounded; on expiry the kernel records
// ERR_WAIT_TIMEOUT, drains its outstanding copies (again bounded) and exits.
#include "gemv_common.cuh"
#include "tensor_map.h"

#include <cstdlib>

namespace tcb {
cudaError_t init_tc_kernels(int smem_optin);
cudaError_t launch_gemv_q4_tc(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                              const char** name);
cudaError_t init_decode_kernel(int smem_optin);
namespace {


// ---------------------------------------------------------------------------------------
// The streaming kernel.
// ---------------------------------------------------------------------------------------
template <int FMT, int MB>
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
    stage_activations_i16<MB>(p, smem, FMT == FMT_Q4_0 ? 8 : 0, red_scratch);

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
            group_dot_i16<FMT, MB>(w, xs, reinterpret_cast<const float2*>(sx), kg, gpr, p.K, p.nb, out);
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
        group_dot_i16<FMT, MB, true>(w, xs, sx2, kg, gpr, p.K, p.nb, out);
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
StreamPlan plan_stream(const GemvQArgs& a, int mb, const LaunchEnv& env) {
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
    off += align_up(mb * a.K * 2, 128);
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
    return pl;
}

template <int FMT>
cudaError_t launch_stream_mb(int mb, const StreamPlan& pl, cudaStream_t st, bool pdl) {
    const dim3 grid(pl.grid), block(pl.warps * 32);
    switch (mb) {
        case 1: return launch_with_attrs(gemv_q_stream_kernel<FMT, 1>, grid, block, pl.smem, st, pdl, pl.p);
        case 2: return launch_with_attrs(gemv_q_stream_kernel<FMT, 2>, grid, block, pl.smem, st, pdl, pl.p);
        case 3: return launch_with_attrs(gemv_q_stream_kernel<FMT, 3>, grid, block, pl.smem, st, pdl, pl.p);
        default: return launch_with_attrs(gemv_q_stream_kernel<FMT, 4>, grid, block, pl.smem, st, pdl, pl.p);
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

cudaError_t init_gemv_kernels(int smem_optin) {
    cudaError_t e = init_tc_kernels(smem_optin);
    if (e == cudaSuccess) e = init_gemm_tc_kernel(smem_optin);
    if (e != cudaSuccess) return e;
    e = init_decode_kernel(smem_optin);
    if (e != cudaSuccess) return e;
#define TCB_SETB(FMT, MB)                                                         \
    e = set_smem(gemv_q_box_kernel<FMT, MB>, smem_optin);                         \
    if (e != cudaSuccess) return e;
    TCB_SETB(FMT_Q4_0, 1) TCB_SETB(FMT_Q4_0, 2) TCB_SETB(FMT_Q4_0, 3) TCB_SETB(FMT_Q4_0, 4)
    TCB_SETB(FMT_Q8_0, 1) TCB_SETB(FMT_Q8_0, 2) TCB_SETB(FMT_Q8_0, 3) TCB_SETB(FMT_Q8_0, 4)
#undef TCB_SETB
#define TCB_SET(FMT, MB)                                                          \
    e = set_smem(gemv_q_stream_kernel<FMT, MB>, smem_optin);                      \
    if (e != cudaSuccess) return e;
    TCB_SET(FMT_Q4_0, 1) TCB_SET(FMT_Q4_0, 2) TCB_SET(FMT_Q4_0, 3) TCB_SET(FMT_Q4_0, 4)
    TCB_SET(FMT_Q8_0, 1) TCB_SET(FMT_Q8_0, 2) TCB_SET(FMT_Q8_0, 3) TCB_SET(FMT_Q8_0, 4)
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

    // Batched decode: the tcgen05 kernel reads the weights once for up to 32 activation rows.
    // It rounds dequantised weights to fp16, which only the fp16-activation bound allows.
    const bool want_tc = env.variant == VARIANT_TC ||
                         (env.variant == VARIANT_AUTO && batched_tc_rows(a.M, a.N, a.K));
    // The fused RMSNorm form takes it too, behind a pass that normalises the rows into the stream's
    // scratch as fp16 (one more rounding, inside the same bound).
    const size_t slab_rows = a.M < 32 ? a.M : 32;
    const size_t norm_need = slab_rows * static_cast<size_t>(a.K) * 2 + slab_rows * 4;
    const bool fuse_tc = fuse && a.norm_scratch && a.norm_scratch_bytes >= norm_need && a.K % 256 == 0;
    // Prefill-sized calls: the weights are dequantised once into the stream's scratch (fp16, the same
    // rounding as the kernel below applies on the fly) and multiplied on the tensor cores as a GEMM
    // with B transposed; Q8_0 too.  fp16 activations and results only (the rounding of the weights is
    // inside their bound, not inside the fp32 one).
    if (env.variant == VARIANT_AUTO && a.M >= gemm_min_rows(a.fmt) && !a.x_f32 && !a.y_f32 && a.dequant_scratch &&
        a.dequant_scratch_bytes >= static_cast<size_t>(a.N) * a.K * 2 && a.K % 32 == 0 &&
        (!fuse || (a.norm_scratch && a.norm_scratch_bytes >= static_cast<size_t>(a.M) * a.K * 2 + static_cast<size_t>(a.M) * 4))) {
        cudaError_t e = launch_dequantize(a.W, a.dequant_scratch, a.fmt, a.N, a.K, stream);
        const void* x = a.X;
        int n_launch = 1;
        if (e == cudaSuccess && fuse) {
            float* rstd = reinterpret_cast<float*>(static_cast<uint8_t*>(a.norm_scratch) + static_cast<size_t>(a.M) * a.K * 2);
            e = launch_norm_forward(a.X, a.gamma, nullptr, a.norm_scratch, nullptr, rstd, a.M, a.K, a.eps, stream);
            x = a.norm_scratch;
            ++n_launch;
        }
        if (e == cudaSuccess) {
            e = launch_gemm_f16_tc(x, a.dequant_scratch, a.Y, a.M, a.N, a.K, a.K, a.K, a.N, true, 1.0f, 0.0f, env, stream);
            ++n_launch;
        }
        if (e == cudaSuccess) {
            if (launches) *launches += n_launch;
            if (name) *name = a.fmt == FMT_Q4_0 ? "q4_0_dequant_gemm_tcgen05_sm100" : "q8_0_dequant_gemm_tcgen05_sm100";
            return cudaSuccess;
        }
        if (e != cudaErrorNotSupported) return e;
        (void)cudaGetLastError();
    }
    if (want_tc && a.fmt == FMT_Q4_0 && !a.x_f32 && (!fuse || fuse_tc)) {
        bool done = true;
        for (int m0 = 0; m0 < a.M; m0 += 32) {
            GemvQArgs s = a;
            s.M = (a.M - m0) < 32 ? (a.M - m0) : 32;
            s.X = static_cast<const uint8_t*>(a.X) + static_cast<size_t>(m0) * a.K * xsz;
            s.Y = static_cast<uint8_t*>(a.Y) + static_cast<size_t>(m0) * a.N * ysz;
            if (fuse) {
                float* rstd = reinterpret_cast<float*>(static_cast<uint8_t*>(a.norm_scratch) + slab_rows * static_cast<size_t>(a.K) * 2);
                const cudaError_t ne = launch_norm_forward(s.X, a.gamma, nullptr, a.norm_scratch, nullptr, rstd, s.M, a.K,
                                                           a.eps, stream);
                if (ne != cudaSuccess) { err = ne; break; }
                ++count;
                s.X = a.norm_scratch;
                s.gamma = nullptr;
            }
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

    // Up to kMaxMB activation rows per pass on the integer dot-product kernels.
    for (int m0 = 0; m0 < a.M && err == cudaSuccess; m0 += kMaxMB) {
        const int mb = (a.M - m0) < kMaxMB ? (a.M - m0) : kMaxMB;
        GemvQArgs s = a;
        s.X = static_cast<const uint8_t*>(a.X) + static_cast<size_t>(m0) * a.K * xsz;
        s.Y = static_cast<uint8_t*>(a.Y) + static_cast<size_t>(m0) * a.N * ysz;
        s.M = mb;
        StreamPlan pl;
        if (env.variant != VARIANT_GENERIC && env.variant != VARIANT_STREAM) {
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
        if (env.variant != VARIANT_GENERIC) pl = plan_stream(s, mb, env);
        if (pl.ok) {
            pl.p.x_src_f16 = a.x_f32 ? 0 : 1;
            err = a.fmt == FMT_Q4_0 ? launch_stream_mb<FMT_Q4_0>(mb, pl, stream, env.pdl)
                                    : launch_stream_mb<FMT_Q8_0>(mb, pl, stream, env.pdl);
            used = a.fmt == FMT_Q4_0 ? "q4_0_gemv_stream_sm100" : "q8_0_gemv_stream_sm100";
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
}  // namespace tcb
