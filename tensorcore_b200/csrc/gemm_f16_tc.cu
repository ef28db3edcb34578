// Dense fp16 / bf16 GEMM on the sm_100a tensor cores: C[M,N] = alpha * A[M,K] . op(B) + beta * C, 16-bit
// storage, fp32 accumulation - the case of tc_gemm that the fused-norm callers and a prefill of
// dequantised weights use (include/tensorcore/gemm.h:16-58; arithmetic lib/ops/gemm_cpu.cpp:544-568,
// which adds the products in k order; here the tensor core's order, same fp32 accumulation).
//
//   * One CTA per SM walks the 128 x BN tiles of C (BN = 128 or 256), each over the whole K, 64 at a
//     time, through a ring of four stages (16 KB of A + BN * 128 bytes of B each) that keeps running
//     across tiles; two accumulators in tensor memory, so that one tile is read out and stored while
//     the next one's MMAs run.
//   * Operands reach shared memory by tiled TMA copies of 128-byte rows written with the 128-byte
//     swizzle, the layout the MMA's shared-memory descriptors read directly:
//       - A ([M][K]) and a transposed B ([N][K]) are K-major: a box of 64 k x 128 (or BN) rows;
//         8-row groups 1024 bytes apart, a K step of 16 elements 32 bytes further along the row.
//       - B as given ([K][N], N contiguous) is MN-major: boxes of 64 n x 64 k, one per 64 columns,
//         8192 bytes apart; 8 k are 1024 bytes, a K step of 16 is 2048 bytes.  A transposed
//         ([K][M]) is loaded the same way.
//     (Which of the descriptor's two strides is which was settled on the device: for the swizzled
//     MN-major form the first is the stride along N, the second the one along K; for the K-major
//     form the second is the stride between 8-row groups and the first is not used.)
//   * One thread issues tcgen05.mma (M128 x N{128,256} x K16, kind::f16, both operands from shared
//     memory) into BN columns of tensor memory; tcgen05.commit hands the stage back to the producer.
//   * Four warps read the accumulator (one TMEM lane = one row of the tile per thread), apply
//     alpha and beta and store fp16.
// Rows and columns past M, N and K are zero-filled by TMA and masked at the store.  Every wait is
// bounded: it sets the error word and lets the kernel end.
#include "kernels.h"
#include "sm100_prims.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tcb {
namespace {

using namespace sm100;

constexpr int kBM = 128, kBK = 64;
constexpr int kMaxStages = 12;   // the ring is as deep as shared memory allows, up to this
constexpr int kAStage = kBM * kBK * 2;
constexpr int kGemmThreads = 6 * 32;          // producer, MMA issuer, four epilogue warps
constexpr int kGemmBarBytes = 1024;
constexpr uint32_t kSwizzle128 = 2;           // layout type of the shared-memory descriptor

struct GemmParams {
    __half* C;
    uint32_t* err;
    int M, N, K, ldc;
    float alpha, beta;
    int b_kmajor;      // B was given transposed ([N][K])
    int a_mnmajor;     // A was given transposed ([K][M])
    int bf16;          // operands and result are bfloat16 (else binary16)
    // Bytes one stage's copy of A delivers.  With fewer than 128 rows of A (given row-major) the box
    // holds only the rows there are, rounded up to the 8-row swizzle atom: the tile's other rows stay
    // whatever shared memory held, and feed accumulator rows that the epilogue never stores.
    uint32_t a_tx;
    uint32_t a_stage;  // bytes between the stages of the A ring (a_tx rounded to the 1024-byte swizzle atom)
    int stages;        // ring depth: a stage's copy takes about 1.4 us to land, so a call that streams B
                       // with few rows of A needs many stages in flight to use the memory system
};

struct GemmBars {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];     // MMA issuer -> epilogue warps, per accumulator
    uint64_t acc_empty[2];    // epilogue warps -> MMA issuer
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(GemmBars) <= kGemmBarBytes, "barrier block too large");

// Shared-memory operand descriptor with a layout type; strides in bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    return smem_desc_kmajor(saddr, lbo, sbo) | (static_cast<uint64_t>(layout) << 61);
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
    constexpr int kBStage = BN * kBK * 2;
    extern __shared__ __align__(1024) uint8_t smem[];
    GemmBars* bars = reinterpret_cast<GemmBars*>(smem);
    volatile int* abort_flag = &bars->abort_flag;
    uint8_t* a_ring = smem + kGemmBarBytes;
    const int stages = p.stages;
    const uint32_t a_stage = p.a_stage;
    uint8_t* b_ring = a_ring + stages * a_stage;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ksteps = (p.K + kBK - 1) / kBK;
    // Tiles of C, numbered column-block-major (the CTAs running at the same time share a block of B's
    // columns and walk down A); CTA c takes tiles c, c + gridDim.x, ...
    const int tiles_m = (p.M + kBM - 1) / kBM, tiles_n = (p.N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;

    if (tid == 0) {
        for (int i = 0; i < stages; ++i) { bar_init(&bars->full[i], 1); bar_init(&bars->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { bar_init(&bars->acc_full[i], 1); bar_init(&bars->acc_empty[i], 4); }
        bar_init(&bars->drain, 1);
        bars->abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&amap);
        prefetch_tensormap(&bmap);
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, 2 * BN);     // two accumulators: a tile's epilogue overlaps the next tile's MMAs
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0, s = 0;
            uint32_t par = 0;
            for (int t = blockIdx.x; t < n_tiles && !failed; t += gridDim.x) {
                const int m0 = (t % tiles_m) * kBM, n0 = (t / tiles_m) * BN;
                for (int ks = 0; ks < ksteps; ++ks, ++issued, s = (s + 1 == stages ? 0 : s + 1), par ^= (s == 0 ? 1u : 0u)) {
                    if (!bar_wait(&bars->empty[s], par ^ 1u, abort_flag)) { failed = true; break; }
                    bar_expect_tx(&bars->full[s], p.a_tx + kBStage);
                    if (p.a_mnmajor) {       // [K][M]: two boxes of 64 m x 64 k, like B as given
                        tensor_load_2d(a_ring + s * a_stage, &amap, m0, ks * kBK, &bars->full[s]);
                        tensor_load_2d(a_ring + s * a_stage + 8192, &amap, m0 + 64, ks * kBK, &bars->full[s]);
                    } else {
                        tensor_load_2d(a_ring + s * a_stage, &amap, ks * kBK, m0, &bars->full[s]);
                    }
                    if (p.b_kmajor) {
                        tensor_load_2d(b_ring + s * kBStage, &bmap, ks * kBK, n0, &bars->full[s]);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tensor_load_2d(b_ring + s * kBStage + c * 8192, &bmap, n0 + 64 * c, ks * kBK, &bars->full[s]);
                    }
                }
            }
            if (failed || *abort_flag) {
                // Let copies already in flight land before the CTA's shared memory is released.
                const int first = issued > stages ? issued - stages : 0;
                for (int c = first; c < issued; ++c)
                    bar_wait(&bars->full[c % stages], static_cast<uint32_t>(c / stages) & 1u, nullptr, 100000000LL);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // bit 16: B is MN-major; bits 7-9 and 10-12: operand formats (0 binary16, 1 bfloat16)
            const uint32_t idesc = idesc_f16_f32(kBM, BN) | (p.b_kmajor ? 0u : (1u << 16)) | (p.a_mnmajor ? (1u << 15) : 0u) |
                                   (p.bf16 ? ((1u << 7) | (1u << 10)) : 0u);
            int it = 0, s = 0;
            uint32_t par = 0;
            for (int t = blockIdx.x; t < n_tiles && !failed; t += gridDim.x, ++it) {
                const int acc = it & 1;
                // the accumulator's previous tile (two tiles ago) has been read out
                if (!bar_wait(&bars->acc_empty[acc], (static_cast<uint32_t>(it >> 1) & 1u) ^ 1u, abort_flag)) { failed = true; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int ks = 0; ks < ksteps; ++ks, s = (s + 1 == stages ? 0 : s + 1), par ^= (s == 0 ? 1u : 0u)) {
                    if (!bar_wait(&bars->full[s], par, abort_flag)) { failed = true; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = s_u32(a_ring + s * a_stage), b_addr = s_u32(b_ring + s * kBStage);
#pragma unroll
                    for (int j = 0; j < kBK / 16; ++j) {
                        const uint64_t adesc = p.a_mnmajor ? smem_desc(a_addr + j * 2048, 8192u, 1024u, kSwizzle128)
                                                           : smem_desc(a_addr + j * 32, 16u, 1024u, kSwizzle128);
                        const uint64_t bdesc = p.b_kmajor ? smem_desc(b_addr + j * 32, 16u, 1024u, kSwizzle128)
                                                          : smem_desc(b_addr + j * 2048, 8192u, 1024u, kSwizzle128);
                        mma_f16_ss(d_tmem, adesc, bdesc, idesc, (ks > 0 || j > 0) ? 1u : 0u);
                    }
                    mma_commit(&bars->empty[s]);
                }
                if (!failed) mma_commit(&bars->acc_full[acc]);
            }
            if (failed || *abort_flag) {
                // every MMA issued so far has completed before the tensor memory is released
                mma_commit(&bars->drain);
                bar_wait(&bars->drain, 0, nullptr, 100000000LL);
            }
        }
    }
    if (failed) {
        *abort_flag = 1;
        if (p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
    }
    __syncwarp();

    if (warp >= 2) {
        const int quad = warp & 3;                          // the TMEM lanes this warp may read
        const bool vec = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && p.beta == 0.f;
        int it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++it) {
            const int m0 = (t % tiles_m) * kBM, n0 = (t / tiles_m) * BN;
            const int acc = it & 1;
            const int row = m0 + quad * 32 + lane;
            const bool ok = bar_wait_warp(&bars->acc_full[acc], static_cast<uint32_t>(it >> 1) & 1u, abort_flag) &&
                            __all_sync(0xffffffffu, !*abort_flag);
            if (!ok) {
                if (lane == 0 && !*abort_flag) {
                    *abort_flag = 1;
                    if (p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
                }
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + c0, v);
                tmem_wait_ld();
                if (row < p.M && n0 + c0 < p.N) {
                    __half* crow = p.C + static_cast<size_t>(row) * p.ldc + n0 + c0;
                    if (vec && n0 + c0 + 16 <= p.N) {
                        uint32_t h[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float f0 = p.alpha * __uint_as_float(v[2 * e]), f1 = p.alpha * __uint_as_float(v[2 * e + 1]);
                            if (p.bf16) {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(f0, f1);
                                h[e] = *reinterpret_cast<const uint32_t*>(&b2);
                            } else {
                                const __half2 h2 = __floats2half2_rn(f0, f1);
                                h[e] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
                        }
                        reinterpret_cast<uint4*>(crow)[0] = make_uint4(h[0], h[1], h[2], h[3]);
                        reinterpret_cast<uint4*>(crow)[1] = make_uint4(h[4], h[5], h[6], h[7]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            if (n0 + c0 + e >= p.N) break;
                            float f = p.alpha * __uint_as_float(v[e]);
                            if (p.bf16) {
                                __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(crow);
                                if (p.beta != 0.f) f += p.beta * __bfloat162float(cb[e]);
                                cb[e] = __float2bfloat16_rn(f);
                            } else {
                                if (p.beta != 0.f) f += p.beta * __half2float(crow[e]);
                                crow[e] = __float2half_rn(f);
                            }
                        }
                    }
                }
            }
            // the accumulator may take the tile after next
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) bar_arrive(&bars->acc_empty[acc]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

// Row-major fp16 matrix [rows][cols] (leading dimension ld) with a box of box_rows x 64 elements (128
// bytes), written to shared memory with the 128-byte swizzle.
bool encode_rows_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (!encode || ld % 8) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
cudaError_t launch_tile(const GemmParams& p, const void* A, const void* B, int lda, int ldb, bool transpose_b,
                        const LaunchEnv& env, cudaStream_t stream) {
    const bool transpose_a = p.a_mnmajor != 0;
    CUtensorMap amap, bmap;
    // A decode batch or a short prefill block has far fewer than 128 rows: copying only those (2 KB
    // instead of 16 KB a stage at 16 rows) leaves the SM's copy bandwidth to B, which is what such a
    // call streams.
    const int a_rows = (!transpose_a && p.M < kBM) ? ((p.M + 7) & ~7) : kBM;
    GemmParams q = p;
    q.a_tx = transpose_a ? static_cast<uint32_t>(kAStage) : static_cast<uint32_t>(a_rows) * kBK * 2u;
    q.a_stage = q.a_tx;     // a multiple of 1024: a_rows is a multiple of 8 rows of 128 bytes
    const int stage_bytes = static_cast<int>(q.a_stage) + BN * kBK * 2;
    q.stages = (env.smem_optin - kGemmBarBytes) / stage_bytes;
    if (q.stages > kMaxStages) q.stages = kMaxStages;
    if (q.stages < 2) return cudaErrorNotSupported;
    const int smem = kGemmBarBytes + q.stages * stage_bytes;
    const bool oka = transpose_a
        ? encode_rows_sw128(&amap, A, static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M), static_cast<uint64_t>(lda), kBK)
        : encode_rows_sw128(&amap, A, static_cast<uint64_t>(p.M), static_cast<uint64_t>(p.K), static_cast<uint64_t>(lda), a_rows);
    if (!oka) return cudaErrorNotSupported;
    const bool okb = transpose_b
        ? encode_rows_sw128(&bmap, B, static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.K), static_cast<uint64_t>(ldb), BN)
        : encode_rows_sw128(&bmap, B, static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.N), static_cast<uint64_t>(ldb), kBK);
    if (!okb) return cudaErrorNotSupported;
    const long tiles = static_cast<long>((p.N + BN - 1) / BN) * ((p.M + kBM - 1) / kBM);
    const long sms = env.sm_count > 0 ? env.sm_count : 148;
    const dim3 grid(static_cast<unsigned>(tiles < sms ? tiles : sms));     // one CTA per SM walks the tiles
    gemm_f16_tc_kernel<BN><<<grid, kGemmThreads, smem, stream>>>(q, amap, bmap);
    return cudaGetLastError();
}

}  // namespace

cudaError_t init_gemm_tc_kernel(int smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(gemm_f16_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_f16_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
}

// cudaErrorNotSupported when the operands are outside what the tiled copies can describe: the leading
// dimensions must be multiples of 8 elements and the bases 16-byte aligned.
cudaError_t launch_gemm_f16_tc(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                               bool transpose_b, float alpha, float beta, const LaunchEnv& env, cudaStream_t stream,
                               bool bf16, bool transpose_a) {
    if (M <= 0 || N <= 0 || K <= 0 || lda % 8 || ldb % 8) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u)) return cudaErrorNotSupported;
    GemmParams p{};
    p.C = static_cast<__half*>(C);
    p.err = env.err_word;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc;
    p.alpha = alpha; p.beta = beta;
    p.b_kmajor = transpose_b ? 1 : 0;
    p.bf16 = bf16 ? 1 : 0;
    p.a_mnmajor = transpose_a ? 1 : 0;
    // 256-wide tiles halve the re-reads of A and the number of MMA instructions; measured faster than 128-wide
    // ones whenever N fills them (4096^3: 1119 against 769 TFLOP/s; 512 x 11008 x 4096: 629 against 523).
    const long sms = env.sm_count > 0 ? env.sm_count : 148;
    const long tiles256 = static_cast<long>((M + kBM - 1) / kBM) * ((N + 255) / 256);
    const bool wide = N >= 256 && tiles256 >= sms;      // few rows of A: narrower tiles spread over more SMs
    return wide ? launch_tile<256>(p, A, B, lda, ldb, transpose_b, env, stream)
                : launch_tile<128>(p, A, B, lda, ldb, transpose_b, env, stream);
}

}  // namespace tcb
