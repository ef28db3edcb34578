// Dense fp16 GEMM on the sm_100a tensor cores: C[M,N] = alpha * A[M,K] . op(B) + beta * C, fp16
// storage, fp32 accumulation - the case of tc_gemm that the fused-norm callers and a prefill of
// dequantised weights use (include/tensorcore/gemm.h:16-58; arithmetic lib/ops/gemm_cpu.cpp:544-568,
// which adds the products in k order; here the tensor core's order, same fp32 accumulation).
//
//   * A CTA computes a 128 x 128 tile of C over the whole K, 64 at a time, through a ring of four
//     stages (16 KB of A + 16 KB of B each).
//   * Operands reach shared memory by TMA, already in the layout the MMA reads without swizzling:
//     the matrix is described to TMA as a 3-D tensor [K/8 chunks][rows][8 elements] (the chunks of
//     a row lie 16 bytes apart), so a box of 8 chunks x 128 rows x 16 bytes lands as eight slabs
//     of [128 rows][16 bytes] - 8-row x 16-byte core matrices, 128 bytes apart along the rows and
//     2048 bytes apart along K (K-major).  B as given ([K][N], N contiguous) is described the same
//     way with the roles of its two dimensions swapped and lands as [N/8 chunks][64 k][16 bytes]:
//     core matrices of 8 k x 8 n, the "MN-major" form of the operand; B transposed ([N][K]) takes
//     the K-major form like A.
//   * One thread issues tcgen05.mma (M128 x N128 x K16, kind::f16, both operands from shared
//     memory descriptors) into 128 columns of tensor memory; tcgen05.commit hands the stage back.
//   * Four warps read the accumulator (one TMEM lane = one row of the tile per thread), apply
//     alpha and beta and store fp16.
// Rows and columns past M, N and K are zero-filled by TMA and masked at the store.  Every wait is
// bounded: it sets the error word and lets the kernel end.
#include "kernels.h"
#include "sm100_prims.cuh"

#include <cuda.h>
#include <cuda_fp16.h>


namespace tcb {
namespace {

using namespace sm100;

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kStages = 4;
constexpr int kAStage = kBM * kBK * 2, kBStage = kBN * kBK * 2;
constexpr int kGemmThreads = 6 * 32;          // producer, MMA issuer, four epilogue warps
constexpr int kGemmBarBytes = 1024;
constexpr uint32_t kAccCols = 128;

struct GemmParams {
    __half* C;
    uint32_t* err;
    int M, N, K, ldc;
    float alpha, beta;
    int b_kmajor;      // B was given transposed ([N][K])
};

struct GemmBars {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t d_full;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(GemmBars) <= kGemmBarBytes, "barrier block too large");

__device__ __forceinline__ void tensor_load_3d(void* dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(s_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(s_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_f16_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
    extern __shared__ __align__(1024) uint8_t smem[];
    GemmBars* bars = reinterpret_cast<GemmBars*>(smem);
    volatile int* abort_flag = &bars->abort_flag;
    uint8_t* a_ring = smem + kGemmBarBytes;
    uint8_t* b_ring = a_ring + kStages * kAStage;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    const int ksteps = (p.K + kBK - 1) / kBK;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) { bar_init(&bars->full[i], 1); bar_init(&bars->empty[i], 1); }
        bar_init(&bars->d_full, 1);
        bars->abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&amap);
        prefetch_tensormap(&bmap);
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, kAccCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int ks = 0; ks < ksteps; ++ks) {
                const int s = ks % kStages;
                const uint32_t par = static_cast<uint32_t>(ks / kStages) & 1u;
                if (!bar_wait(&bars->empty[s], par ^ 1u, abort_flag)) { failed = true; break; }
                bar_expect_tx(&bars->full[s], kAStage + kBStage);
                tensor_load_3d(a_ring + s * kAStage, &amap, 0, m0, ks * (kBK / 8), &bars->full[s]);
                if (p.b_kmajor) tensor_load_3d(b_ring + s * kBStage, &bmap, 0, n0, ks * (kBK / 8), &bars->full[s]);
                else tensor_load_3d(b_ring + s * kBStage, &bmap, 0, ks * kBK, n0 / 8, &bars->full[s]);
                ++issued;
            }
            if (failed || *abort_flag) {
                // Let copies already in flight land before the CTA's shared memory is released.
                const int first = issued > kStages ? issued - kStages : 0;
                for (int ks = first; ks < issued; ++ks)
                    bar_wait(&bars->full[ks % kStages], static_cast<uint32_t>(ks / kStages) & 1u, nullptr, 100000000LL);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = idesc_f16_f32(kBM, kBN) | (p.b_kmajor ? 0u : (1u << 16));
            const uint32_t a_lbo = kBM * 16, a_sbo = 128;                 // K-major: along K, along the rows
            // MN-major B: core matrices 128 bytes apart along K and 1024 along N (64 k x 16 bytes per chunk of
            // 8 n).  In both forms the descriptor's first stride is the one along K, the second the one
            // along M/N (checked on the device with the two assignments: only this one gives the product).
            const uint32_t b_lbo = 128u, b_sbo = 1024u;
            for (int ks = 0; ks < ksteps && !failed; ++ks) {
                const int s = ks % kStages;
                const uint32_t par = static_cast<uint32_t>(ks / kStages) & 1u;
                if (!bar_wait(&bars->full[s], par, abort_flag)) { failed = true; break; }
                tc_fence_after_sync();
                const uint32_t a_addr = s_u32(a_ring + s * kAStage), b_addr = s_u32(b_ring + s * kBStage);
#pragma unroll
                for (int j = 0; j < kBK / 16; ++j) {
                    const uint64_t adesc = smem_desc_kmajor(a_addr + j * 2 * a_lbo, a_lbo, a_sbo);
                    const uint64_t bdesc = p.b_kmajor ? smem_desc_kmajor(b_addr + j * 2 * (kBN * 16), kBN * 16, 128u)
                                                      : smem_desc_kmajor(b_addr + j * 2 * 128, b_lbo, b_sbo);
                    mma_f16_ss(tmem_base, adesc, bdesc, idesc, (ks > 0 || j > 0) ? 1u : 0u);
                }
                mma_commit(&bars->empty[s]);
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

    if (warp >= 2) {
        const int quad = warp & 3;                          // the TMEM lanes this warp may read
        const int row = m0 + quad * 32 + lane;
        const bool ok = bar_wait_warp(&bars->d_full, 0, abort_flag) && __all_sync(0xffffffffu, !*abort_flag);
        if (!ok && lane == 0 && !*abort_flag) {
            *abort_flag = 1;
            if (p.err) atomicOr(p.err, ERR_WAIT_TIMEOUT);
        }
        tc_fence_after_sync();
        if (ok) {
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < kBN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + c0, v);
                tmem_wait_ld();
                if (row < p.M) {
                    __half* crow = p.C + static_cast<size_t>(row) * p.ldc + n0 + c0;
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        if (n0 + c0 + e >= p.N) break;
                        float f = p.alpha * __uint_as_float(v[e]);
                        if (p.beta != 0.f) f += p.beta * __half2float(crow[e]);
                        crow[e] = __float2half_rn(f);
                    }
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kAccCols);
    }
}

// [chunks of 8][rows][8 elements] view of a row-major fp16 matrix [rows][cols] with leading
// dimension ld (elements): box = box_chunks x box_rows x 16 bytes.
bool encode_chunks_3d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_chunks) {
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
    if (!encode || cols % 8 || ld % 8) return false;
    const cuuint64_t dims[3] = {8, rows, cols / 8};
    const cuuint64_t strides[2] = {ld * 2, 16};
    const cuuint32_t box[3] = {8, box_rows, box_chunks};
    const cuuint32_t estr[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t init_gemm_tc_kernel(int smem_optin) {
    return cudaFuncSetAttribute(gemm_f16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
}

// cudaErrorNotSupported when the shapes or addresses are outside what the tiled copies can describe
// (K, the leading dimensions and - for B as given - N must be multiples of 8, bases 16-byte aligned).
cudaError_t launch_gemm_f16_tc(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                               bool transpose_b, float alpha, float beta, const LaunchEnv& env, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 || lda % 8 || ldb % 8) return cudaErrorNotSupported;
    if (!transpose_b && N % 8) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u)) return cudaErrorNotSupported;
    const int smem = kGemmBarBytes + kStages * (kAStage + kBStage);
    if (smem > env.smem_optin) return cudaErrorNotSupported;
    CUtensorMap amap, bmap;
    if (!encode_chunks_3d(&amap, A, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint64_t>(lda), kBM, kBK / 8))
        return cudaErrorNotSupported;
    const bool okb = transpose_b
        ? encode_chunks_3d(&bmap, B, static_cast<uint64_t>(N), static_cast<uint64_t>(K), static_cast<uint64_t>(ldb), kBN, kBK / 8)
        : encode_chunks_3d(&bmap, B, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(ldb), kBK, kBN / 8);
    if (!okb) return cudaErrorNotSupported;
    GemmParams p{};
    p.C = static_cast<__half*>(C);
    p.err = env.err_word;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc;
    p.alpha = alpha; p.beta = beta;
    p.b_kmajor = transpose_b ? 1 : 0;
    const dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
    gemm_f16_tc_kernel<<<grid, kGemmThreads, smem, stream>>>(p, amap, bmap);
    return cudaGetLastError();
}

}  // namespace tcb
