// Block quantiser for sm_100a: fp16 [N,K] -> GGUF Q4_0 / Q8_0 blocks, byte-identical to the
// reference's portable-CPU quantiser.
//
// Exactness notes.  Every floating-point step is an IEEE fp32 operation with one rounding,
// spelled with the _rn intrinsics so that no contraction or fast-math substitution can change
// it: a = max|w| (a NaN never replaces the running maximum), d = a / d0, inv = d0 / a (0 when
// d is not positive), code = round-half-away(w * inv), stored scale = fp16(d) rounded to
// nearest even.  roundf() is exact (no error ulp) in CUDA's math library.
//
// One thread quantises one block: it reads its 32 halves with four 128-bit loads (a warp covers
// 2 KB of contiguous input) and the warp assembles its 32 output blocks (576 or 1088
// contiguous bytes, always 16-byte aligned because a warp starts on a multiple of 32 blocks)
// in shared memory and stores them with 128-bit writes.
#include "kernels.h"

#include <cuda_fp16.h>

namespace tcb {
namespace {

constexpr int kQThreads = 256;

template <int FMT>
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const uint4* __restrict__ W,
                                                             uint8_t* __restrict__ out,
                                                             long long total_blocks) {
    constexpr int BB = FMT == FMT_Q4_0 ? 18 : 34;
    constexpr float D0 = FMT == FMT_Q4_0 ? 8.0f : 127.0f;
    __shared__ __align__(16) uint8_t stage[kQThreads / 32][32 * BB];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warp_first =
        (static_cast<long long>(blockIdx.x) * kQThreads + warp * 32);
    if (warp_first >= total_blocks) return;
    const long long blk = warp_first + lane;
    const bool valid = blk < total_blocks;

    if (valid) {
        float w[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 v = __ldg(W + blk * 4 + c);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w[c * 8 + e * 2 + 0] = __half2float(__ushort_as_half(static_cast<uint16_t>(u[e])));
                w[c * 8 + e * 2 + 1] = __half2float(__ushort_as_half(static_cast<uint16_t>(u[e] >> 16)));
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float av = fabsf(w[i]);
            if (amax < av) amax = av;  // false for NaN: a NaN never becomes the maximum
        }
        const float scale = __fdiv_rn(amax, D0);
        const float inv = scale > 0.0f ? __fdiv_rn(D0, amax) : 0.0f;
        uint8_t* dst = &stage[warp][lane * BB];
        const uint16_t sb = __half_as_ushort(__float2half_rn(scale));
        dst[0] = static_cast<uint8_t>(sb);
        dst[1] = static_cast<uint8_t>(sb >> 8);
        if (FMT == FMT_Q4_0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                int lo = static_cast<int>(roundf(__fmul_rn(w[i], inv))) + 8;
                int hi = static_cast<int>(roundf(__fmul_rn(w[i + 16], inv))) + 8;
                lo = max(0, min(15, lo));
                hi = max(0, min(15, hi));
                dst[2 + i] = static_cast<uint8_t>((hi << 4) | lo);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                int q = static_cast<int>(roundf(__fmul_rn(w[i], inv)));
                q = max(-128, min(127, q));
                dst[2 + i] = static_cast<uint8_t>(static_cast<int8_t>(q));
            }
        }
    }
    __syncwarp();
    const long long remaining = total_blocks - warp_first;
    const int nvalid = remaining < 32 ? static_cast<int>(remaining) : 32;
    const int nbytes = nvalid * BB;
    uint8_t* gdst = out + warp_first * BB;
    // 128-bit stores need a 16-byte aligned destination; otherwise fall back to byte stores.
    const int nv4 = (reinterpret_cast<uintptr_t>(gdst) & 15u) == 0 ? nbytes / 16 : 0;
    const uint4* s4 = reinterpret_cast<const uint4*>(&stage[warp][0]);
    for (int i = lane; i < nv4; i += 32) reinterpret_cast<uint4*>(gdst)[i] = s4[i];
    for (int i = nv4 * 16 + lane; i < nbytes; i += 32) gdst[i] = stage[warp][i];
}

}  // namespace

// Blocks back to fp16, [N][K] row-major: (q - 8) * d for Q4_0, q * d for Q8_0, one rounding each (the
// product of an integer of at most 8 bits and an fp16 has at most 19 significant bits).  A thread
// per eight weights: it reads the block's scale and eight bytes of quants (blocks are 2-byte
// aligned: four 16-bit loads) and writes one 16-byte piece, so a warp writes 512 contiguous bytes.
// For the prefill-sized path of the quantized GEMV (many activation rows), which multiplies the
// result on the tensor cores.
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ Wq, __half* __restrict__ W,
                                                         long long pieces, int q8) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= pieces) return;
    const long long b = t >> 2;
    const int q = static_cast<int>(t & 3);
    const uint8_t* blk = Wq + b * (q8 ? 34 : 18);
    const float d = __half2float(*reinterpret_cast<const __half*>(blk));
    // Q8_0: elements 8q .. 8q+7 are bytes 8q .. 8q+7.  Q4_0: elements 0-15 are the low nibbles of bytes
    // 0-15, elements 16-31 the high nibbles: piece q takes bytes 8 (q & 1) .. + 7, high nibbles for q >= 2.
    const uint16_t* src = reinterpret_cast<const uint16_t*>(blk + 2 + (q8 ? 8 * q : 8 * (q & 1)));
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t two = src[i];
        float f0, f1;
        if (q8) {
            f0 = static_cast<float>(static_cast<int8_t>(two & 0xffu));
            f1 = static_cast<float>(static_cast<int8_t>(two >> 8));
        } else {
            const int sh = (q >> 1) * 4;
            f0 = static_cast<float>(static_cast<int>((two >> sh) & 15u) - 8);
            f1 = static_cast<float>(static_cast<int>((two >> (8 + sh)) & 15u) - 8);
        }
        const __half2 h = __floats2half2_rn(f0 * d, f1 * d);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(W)[t] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

cudaError_t launch_dequantize(const void* W_quant, void* W_f16, int fmt, int N, int K, cudaStream_t stream) {
    if ((fmt != FMT_Q4_0 && fmt != FMT_Q8_0) || N <= 0 || K <= 0 || K % 32) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(W_f16) & 15u) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(W_quant) & 1u) return cudaErrorNotSupported;
    const long long pieces = static_cast<long long>(N) * (K / 32) * 4;
    const long long grid = (pieces + 255) / 256;
    if (grid > 0x7fffffffLL) return cudaErrorNotSupported;
    dequantize_kernel<<<static_cast<unsigned>(grid), 256, 0, stream>>>(static_cast<const uint8_t*>(W_quant),
                                                                      static_cast<__half*>(W_f16), pieces, fmt == FMT_Q8_0);
    return cudaGetLastError();
}

cudaError_t launch_quantize(const void* W_f16, void* W_quant, int fmt, int N, int K,
                            const LaunchEnv& env, cudaStream_t stream, int* launches,
                            const char** name) {
    (void)env;
    const long long total = static_cast<long long>(N) * (K / 32);
    const unsigned grid = static_cast<unsigned>((total + kQThreads - 1) / kQThreads);
    if (fmt == FMT_Q4_0) {
        quantize_kernel<FMT_Q4_0><<<grid, kQThreads, 0, stream>>>(
            static_cast<const uint4*>(W_f16), static_cast<uint8_t*>(W_quant), total);
        if (name) *name = "q4_0_quantize_sm100";
    } else {
        quantize_kernel<FMT_Q8_0><<<grid, kQThreads, 0, stream>>>(
            static_cast<const uint4*>(W_f16), static_cast<uint8_t*>(W_quant), total);
        if (name) *name = "q8_0_quantize_sm100";
    }
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace tcb
