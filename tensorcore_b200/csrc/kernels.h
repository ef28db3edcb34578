// Launch interface between the host layer (runtime.cu) and the sm_100a kernels.
// Everything here works on raw device pointers; handle validation happens above.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tcb {

enum QuantFmt : int { FMT_Q4_0 = 0, FMT_Q8_0 = 1 };

// Kernel families for the quantized GEMV (see gemv_q.cu).
enum GemvVariant : int {
    VARIANT_AUTO = 0,
    VARIANT_SIMT = 1,     // CUDA-core dequant-dot, streamed through shared memory
    VARIANT_MMA = 2,      // warp-level tensor-core dot for 1 <= M <= 8
    VARIANT_TC = 3,       // tcgen05 path for batched decode
    VARIANT_GENERIC = 4,  // any K % 32 == 0, any alignment; correctness path for odd shapes
};

struct LaunchEnv {
    int sm_count = 0;
    int smem_optin = 0;        // max dynamic shared memory per block (opt-in), bytes
    bool pdl = false;          // launch with programmatic stream serialization
    int variant = VARIANT_AUTO;
    uint32_t* err_word = nullptr;  // device-visible word a kernel ORs an error bit into
};

struct GemvQArgs {
    const uint8_t* W = nullptr;   // [N][K/32] blocks
    const void* X = nullptr;      // [M,K] fp16 or fp32
    void* Y = nullptr;            // [M,N] fp16 or fp32
    const void* gamma = nullptr;  // [K], activation dtype; non-null => RMSNorm prologue
    int fmt = 0, M = 0, N = 0, K = 0;
    bool x_f32 = false, y_f32 = false;
    float eps = 0.f;
};

struct DenseNormGemvArgs {
    const void* X = nullptr;      // [M,K] fp16
    const void* gamma = nullptr;  // [K] fp16
    const void* beta = nullptr;   // [K] fp16 or null (null => RMSNorm, else LayerNorm)
    const void* W = nullptr;      // [K,N] fp16, N contiguous
    void* Y = nullptr;            // [M,N] fp16
    int M = 0, N = 0, K = 0;
    float eps = 0.f;
};

// One operation of a persistent decode launch (Q4_0, M = 1); 64 bytes, read by the device.
struct MegaOp {
    const uint8_t* W;
    const void* X;
    void* Y;
    const void* gamma;
    int N, K;
    uint32_t flags;
    float eps;
    int pad[4];
};
enum : uint32_t {
    MOP_BARRIER = 1u,   // grid-wide barrier before this operation (it depends on earlier output)
    MOP_X_F32 = 2u,     // activations (and gamma) are fp32
    MOP_Y_F32 = 4u,     // result is fp32
    MOP_FUSED = 8u,     // RMSNorm prologue with gamma
    MOP_RESTAGE = 16u,  // (re)load the activations into shared memory for this operation
};
struct MegaParams {
    const MegaOp* ops;              // device memory
    const void* maps;               // device memory: one 128-byte TMA tensor map per operation
    int n_ops;
    unsigned long long* counter;    // device memory: grid-barrier arrival counter, never reset
    unsigned long long base;        // counter value all earlier launches add up to
    uint32_t* err;
    int ns;
    int off_rowacc, off_sx, off_x, off_ring;
    int off_ops;                    // shared-memory copy of the operation table, or -1
    int dbg_skip;                   // measurement aid: stream and synchronise, skip arithmetic
    long long* trace = nullptr;     // debug builds: 8 clock64 stamps per operation from CTA 0
};

// Error bits ORed into LaunchEnv::err_word by kernels.
enum : uint32_t { ERR_WAIT_TIMEOUT = 1u, ERR_BAD_SHAPE = 2u };

// Each launcher enqueues on `stream`, adds the number of kernels it launched to *launches (may
// be null) and stores a static string naming the kernel variant in *name (may be null).
cudaError_t launch_quantize(const void* W_f16, void* W_quant, int fmt, int N, int K,
                            const LaunchEnv& env, cudaStream_t stream, int* launches,
                            const char** name);
cudaError_t launch_gemv_q(const GemvQArgs& a, const LaunchEnv& env, cudaStream_t stream,
                          int* launches, const char** name);
cudaError_t launch_dense_norm_gemv(const DenseNormGemvArgs& a, const LaunchEnv& env,
                                   cudaStream_t stream, int* launches, const char** name);

// Persistent decode launch of `n_ops` operations described by `host_ops` (already uploaded to
// `dev_ops`).  Returns cudaErrorNotSupported when the list does not fit the kernel's shared
// memory.  *barriers receives the number of grid barriers the launch executes.
cudaError_t launch_gemv_q4_decode(const MegaOp* host_ops, const MegaOp* dev_ops, const void* dev_maps,
                                  int n_ops, unsigned long long* counter, unsigned long long base,
                                  const LaunchEnv& env, cudaStream_t stream, int* barriers);

// Bytes of one tensor map, and the encoder for the maps of a table of operations: writes
// n_ops * kDecodeMapBytes bytes (64-byte aligned destination), one tiled map per operation over its
// weights as a [N][K/32*18] byte matrix with a 32-row x 144-byte box.
constexpr int kDecodeMapBytes = 128;
cudaError_t encode_decode_maps(const MegaOp* host_ops, int n_ops, void* host_maps);

// The same launch with its scratch (operation table, barrier counter) in a static device array:
// no allocation.  At most 256 operations; cudaErrorInvalidValue beyond that or for operations
// outside the kernel's domain.  First use on a device looks up the array's device address.
cudaError_t launch_gemv_q4_decode_static(const GemvQArgs* ops, int n_ops, const LaunchEnv& env,
                                         cudaStream_t stream);

// One-time per-device kernel attribute setup (max dynamic shared memory).
cudaError_t init_kernels_for_device(int smem_optin);

}  // namespace tcb
