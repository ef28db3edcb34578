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
    VARIANT_SIMT = 1,     // integer dot products on the CUDA cores (never the tcgen05 kernel)
    VARIANT_STREAM = 2,   // as SIMT, but the streaming kernel (a lane per K group) instead of the box kernel
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
    // scratch of the stream the call runs on, for the batched fused form (batched_tc_rows, fp16): room for
    // min(M, 32) normalised rows of K halves and as many floats; without it that form takes the
    // integer dot-product kernels, four rows per pass
    void* norm_scratch = nullptr;
    size_t norm_scratch_bytes = 0;
    // scratch of the stream for prefill-sized calls (gemm_min_rows activation rows or more, fp16 in and
    // out): room for the weights as fp16, N * K halves; with it they are dequantised once and multiplied
    // on the tensor cores instead of streamed once per 32 (Q4_0) or 4 (Q8_0) rows
    void* dequant_scratch = nullptr;
    size_t dequant_scratch_bytes = 0;
};
// Measured back to back on a stream over rotating weight copies.  Q4_0 14336 x 4096: the batched
// kernel takes 32 rows a pass, 64 rows 44 us, 80 rows 63 us, against 64 us this way whatever the row
// count.  Q8_0 has no batched tensor-core kernel and streams the blocks once per 4 rows: 14336 x 4096
// 8 / 12 / 16 / 32 rows 53 / 80 / 105 / 210 us against 66 - 78 us this way; 4096 x 4096 24 / 35 / 46 /
// 90 against 31; 28672 x 8192 155 / 232 / 308 / 615 against 243 - on every shape measured the fourth
// pass (13 rows) is where this way wins.
inline int gemm_min_rows(int fmt) { return fmt == 0 ? 96 : 13; }
// Whether a Q4_0 call with fp16 activations of M rows goes to the batched tcgen05 kernel by default.
// Five rows or more always; four rows where the matrix is large enough that two passes' worth of
// integer dot products cost more than the tensor-core kernel's fixed part (measured back to back on
// a stream, M = 4: 14336 x 4096 21.3 -> 17.8 us, 4096 x 14336 28.6 -> 20.9, 8192 x 8192 23.4 -> 18.7,
// 28672 x 8192 59.2 -> 51.5, 1024 x 8192 14.1 -> 10.7, 32000 x 4096 32.0 -> 28.8; 4096 x 4096 stays
// on the dot-product kernel, 9.6 against 11.0 us; at three rows the two are level or the
// dot-product kernel wins).
inline bool batched_tc_rows(int M, int N, int K) { return M >= 5 || (M == 4 && (K >= 8192 || N > 4096)); }

struct DenseNormGemvArgs {
    const void* X = nullptr;      // [M,K] fp16
    const void* gamma = nullptr;  // [K] fp16
    const void* beta = nullptr;   // [K] fp16 or null (null => RMSNorm, else LayerNorm)
    const void* W = nullptr;      // [K,N] fp16, N contiguous
    void* Y = nullptr;            // [M,N] fp16
    int M = 0, N = 0, K = 0;
    float eps = 0.f;
    // scratch of the stream for five rows or more: M normalised rows of K halves + 2 M floats; with it
    // the rows are normalised once and multiplied on the tensor cores, W read once
    void* norm_scratch = nullptr;
    size_t norm_scratch_bytes = 0;
    // scratch of the stream the call runs on (dense_norm_gemv_scratch says how much): partial sums
    // and one ticket counter per column strip, all zero between launches; without it a slower
    // kernel that needs none is used
    float* scratch = nullptr;
    size_t scratch_floats = 0;
    int* counters = nullptr;
    size_t counters_n = 0;
};
void dense_norm_gemv_scratch(int M, int N, int K, int sm_count, size_t* floats, size_t* ints);

// ---------------------------------------------------------------------------------------
// Persistent decode launch (decode_q4.cu): a list of Q4_0, M = 1 GEMVs as one cooperative kernel.
// ---------------------------------------------------------------------------------------
// One operation of the list; 80 bytes, read by the device.
struct MegaOp {
    const uint8_t* W;
    const void* X;
    void* Y;
    const void* gamma;
    int N, K;
    uint32_t flags;
    float eps;
    uint32_t acc_off;   // accumulator pool: float index of Y's row 0
    int32_t xacc_off;   // >= 0: the activations are the accumulators at this float index (results of
                        // the epoch before); < 0: read X
    uint32_t y_row0;    // this operation's row 0 is row y_row0 of Y (row-sharded results that are
                        // gathered into one vector); 0 otherwise
    uint32_t y_rows;    // rows of Y (>= y_row0 + N)
    uint32_t ss_off;    // MOP_FUSED: pool index of the per-band sums of squares of this operation's
                        // input (written while it is staged; 1/rms is applied by whoever reads the
                        // accumulators afterwards)
    int32_t xss_off;    // >= 0: the accumulators at xacc_off still lack their producer's 1/rms
                        // factor, whose sums of squares are at this pool index ...
    int32_t xss_k;      // ... for a row of this many elements ...
    float xss_eps;      // ... and this epsilon
    uint32_t expect;    // one GPU: partial sums that make a row of this operation complete (its boxes per row)
    uint32_t xexpect;   // the same for the operation whose accumulators are read at xacc_off
    uint32_t x_epoch;   // one GPU: 1 + the epoch of the latest operation of this list that wrote into X, when
                        // X is read from memory (not from the accumulators of the epoch before); else 0
    uint32_t pad;
};
static_assert(sizeof(MegaOp) == 96, "the device copies the table in 16-byte pieces");
enum : uint32_t {
    MOP_BARRIER = 1u,   // grid-wide barrier before this operation (it depends on earlier output)
    MOP_X_F32 = 2u,     // activations (and gamma) are fp32
    MOP_Y_F32 = 4u,     // result is fp32
    MOP_FUSED = 8u,     // RMSNorm prologue with gamma
    MOP_RESTAGE = 16u,  // (re)load the activations into shared memory for this operation
    MOP_XACC_F16 = 32u, // activations taken from accumulators are rounded to fp16 first
    MOP_PEERS = 64u,    // partial sums are added into every rank's accumulators (tensor parallel)
    MOP_BARRIER2 = 128u, // with MOP_BARRIER: two barriers, i.e. one empty epoch, before this operation
};
constexpr int kDecodeMaxRanks = 8;
struct DecodeParams {
    const MegaOp* ops;              // device memory
    const void* maps;               // device memory: one 128-byte TMA tensor map per operation
    int n_ops;
    float* pool;                    // device memory: fp32 accumulators, all zero between launches
    unsigned long long* counter;    // device memory: grid-barrier arrival counter, never reset
    unsigned long long base;        // counter value all earlier launches add up to
    uint32_t* err;
    int ns;
    int off_sx, off_x, off_ring;
    int off_ops;                    // shared-memory copy of the operation table, or -1
    int off_desc, off_phases;       // shared memory: box descriptors of the ring slots, per-phase records
    int n_phases;                   // phases in the table (runs of operations that share their staged input)
    int off_epochs, n_epochs;       // shared memory: first operation of every epoch; epochs in the table
    int off_jscale, jscale_cap;     // shared memory: 1/rms factors of the operations of one epoch, and how many fit
    uint32_t inv_grid;              // ceil(2^32 / gridDim.x): divisions by the grid size as multiplies
    // tensor parallel: every barrier spans all ranks' grids; peer pointers are device addresses
    // of the other ranks' pools and counters, valid on this device
    int n_ranks, rank;
    float* peer_pool[kDecodeMaxRanks];
    unsigned long long* peer_counter[kDecodeMaxRanks];
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

// --- persistent decode launch: planning on the host, then the launch -----------------------
struct DecodeSpan { uintptr_t lo, hi; };
struct DecodePlan {
    int n_ops = 0;
    int max_epoch_ops = 0;     // operations of the longest epoch
    int epochs = 0;            // epochs of the table (runs of operations between two barriers), empty ones included
    int barriers = 0;          // arrivals of one CTA on the arrival counter during a single-GPU launch
    size_t pool_floats = 0;    // accumulator pool the table addresses
};
// Tensor-parallel extras of one operation (all zero on one GPU).
struct DecodeTpOp {
    int peers = 0;             // add the partial sums into every rank's accumulators
    int y_row0 = 0, y_rows = 0;   // placement of the N rows inside a longer gathered vector
    int expect = 0;            // partial sums that complete a row of the result, over all ranks (0 = K / 256):
                               // ranks that split K among them each add K_rank / 256 per row
    int layout_rows = 0;       // accumulators reserved for this result (>= its rows; 0 = its rows): the
                               // same value on every rank keeps the pool layout identical across ranks
                               // when their row shards differ in size
};
// Builds the device table for `ops` (GemvQArgs with M == 1, Q4_0): barriers from pointer overlap,
// accumulator placement, hand-over of results through the accumulators.  `work` is caller scratch
// of 5 * n_ops spans, `table` receives n_ops entries; nothing is allocated.  `tp` may be null.
// cudaErrorNotSupported: the list is outside the kernel's domain (shapes, alignment, an
// operation that writes a later operation's weights, a partial overlap between a result and the
// next epoch's input, more accumulators than pool_capacity_floats when that is non-zero).
// n_ranks > 1 plans for tensor parallelism: four accumulator generations instead of three and a
// choice per barrier between one that spans all ranks and one that spans this rank only.
cudaError_t plan_decode(const GemvQArgs* ops, const DecodeTpOp* tp, int n_ops, DecodeSpan* work,
                        MegaOp* table, DecodePlan* plan, size_t pool_capacity_floats, int n_ranks = 1);
// Device-side state of one launch site (a tc_stream, or the static scratch).
struct DecodeDevice {
    const MegaOp* ops = nullptr;
    const void* maps = nullptr;
    float* pool = nullptr;
    unsigned long long* counter = nullptr;
    unsigned long long base = 0;
    int n_ranks = 1, rank = 0;
    float* peer_pool[kDecodeMaxRanks] = {};
    unsigned long long* peer_counter[kDecodeMaxRanks] = {};
};
// What a completed launch has added to the site's arrival counters: every housekeeping warp of a
// CTA arrives plan.barriers times on a counter of its own (they sit 32 bytes apart in the counter
// allocation and share one base); tensor parallel: on that counter of every rank.
inline void decode_advance(const DecodePlan& plan, int sm_count, int n_ranks, unsigned long long* base) {
    *base += static_cast<unsigned long long>(plan.barriers) * static_cast<unsigned long long>(sm_count) *
             static_cast<unsigned long long>(n_ranks > 1 ? n_ranks : 1);
}
// Launches the table (already uploaded to dev.ops with its tensor maps in dev.maps).
// cudaErrorNotSupported when the list does not fit the kernel's shared memory.
cudaError_t launch_decode(const MegaOp* host_ops, const DecodePlan& plan, const DecodeDevice& dev,
                          const LaunchEnv& env, cudaStream_t stream);

// Bytes of one tensor map, and the encoder for the maps of a table of operations: writes
// n_ops * kDecodeMapBytes bytes (64-byte aligned destination), one tiled map per operation over its
// weights as a [N][K/32*18] byte matrix with a 32-row x 144-byte box.
constexpr int kDecodeMapBytes = 128;
cudaError_t encode_decode_maps(const MegaOp* host_ops, int n_ops, void* host_maps);

// The same launch with all of its scratch (operation table, tensor maps, barrier counter,
// accumulators) in a static device array: no allocation.  At most kDecodeStaticMaxOps operations
// and kDecodeStaticPoolFloats accumulators; cudaErrorNotSupported beyond that or for operations
// outside the kernel's domain (any other error comes from the CUDA runtime).  First use on a device looks up the array's device address.
constexpr int kDecodeStaticMaxOps = 256;
constexpr size_t kDecodeStaticPoolFloats = 24 * 136 * 1024;   // twelve generations of (sum, count) pairs
cudaError_t launch_gemv_q4_decode_static(const GemvQArgs* ops, int n_ops, const LaunchEnv& env,
                                         cudaStream_t stream);

// --- the small operations between the GEMVs of a decode step (step_ops.cu); fp16 data --------
cudaError_t launch_norm_forward(const void* X, const void* gamma, const void* beta /* null = RMSNorm */,
                                void* Y, float* mean_out /* may be null */, float* rstd_out, int N, int D,
                                float eps, cudaStream_t stream);
cudaError_t launch_swiglu(const void* gate, const void* up, void* out, int n, cudaStream_t stream);
cudaError_t launch_rope(void* X, const float* cos_t, const float* sin_t, int batch, int heads, int seq,
                        int head_dim, cudaStream_t stream);
// cudaErrorNotSupported when K floats do not fit a CTA's static shared-memory budget.
// Q4_0 / Q8_0 blocks [N][K/32] back to fp16 [N][K] (quantize.cu).
cudaError_t launch_dequantize(const void* W_quant, void* W_f16, int fmt, int N, int K, cudaStream_t stream);
cudaError_t launch_gemm_f16_rows(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                 int ldc, float alpha, float beta, cudaStream_t stream);
// The same product on the tensor cores (gemm_f16_tc.cu), B as given ([K][N]) or transposed ([N][K]).
// cudaErrorNotSupported when lda or ldb is not a multiple of 8 elements or a base is not 16-byte aligned.
cudaError_t init_gemm_tc_kernel(int smem_optin);
cudaError_t launch_gemm_f16_tc(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                               bool transpose_b, float alpha, float beta, const LaunchEnv& env, cudaStream_t stream,
                               bool bf16 = false, bool transpose_a = false);

// --- attention forward for decode (attention.cu); fp16 data, fp32 softmax ----------------------------
// Floats of scratch the launch needs, and into how many key chunks it will cut a row (1 = no scratch).
size_t attention_scratch_floats(int B, int Hq, int Hkv, int Sq, int Sk, int D, int sm_count, int* chunks_out);
// cudaErrorNotSupported: head_dim above 128.  slopes_dev: ALiBi slopes on the device, or null.
cudaError_t launch_attention_forward(const void* Q, const void* K, const void* V, void* O, float* LSE,
                                     float* scratch, const float* slopes_dev, int B, int Hq, int Hkv, int Sq,
                                     int Sk, int D, float scale, bool causal, int window, int sm_count,
                                     cudaStream_t stream, int* launches);

// --- collectives over NCCL (dist_nccl.cpp); return 0, or -1 bad arguments, -2 NCCL not found,
// -3 rendezvous failed, -4 NCCL / CUDA error ----------------------------------------------------
struct DistComm;
int dist_create(int world, int rank, const char* rendezvous_url, DistComm** out);
void dist_destroy(DistComm* d);
int dist_world(const DistComm* d);
int dist_rank(const DistComm* d);
int dist_allreduce(DistComm* d, void* buf, size_t count, int dtype, int op, cudaStream_t st);
int dist_broadcast(DistComm* d, void* buf, size_t count, int dtype, int root, cudaStream_t st);
int dist_allgather(DistComm* d, const void* in, void* out, size_t count_per_rank, int dtype, cudaStream_t st);
int dist_barrier(DistComm* d, cudaStream_t st);

// One-time per-device kernel attribute setup (max dynamic shared memory).
cudaError_t init_kernels_for_device(int smem_optin);

}  // namespace tcb
