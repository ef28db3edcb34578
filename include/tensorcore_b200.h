/*
 * tensorcore_b200.h - C ABI of the B200 (sm_100a) implementation of tensorcore's
 * quantized-decode path.
 *
 * The library built from tensorcore_b200/csrc is named libtensorcore.so and is a drop-in for
 * the reference library on this path: every tc_* entry point declared in PART 1 has the name,
 * argument list, status codes and buffer layouts of the reference declaration cited beside it
 * (paths are relative to the tsotchke/tensorcore source tree).  A program compiled against
 * the reference's own <tensorcore/tensorcore.h> links and runs against this library
 * unchanged; this header exists so that the boundary can be read in one place.
 *
 * PART 2 declares additive tcx_* entry points that have no counterpart in the reference:
 * fp32-activation / fp32-output forms of the same kernels, explicit host<->device copies for
 * buffers that must never become host-visible, and raw device-pointer launches for callers
 * that own their memory (for example a tensor-parallel driver that allocates with another
 * runtime).  None of them changes the behaviour of a PART 1 symbol.
 *
 * All other tc_* symbols of the reference's export list (cmake/tensorcore.exports) are
 * exported as well so that the reference's ctypes binding, which resolves every symbol at
 * import (python/tensorcore/__init__.py:438-705), loads; outside this path they return
 * TC_ERR_UNSUPPORTED_FAMILY (or 0 / NULL where the return type is not a status).
 *
 * There is no CPU fallback: without an sm_100 device tc_init fails with TC_ERR_NO_DEVICE.
 */
#ifndef TENSORCORE_B200_H
#define TENSORCORE_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================================== *
 * PART 1 - the reference ABI on this path
 * ===================================================================================== */

/* include/tensorcore/status.h:8-22 */
typedef enum {
    TC_OK = 0,
    TC_ERR_NOT_INITIALIZED = -1,
    TC_ERR_ALREADY_INITIALIZED = -2,
    TC_ERR_NO_DEVICE = -3,
    TC_ERR_UNSUPPORTED_FAMILY = -4,
    TC_ERR_UNSUPPORTED_DTYPE = -5,
    TC_ERR_INVALID_SHAPE = -6,
    TC_ERR_INVALID_ARG = -7,
    TC_ERR_ALLOC = -8,
    TC_ERR_KERNEL_NOT_FOUND = -9,
    TC_ERR_PIPELINE = -10,
    TC_ERR_DISPATCH = -11,
    TC_ERR_INTERNAL = -99
} tc_status_t;

/* include/tensorcore/dtype.h:16-27 (numbering is ABI) */
typedef enum {
    TC_DTYPE_F16 = 0, TC_DTYPE_BF16 = 1, TC_DTYPE_F32 = 2, TC_DTYPE_I8 = 3, TC_DTYPE_I32 = 4,
    TC_DTYPE_F64 = 5, TC_DTYPE_SF64 = 6, TC_DTYPE_DF64 = 7, TC_DTYPE_FP24 = 8, TC_DTYPE_FP53 = 9
} tc_dtype_t;

/* include/tensorcore/gemm.h:75-87.  Successful operations of this library record
 * TC_BACKEND_CUDA. */
typedef enum {
    TC_BACKEND_NONE = 0, TC_BACKEND_SIMDGROUP_MATRIX = 1, TC_BACKEND_TENSOROPS_M5 = 2,
    TC_BACKEND_MPS = 3, TC_BACKEND_ACCELERATE_CPU = 4, TC_BACKEND_SF64_EMULATED = 5,
    TC_BACKEND_OZAKI_II = 6, TC_BACKEND_PORTABLE_CPU = 7, TC_BACKEND_METAL_COMPUTE = 8,
    TC_BACKEND_CUDA = 9, TC_BACKEND_HIP = 10
} tc_backend_t;

/* include/tensorcore/device.h:17-43 */
typedef struct tc_context tc_context;
typedef struct tc_buffer tc_buffer;
typedef struct tc_stream tc_stream;

typedef enum {
    TC_FAMILY_UNKNOWN = 0, TC_FAMILY_APPLE7 = 7, TC_FAMILY_APPLE8 = 8, TC_FAMILY_APPLE9 = 9,
    TC_FAMILY_APPLE10 = 10, TC_FAMILY_APPLE11 = 11
} tc_family_t;

typedef struct {
    tc_family_t family;
    char name[128];
    uint64_t max_buffer_bytes;
    uint64_t recommended_working_set_bytes;
    uint32_t max_threadgroup_memory;
    uint32_t max_threads_per_threadgroup;
    uint32_t thread_execution_width;
    bool unified_memory;
    bool supports_bf16_simdgroup;
    bool supports_i8_simdgroup;
    bool supports_tensorops_m5;
    bool supports_fp64_native;
} tc_device_info;

/* include/tensorcore/quantized.h:26-29.  Block layouts (little-endian, no padding):
 *   Q4_0  { fp16 d; uint8 qs[16]; }  18 bytes; qs[i] = code(i) | code(i+16) << 4; w = (code-8)*d
 *   Q8_0  { fp16 d; int8  qs[32]; }  34 bytes; w = qs[i]*d
 * A matrix [N,K] is stored as N rows of K/32 consecutive blocks. */
typedef enum { TC_QUANT_Q4_0 = 0, TC_QUANT_Q8_0 = 1 } tc_quant_t;

/* --- context, include/tensorcore/device.h:45-52; lib/core/device_cpu.cpp:105-179 ---------
 * Process-wide singleton.  A second tc_init bumps a reference count, still stores the handle
 * and returns TC_ERR_ALREADY_INITIALIZED, which callers treat as success.  The context binds
 * the CUDA device that is current in the calling thread (device 0 unless the caller selected
 * another one first); tc_cuda_select_device rebinds it. */
tc_status_t tc_init(tc_context** out_ctx);
tc_status_t tc_shutdown(tc_context* ctx);
tc_status_t tc_device_info_get(tc_context* ctx, tc_device_info* out_info);
const char* tc_version(void);                       /* include/tensorcore/tensorcore.h:31 */
const char* tc_status_string(tc_status_t s);        /* lib/core/status.c:3-20 */
const char* tc_dtype_name(tc_dtype_t d);            /* lib/core/dtype.c:3-17 */
tc_backend_t tc_last_backend(void);                 /* lib/core/device_cpu.cpp:56-59, per thread */
const char* tc_backend_name(tc_backend_t b);        /* lib/core/device_cpu.cpp:61-76 */

/* --- buffers, include/tensorcore/device.h:54-79; lib/core/device_cpu.cpp:190-322 -----------
 * tc_buffer_alloc gives device memory (HBM).  tc_buffer_map keeps the reference's contract -
 * a pointer that stays valid for the buffer's life, coherent with operations at
 * synchronisation points, no unmap - by moving the buffer's storage to CUDA managed memory on
 * the first map; a buffer that is never mapped stays plain device memory.
 * tc_buffer_from_ptr accepts a device pointer (used in place), a managed pointer (used in
 * place, mappable) or a host pointer (each operation stages it through a device mirror:
 * inputs are copied in before the kernel, outputs copied back after it). */
tc_status_t tc_buffer_alloc(tc_context* ctx, size_t bytes, tc_buffer** out);
tc_status_t tc_buffer_free(tc_context* ctx, tc_buffer* buf);
tc_status_t tc_buffer_map(tc_buffer* buf, void** out_ptr);
size_t tc_buffer_size(const tc_buffer* buf);
tc_status_t tc_buffer_from_ptr(tc_context* ctx, void* ptr, size_t bytes, tc_buffer** out);

/* --- streams, include/tensorcore/device.h:81-84; Metal semantics lib/core/device.mm:410-463 -
 * A tc_stream is one in-order CUDA stream plus a list of operations recorded since the last
 * tc_stream_sync.  *_async calls append to the list; tc_stream_sync submits the list (as a
 * replayed CUDA graph once the same list has been seen before) and waits for it - the same
 * "one open command buffer, committed at sync" model the reference's GPU backend has. */
tc_status_t tc_stream_create(tc_context* ctx, tc_stream** out);
tc_status_t tc_stream_destroy(tc_context* ctx, tc_stream* s);
tc_status_t tc_stream_sync(tc_stream* s);

/* --- quantized operations, include/tensorcore/quantized.h:31-80 ----------------------------
 * Status order mirrors lib/ops/quantized_cpu.cpp:108-112,171-177: NULL ctx ->
 * TC_ERR_NOT_INITIALIZED; NULL buffer, non-positive dimension, K % 32 != 0 or unknown fmt ->
 * TC_ERR_INVALID_ARG; buffer of another context -> TC_ERR_INVALID_ARG; buffer too small ->
 * TC_ERR_INVALID_SHAPE. */
size_t tc_quantized_size(tc_quant_t fmt, int N, int K);          /* quantized_cpu.cpp:90-100 */

/* W_fp16 [N,K] binary16 row-major -> W_quant blocks; result bytes are identical to the
 * reference's portable-CPU quantiser (quantized_cpu.cpp:102-162). */
tc_status_t tc_quantize_weights(tc_context* ctx, const tc_buffer* W_fp16, tc_buffer* W_quant,
                                tc_quant_t fmt, int N, int K);

/* Y[M,N] = X[M,K] . W^T, X and Y binary16, fp32 accumulation (quantized_cpu.cpp:164-230).
 * By the number of rows M: one to four rows stream the blocks with integer dot products (a
 * recorded list of one-row Q4_0 calls becomes one persistent launch); five rows or more of Q4_0
 * (four, when K >= 8192 or N > 4096) take the tcgen05 kernel that dequantises into tensor memory; from 96 rows (Q4_0) or 13 rows
 * (Q8_0) the weights are dequantised once into scratch owned by the stream (N * K halves, at most
 * 1.5 GB, else the previous kinds) and multiplied as a dense GEMM on the tensor cores.  The two
 * tensor-core kinds round the dequantised weights to binary16 (inside the 2e-3 bound of binary16
 * activations). */
tc_status_t tc_gemv_quantized(tc_context* ctx, const tc_buffer* X, const tc_buffer* W_quant,
                              tc_buffer* Y, tc_quant_t fmt, int M, int N, int K);

/* Recorded on `stream`; complete after tc_stream_sync (quantized.h:70-77;
 * quantized_cpu.cpp:322-333; lib/ops/quantized.mm:192-211).  NULL stream or a stream of
 * another context -> TC_ERR_INVALID_ARG. */
tc_status_t tc_gemv_quantized_async(tc_context* ctx, const tc_buffer* X,
                                    const tc_buffer* W_quant, tc_buffer* Y, tc_quant_t fmt,
                                    int M, int N, int K, tc_stream* stream);

/* RMSNorm prologue fused into the quantized GEMV; the normalised row stays fp32
 * (quantized.h:49-68; quantized_cpu.cpp:232-320). */
tc_status_t tc_fused_rmsnorm_gemv_quantized(tc_context* ctx, const tc_buffer* X,
                                            const tc_buffer* gamma, const tc_buffer* W_quant,
                                            tc_buffer* Y, tc_quant_t fmt, int M, int N, int K,
                                            float eps);

/* --- fused norm + dense fp16 GEMV, include/tensorcore/training.h:126-164 -------------------
 * W is dense binary16 [K,N], N contiguous.  The normalised row is rounded to binary16 before
 * the product, as lib/ops/training_cpu.cpp:835,912 does.  Unlike the reference's RMS variant
 * (training_cpu.cpp:805-819) both entry points validate every buffer. */
tc_status_t tc_fused_rmsnorm_gemv(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma,
                                  const tc_buffer* W, tc_buffer* Y, int M, int N, int K,
                                  float eps);
tc_status_t tc_fused_layernorm_gemv(tc_context* ctx, const tc_buffer* X,
                                    const tc_buffer* gamma, const tc_buffer* beta,
                                    const tc_buffer* W, tc_buffer* Y, int M, int N, int K,
                                    float eps);

/* --- CUDA device queries, include/tensorcore/cuda.h:50-82; lib/cuda/device.cpp:76-141 ------ */
typedef struct {
    char device_name[128];
    char compute_capability[16];
    int major;
    int minor;
    uint64_t global_memory_bytes;
    uint64_t shared_memory_per_block;
    uint32_t multiprocessor_count;
    uint32_t max_threads_per_block;
    uint32_t warp_size;
    bool supports_fp16;
    bool supports_bf16;
    bool supports_int8_tensor_core;
    bool supports_tf32;
    bool unified_memory;
} tc_cuda_device_info;

tc_status_t tc_cuda_init(tc_context* ctx);
int tc_cuda_device_count(void);
tc_status_t tc_cuda_device_at(int index, tc_cuda_device_info* out_info);
tc_status_t tc_cuda_select_device(tc_context* ctx, int index);
const char* tc_cuda_last_kernel_name(void);         /* per thread; names the kernel variant */

/* --- GGUF v3 reader and loader, include/tensorcore/gguf.h:24-151; lib/io/gguf.c ------------ */
typedef enum {
    TC_GGUF_TYPE_F32 = 0, TC_GGUF_TYPE_F16 = 1, TC_GGUF_TYPE_Q4_0 = 2, TC_GGUF_TYPE_Q4_1 = 3,
    TC_GGUF_TYPE_Q8_0 = 8, TC_GGUF_TYPE_BF16 = 30, TC_GGUF_TYPE_UNSUPPORTED = -1
} tc_gguf_type_t;

typedef struct tc_gguf_file tc_gguf_file;
typedef struct tc_gguf_loaded_model tc_gguf_loaded_model;

typedef struct {
    const char* name;
    int32_t n_dims;
    uint64_t dims[4];
    tc_gguf_type_t type;
    uint64_t offset;
    size_t n_bytes;
    const void* data;          /* into the mapped file */
} tc_gguf_tensor_info;

typedef struct {
    const char* name;
    int32_t n_dims;
    uint64_t dims[4];
    tc_gguf_type_t type;
    uint64_t offset;
    size_t n_bytes;
    tc_buffer* buffer;         /* device buffer owned by the loaded model */
} tc_gguf_loaded_tensor_info;

typedef struct {
    int64_t context_length, embedding_length, feed_forward_length, block_count;
    int64_t attention_head_count, attention_head_count_kv, rope_dimension_count, vocab_size;
    double rms_norm_epsilon, rope_freq_base, rope_freq_scale;
} tc_gguf_llama_config;

typedef struct {
    int N;                     /* output rows = GGUF dims[1] */
    int K;                     /* input columns = GGUF dims[0] */
    tc_gguf_type_t gguf_type;
    tc_quant_t quant_type;
    size_t n_bytes;
    tc_buffer* buffer;
} tc_gguf_quantized_matrix_info;

tc_status_t tc_gguf_open(const char* path, tc_gguf_file** out);              /* gguf.c:341-462 */
void tc_gguf_close(tc_gguf_file* f);
uint64_t tc_gguf_tensor_count(const tc_gguf_file* f);
uint64_t tc_gguf_metadata_count(const tc_gguf_file* f);
tc_status_t tc_gguf_get_tensor(const tc_gguf_file* f, const char* name, tc_gguf_tensor_info* out);
tc_status_t tc_gguf_tensor_at(const tc_gguf_file* f, uint64_t i, tc_gguf_tensor_info* out);
const char* tc_gguf_meta_get_str(const tc_gguf_file* f, const char* key);
int64_t tc_gguf_meta_get_i64(const tc_gguf_file* f, const char* key, int64_t default_val);
double tc_gguf_meta_get_f64(const tc_gguf_file* f, const char* key, double default_val);
uint64_t tc_gguf_meta_array_count(const tc_gguf_file* f, const char* key);
tc_status_t tc_gguf_meta_array_get_str(const tc_gguf_file* f, const char* key, uint64_t index,
                                       const char** out_ptr, size_t* out_len);
int64_t tc_gguf_meta_array_get_i64(const tc_gguf_file* f, const char* key, uint64_t index,
                                   int64_t default_val);
double tc_gguf_meta_array_get_f64(const tc_gguf_file* f, const char* key, uint64_t index,
                                  double default_val);
tc_status_t tc_gguf_get_llama_config(const tc_gguf_file* f, tc_gguf_llama_config* out);
/* gguf.c:695-750: tensor bytes go from the file mapping straight to a device buffer through a
 * pinned staging ring; the buffer is never made host-visible unless the caller maps it. */
tc_status_t tc_gguf_tensor_to_buffer(tc_context* ctx, const tc_gguf_file* f, const char* name,
                                     tc_buffer** out_buffer);
tc_status_t tc_gguf_tensor_quantized_matrix_info(const tc_gguf_tensor_info* tensor,
                                                 tc_gguf_quantized_matrix_info* out);
tc_status_t tc_gguf_loaded_tensor_quantized_matrix_info(const tc_gguf_loaded_tensor_info* tensor,
                                                        tc_gguf_quantized_matrix_info* out);
tc_status_t tc_gguf_load_supported_tensors(tc_context* ctx, const tc_gguf_file* f,
                                           tc_gguf_loaded_model** out_model);  /* gguf.c:819-869 */
void tc_gguf_loaded_model_free(tc_context* ctx, tc_gguf_loaded_model* model);
uint64_t tc_gguf_loaded_tensor_count(const tc_gguf_loaded_model* model);
uint64_t tc_gguf_loaded_skipped_tensor_count(const tc_gguf_loaded_model* model);
tc_status_t tc_gguf_loaded_tensor_at(const tc_gguf_loaded_model* model, uint64_t i,
                                     tc_gguf_loaded_tensor_info* out);
tc_status_t tc_gguf_loaded_get_tensor(const tc_gguf_loaded_model* model, const char* name,
                                      tc_gguf_loaded_tensor_info* out);

/* --- the operations between the GEMVs of a decode step (include/tensorcore/training.h:19-24,
 * 38-45, 60-64, 81-85; arithmetic of lib/ops/training_cpu.cpp:126-186, 287-350, 427-482, 541-573):
 * fp16 data, fp32 arithmetic, statistics accumulated in double.  Synchronous. */
tc_status_t tc_rmsnorm_forward(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma, tc_buffer* Y,
                               tc_buffer* rstd_out, int N, int D, float eps);
tc_status_t tc_layernorm_forward(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma,
                                 const tc_buffer* beta, tc_buffer* Y, tc_buffer* mean_out,
                                 tc_buffer* rstd_out, int N, int D, float eps);
tc_status_t tc_rope_forward(tc_context* ctx, tc_buffer* X, const tc_buffer* cos_t, const tc_buffer* sin_t,
                            int batch, int heads, int seq, int head_dim);
tc_status_t tc_swiglu_forward(tc_context* ctx, const tc_buffer* gate, const tc_buffer* up, tc_buffer* out,
                              int n);

/* include/tensorcore/gemm.h:16-58 (arithmetic: lib/ops/gemm_cpu.cpp:544-568).  Here: binary16 or
 * bfloat16 operands and result (all three the same) with fp32 accumulation, row-major, A and B as
 * given ([M,K], [K,N]) or transposed ([K,M], [N,K]), alpha, beta and leading dimensions - on the tensor cores (tcgen05)
 * when lda and ldb are multiples of 8 elements and A and B are 16-byte aligned; binary16 with up to
 * four rows of A (a decode step: what tests/test_fused_norm_gemv.c compares the fused operations
 * against) or untransposed operands outside that take a row kernel that adds in the reference's k
 * order.  The result is narrowed with round-to-nearest-even.  Every other descriptor answers
 * TC_ERR_UNSUPPORTED_DTYPE (dtypes) or TC_ERR_UNSUPPORTED_FAMILY (bfloat16 or transposed operands
 * the tiled copies cannot describe). */
typedef struct {
    int32_t M, N, K;
    tc_dtype_t a_dtype, b_dtype, c_dtype, accum_dtype;
    bool transpose_a, transpose_b;
    float alpha, beta;
    int32_t lda, ldb, ldc;
} tc_gemm_desc;
tc_status_t tc_gemm(tc_context* ctx, const tc_gemm_desc* desc, const tc_buffer* A, const tc_buffer* B,
                    tc_buffer* C);
/* include/tensorcore/gemm.h:59-72: `batch` products of one shape, consecutive matrices stride_* elements
 * apart (one launch per product).  batch <= 0 -> TC_ERR_INVALID_ARG; batch > 1 with a stride that is
 * not positive or shorter than a matrix -> TC_ERR_INVALID_SHAPE (lib/ops/gemm_cpu.cpp:775-795). */
typedef struct {
    tc_gemm_desc base;
    int32_t batch;
    int64_t stride_a, stride_b, stride_c;
} tc_gemm_batched_desc;
tc_status_t tc_gemm_batched(tc_context* ctx, const tc_gemm_batched_desc* desc, const tc_buffer* A,
                            const tc_buffer* B, tc_buffer* C);
/* include/tensorcore/gemm.h:52-58; runs at once, like the recorded forms of the other step operations. */
tc_status_t tc_gemm_async(tc_context* ctx, const tc_gemm_desc* desc, const tc_buffer* A, const tc_buffer* B,
                          tc_buffer* C, tc_stream* stream);

/* include/tensorcore/attention.h:24-69 (arithmetic: lib/ops/attention_cpu.cpp:131-277).  fp16 Q
 * [batch, heads, seq_q, head_dim], K and V [batch, kv_heads, seq_kv, head_dim], O like Q, optional
 * fp32 LSE [batch, heads, seq_q]; softmax in fp32.  Causal mask (key index > query index), sliding
 * window, ALiBi and grouped-query heads as in the reference.  Here: the forward pass as a
 * streaming kernel per query row - the attention of a decode step (seq_q of one or a few rows over
 * a long K/V cache); head_dim <= 128 (TC_ERR_INVALID_SHAPE above).  The recorded form runs at once,
 * as the reference's CPU backend does.  tc_attention_backward stays a placeholder. */
typedef struct {
    int32_t batch, heads, seq_q, seq_kv, head_dim;
    tc_dtype_t io_dtype;      /* TC_DTYPE_F16 */
    tc_dtype_t accum_dtype;   /* TC_DTYPE_F32 */
    float softmax_scale;      /* <= 0: 1 / sqrt(head_dim) */
    bool causal;
    bool return_lse;
    int32_t kv_heads;         /* 0: heads */
    int32_t window_size;      /* 0: none */
    const float* alibi_slopes; /* host array of `heads` floats, or NULL */
} tc_attention_desc;
tc_status_t tc_attention_forward(tc_context* ctx, const tc_attention_desc* desc, const tc_buffer* Q,
                                 const tc_buffer* K, const tc_buffer* V, tc_buffer* O, tc_buffer* LSE);
tc_status_t tc_attention_forward_async(tc_context* ctx, const tc_attention_desc* desc, const tc_buffer* Q,
                                       const tc_buffer* K, const tc_buffer* V, tc_buffer* O, tc_buffer* LSE,
                                       tc_stream* stream);

/* --- collectives (include/tensorcore/distributed.h:30-87; the reference implements them as a TCP
 * ring between hosts, lib/distributed/distributed_cpu.cpp:202-347).  Here: NCCL between one
 * process per GPU, on device buffers.  TC_DIST_RING and TC_DIST_GLOO both select it; the
 * rendezvous URL "<anything>://host:port" names where rank 0 hands out NCCL's unique id.
 * TC_ERR_UNSUPPORTED_FAMILY when no NCCL library can be loaded.  Element types fp16 and fp32. */
typedef enum { TC_DIST_SINGLE = 0, TC_DIST_RING = 1, TC_DIST_GLOO = 2 } tc_dist_backend_t;
typedef enum { TC_REDUCE_SUM = 0, TC_REDUCE_AVG = 1, TC_REDUCE_MAX = 2, TC_REDUCE_MIN = 3 } tc_reduce_op_t;
typedef struct tc_dist_ctx tc_dist_ctx;
tc_status_t tc_dist_init(tc_context* tc, tc_dist_backend_t backend, int world_size, int rank,
                         const char* rendezvous_url, tc_dist_ctx** out);
tc_status_t tc_dist_finalize(tc_dist_ctx* d);
int tc_dist_world_size(const tc_dist_ctx* d);
int tc_dist_rank(const tc_dist_ctx* d);
tc_status_t tc_allreduce(tc_dist_ctx* d, tc_buffer* buf, size_t num_elements, tc_dtype_t dtype, tc_reduce_op_t op);
tc_status_t tc_broadcast(tc_dist_ctx* d, tc_buffer* buf, size_t num_elements, tc_dtype_t dtype, int root);
tc_status_t tc_allgather(tc_dist_ctx* d, const tc_buffer* in, tc_buffer* out, size_t num_elements_per_rank,
                         tc_dtype_t dtype);
tc_status_t tc_barrier(tc_dist_ctx* d);

extern const int tensorcore_abi_version;            /* lib/c_api/c_api_cpu.c:15-16 */

/* ===================================================================================== *
 * PART 2 - additive entry points (no counterpart in the reference)
 * ===================================================================================== */

/* Quantized GEMV / fused RMSNorm GEMV with selectable activation and result types
 * (TC_DTYPE_F16 or TC_DTYPE_F32 each; gamma has the activation type).  `stream` may be NULL
 * (the call then completes before returning) or a tc_stream (recorded, complete after
 * tc_stream_sync).  Arithmetic is that of the reference loops with the binary16 conversions of
 * the chosen operands removed. */
tc_status_t tcx_gemv_quantized_ex(tc_context* ctx, const tc_buffer* X, const tc_buffer* W_quant,
                                  tc_buffer* Y, tc_quant_t fmt, int M, int N, int K,
                                  tc_dtype_t x_dtype, tc_dtype_t y_dtype, tc_stream* stream);
tc_status_t tcx_fused_rmsnorm_gemv_quantized_ex(tc_context* ctx, const tc_buffer* X,
                                                const tc_buffer* gamma, const tc_buffer* W_quant,
                                                tc_buffer* Y, tc_quant_t fmt, int M, int N, int K,
                                                float eps, tc_dtype_t x_dtype, tc_dtype_t y_dtype,
                                                tc_stream* stream);

/* Copies between host memory and a buffer without making the buffer host-visible.  Both wait
 * for completion. */
tc_status_t tcx_buffer_upload(tc_buffer* buf, size_t offset, const void* src, size_t bytes);
tc_status_t tcx_buffer_download(const tc_buffer* buf, size_t offset, void* dst, size_t bytes);
/* The device address operations use for this buffer (NULL for a host-pointer wrapper's
 * caller memory; its device mirror is returned instead). */
tc_status_t tcx_buffer_device_ptr(const tc_buffer* buf, void** out_dptr);
/* The cudaStream_t behind a tc_stream, as void*. */
tc_status_t tcx_stream_cuda_handle(const tc_stream* s, void** out_cuda_stream);
/* Submit the operations recorded on the stream without waiting for them. */
tc_status_t tcx_stream_flush(tc_stream* s);
/* Recorded lists of Q4_0, M = 1 operations normally run as ONE persistent kernel per
 * tc_stream_sync; enable = 0 makes this stream launch one kernel per operation instead (CUDA
 * graph replay from the second identical list), e.g. to compare the two. */
tc_status_t tcx_stream_set_persistent(tc_stream* s, int enable);

/* Raw launches on caller-owned device memory.  Pointers are device addresses valid on the
 * context's device; `cuda_stream` is a cudaStream_t as void* (NULL = the legacy default
 * stream).  The launch is asynchronous; errors detected at launch are returned.  Shapes and
 * dtypes as for the tc_* operations above. */
tc_status_t tcx_raw_quantize_weights(tc_context* ctx, const void* W_fp16, void* W_quant,
                                     tc_quant_t fmt, int N, int K, void* cuda_stream);
tc_status_t tcx_raw_gemv_quantized(tc_context* ctx, const void* X, const void* W_quant, void* Y,
                                   tc_quant_t fmt, int M, int N, int K, tc_dtype_t x_dtype,
                                   tc_dtype_t y_dtype, void* cuda_stream);
tc_status_t tcx_raw_fused_rmsnorm_gemv_quantized(tc_context* ctx, const void* X,
                                                 const void* gamma, const void* W_quant, void* Y,
                                                 tc_quant_t fmt, int M, int N, int K, float eps,
                                                 tc_dtype_t x_dtype, tc_dtype_t y_dtype,
                                                 void* cuda_stream);
/* tc_attention_forward on raw device pointers, asynchronous on `cuda_stream` (desc->alibi_slopes must
 * be NULL).  The scratch that holds the partial softmax states of a row's key chunks belongs to the
 * context: do not let two of these launches overlap on different streams. */
tc_status_t tcx_raw_attention_forward(tc_context* ctx, const tc_attention_desc* desc, const void* Q,
                                      const void* K, const void* V, void* O, void* LSE /* or NULL */,
                                      void* cuda_stream);
tc_status_t tcx_raw_fused_norm_gemv_f16(tc_context* ctx, const void* X, const void* gamma,
                                        const void* beta /* NULL = RMSNorm */, const void* W,
                                        void* Y, int M, int N, int K, float eps,
                                        void* cuda_stream);

/* Decode launch that allocates nothing (no counterpart in the reference).
 *
 * Runs a whole list of Q4_0, batch-1 GEMVs - one decode step - as one persistent kernel, like a
 * qualifying tc_stream list, but for callers that cannot tolerate an allocation on this path:
 * a server whose HBM is fully handed out to weights and KV cache at start-up, or a decode loop
 * where cudaMalloc's device-wide synchronisation must never occur.  The kernel's scratch (the
 * arrival counters, the operation table, one TMA tensor map per operation and the accumulators
 * the results are summed in) lives in a fixed 13,112 KB device array inside the library image,
 * which every GPU that loads the library holds until the process exits; the call performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *
 *  - `ops`: host array of `n_ops` operations in execution order; all pointers inside are device
 *    addresses owned by the caller (inputs and outputs as for tcx_raw_gemv_quantized with M = 1;
 *    gamma != NULL adds the RMSNorm prologue).  K must be a multiple of 256, pointers 16-byte
 *    aligned.  Dependencies between operations are derived from pointer overlap.
 *  - Limits: n_ops <= TCX_DECODE_STATIC_MAX_OPS (256) and a list whose accumulators fit the
 *    array: the widest group of operations that run side by side may have 139,264 result rows
 *    together (a 128k-row output projection fits; the array holds twelve generations of
 *    (sum, count) pairs of that many rows); beyond either the call returns TC_ERR_INVALID_SHAPE
 *    and launches nothing, as it does for a list whose activations do not fit the kernel's
 *    shared memory.
 *  - The first call on a device looks up the array's device address; make that first call before
 *    starting any stream capture.
 *  - All calls on a device share the one array: the call clears the counters and overwrites the
 *    table itself, but two calls that overlap in time on the GPU (different streams) race.  The
 *    host-side bookkeeping (one record per device) is guarded by a mutex, so calls from several
 *    threads are safe as long as their launches do not overlap on one GPU.
 *  - Asynchronous on `cuda_stream`, like the other tcx_raw_* launches. */
typedef struct {
    const void* W;        /* Q4_0 blocks, [N][K/32] x 18 bytes */
    const void* X;        /* [K] activations */
    void* Y;              /* [N] results */
    const void* gamma;    /* [K] RMSNorm weights (activation dtype) or NULL */
    int N, K;
    tc_dtype_t x_dtype, y_dtype;   /* TC_DTYPE_F16 or TC_DTYPE_F32 */
    float eps;
} tcx_decode_op;
#define TCX_DECODE_STATIC_MAX_OPS 256
tc_status_t tcx_raw_decode_q4_static(tc_context* ctx, const tcx_decode_op* ops, int n_ops,
                                     void* cuda_stream);

/* Tensor-parallel decode (no counterpart in the reference, which has no GPU collectives).
 *
 * One process per GPU.  Every rank records the SAME list of operations on its own shard of the
 * weights: projections split by output rows (q/k/v, gate/up, lm_head) compute their own rows;
 * projections split along K (o_proj, down_proj) compute partial sums over their K range.  An
 * operation marked `peers` adds its partial sums into the accumulators of EVERY rank inside the
 * persistent decode kernel, with vector reductions over NVLink peer memory that carry the sum and
 * a count - that is the all-reduce of a K-split projection and, with `y_row0` / `y_rows` placing
 * a rank's rows inside a longer vector, the all-gather of a row-split one.  The next operation
 * starts on a rank as soon as the counts of its input rows say that every rank's partial sums are
 * there: no barrier lies between two operations.  (An arrival counter that spans all ranks trails
 * the computation by a few operations and tells when accumulators may be reused; its waits are
 * bounded as everywhere else.)  No collective library is involved.  A whole token is one launch
 * per rank.
 *
 *  1. every rank: tcx_stream_tp_export(stream, pool_floats, handles) - allocates the stream's
 *     accumulator pool (24 floats per result row of the widest group of operations that run
 *     side by side; 4 Mi floats cover the 70B shapes) and arrival counters and writes two CUDA IPC
 *     handles (128 bytes);
 *  2. exchange the 128-byte records among the ranks by any host channel, in rank order;
 *  3. every rank: tcx_stream_tp_connect(stream, n_ranks, rank, all_records);
 *  4. per token, every rank: tcx_stream_decode_tp(stream, ops, n_ops) then tc_stream_sync(stream).
 *
 * The lists must have the same structure on every rank (same order, same dependencies, same
 * `layout_rows`), so that accumulator offsets agree; `layout_rows` (the largest row count of the
 * operation over the ranks) keeps them equal when row shards differ in size.  n_ranks == 1 (no
 * connect call) runs the same list on one GPU. */
typedef struct {
    tcx_decode_op op;
    int peers;         /* 1: results are summed into / placed in every rank's copy of Y */
    int y_row0;        /* row of Y that this rank's row 0 maps to (gathered results), else 0 */
    int y_rows;        /* rows of Y (0 = op.N) */
    int layout_rows;   /* accumulators to reserve (0 = y_rows); identical on all ranks */
    int expect;        /* partial sums that complete a row, over all ranks: the sum of op.K / 256 over the
                          ranks that add to the same rows (0 = op.K / 256: only this rank adds to them) */
} tcx_decode_tp_op;
tc_status_t tcx_stream_tp_export(tc_stream* s, size_t pool_floats, void* handles_out_128_bytes);
tc_status_t tcx_stream_tp_connect(tc_stream* s, int n_ranks, int rank, const void* all_records);
tc_status_t tcx_stream_decode_tp(tc_stream* s, const tcx_decode_tp_op* ops, int n_ops);

/* Kernel-variant override for A/B measurements: "auto" (default), "simt" (CUDA-core integer dot
 * products at any M), "stream" (the same arithmetic on the streaming kernel instead of the box
 * kernel), "tc" (tcgen05 kernel where it applies), "generic".  Returns TC_ERR_INVALID_ARG for an
 * unknown name.  Process-wide. */
tc_status_t tcx_set_gemv_variant(const char* name);
/* Device-side error word: non-zero after a kernel gave up on a bounded wait.  Reading clears. */
uint32_t tcx_take_device_error(tc_context* ctx);
/* Number of kernel launches this library has issued in the calling process. */
uint64_t tcx_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TENSORCORE_B200_H */
