// Host layer of the B200 tensorcore library: context, device buffers, streams and the
// operation entry points of the quantized-decode path.  Thin by design - argument checks in
// the reference's order, pointer resolution, then a kernel launch from kernels.h.
//
// There is no CPU fallback anywhere in this file: if the device or a launch is unavailable the
// call fails with a status code.
#include "../../include/tensorcore_b200.h"
#include "kernels.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <mutex>
#include <new>
#include <unordered_map>
#include <vector>

using tcb::LaunchEnv;

namespace tcb {
cudaError_t init_gemv_kernels(int smem_optin);
}

// ---------------------------------------------------------------------------------------
// Handle definitions
// ---------------------------------------------------------------------------------------
enum BufKind : int {
    BUF_DEVICE = 0,        // cudaMalloc, owned; never seen by the host
    BUF_MANAGED = 1,       // cudaMallocManaged, owned; host-visible after tc_buffer_map
    BUF_WRAP_DEVICE = 2,   // caller's device memory
    BUF_WRAP_MANAGED = 3,  // caller's managed memory
    BUF_WRAP_HOST = 4,     // caller's host memory + owned device mirror, staged per operation
    BUF_HOST_SHADOW = 5,   // owned pinned host shadow + device memory (when managed memory is
                           // unavailable), staged per operation
};

struct tc_context {
    tc_device_info info;
    std::atomic<int> ref;
    int device;
    int sm_count;
    int smem_optin;
    bool managed_ok;
    bool pdl;
    bool graphs;
    cudaStream_t stream0;
    uint32_t* err_host;   // pinned, mapped
    uint32_t* err_dev;
    bool mega_on;         // route qualifying recorded lists to the persistent decode kernel
    float* attn_scratch;  // partial softmax states of tc_attention_forward, grown on demand
    size_t attn_scratch_floats;
};

struct tc_buffer {
    void* dptr;
    void* hptr;
    size_t bytes;
    tc_context* owner;
    BufKind kind;
    bool prefetch_hint;   // host may have touched a managed buffer since its last device use
};

namespace {

enum OpKind : int { OP_GEMV_Q = 1 };

struct RecordedOp {
    int kind;
    tcb::GemvQArgs a;
    tc_buffer* X;
    tc_buffer* W;
    tc_buffer* Y;
    tc_buffer* gamma;
    size_t x_bytes, w_bytes, y_bytes, g_bytes;
};

struct CachedGraph {
    cudaGraphExec_t exec = nullptr;
    int kernels = 0;
    int seen = 0;
};

}  // namespace

// Scratch of the persistent decode launch.  One per tc_stream: two streams may submit different
// lists without waiting for each other, and the kernel reads its table, tensor maps, counter and
// accumulators for as long as it runs.
struct DecodeSite {
    tcb::MegaOp* host = nullptr;          // pinned copy of the table that is on the device
    tcb::MegaOp* dev = nullptr;
    unsigned char* maps_host = nullptr;   // pinned: one tensor map per operation
    unsigned char* maps_dev = nullptr;
    float* pool = nullptr;                // fp32 accumulators, all zero between launches
    size_t pool_floats = 0;
    unsigned long long* counter = nullptr;   // grid-barrier arrival counter
    unsigned long long base = 0;             // what all earlier launches add up to
    int uploaded = 0;                        // table entries currently valid on the device
    tcb::DecodePlan plan;
    // tensor parallel (tcx_stream_tp_export / _connect): the other ranks' pools and counters,
    // opened from their CUDA IPC handles
    int n_ranks = 1, rank = 0;
    float* peer_pool[tcb::kDecodeMaxRanks] = {};
    unsigned long long* peer_counter[tcb::kDecodeMaxRanks] = {};
    std::vector<tcb::DecodeTpOp> tp_ops;
};

struct tc_stream {
    tc_context* owner;
    cudaStream_t s;
    std::vector<RecordedOp> pending;
    std::unordered_map<uint64_t, CachedGraph> cache;
    DecodeSite site;
    bool persistent = true;               // qualifying lists may run as one persistent launch
    std::vector<tcb::MegaOp> table;       // planning scratch, kept to avoid reallocation
    std::vector<tcb::DecodeSpan> spans;
    std::vector<tcb::GemvQArgs> args;
    std::vector<tcb::GemvQArgs> planned;  // the list the table on the device was planned from
};

namespace {

tc_context* g_ctx = nullptr;
std::mutex g_ctx_mutex;
thread_local tc_backend_t t_last_backend = TC_BACKEND_NONE;
thread_local const char* t_last_kernel = "none";
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_variant{tcb::VARIANT_AUTO};

bool env_flag(const char* name, bool dflt) {
    const char* v = std::getenv(name);
    if (!v || !v[0]) return dflt;
    return v[0] != '0';
}

bool trace_enabled() {
    static const bool on = env_flag("TC_TRACE", false);
    return on;
}

// lib/core/trace.cpp:22-37 - remember the backend on success, optional one-line trace.
tc_status_t record(const char* op, tc_status_t st) {
    if (st == TC_OK) t_last_backend = TC_BACKEND_CUDA;
    if (trace_enabled()) {
        std::fprintf(stderr, "[tensorcore] trace op=%s status=%s backend=%s\n", op ? op : "?",
                     tc_status_string(st), tc_backend_name(tc_last_backend()));
    }
    return st;
}

tc_status_t from_cuda(cudaError_t e, tc_status_t fallback) {
    if (e == cudaSuccess) return TC_OK;
    if (e == cudaErrorMemoryAllocation) return TC_ERR_ALLOC;
    if (trace_enabled())
        std::fprintf(stderr, "[tensorcore] cuda error: %s\n", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return fallback;
}

bool checked_mul(size_t a, size_t b, size_t* out) {
    if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
    *out = a * b;
    return true;
}

bool matrix_bytes(int rows, int cols, size_t elem, size_t* out) {
    size_t n = 0;
    if (rows <= 0 || cols <= 0) return false;
    if (!checked_mul(static_cast<size_t>(rows), static_cast<size_t>(cols), &n)) return false;
    return checked_mul(n, elem, out);
}

// lib/core/device_cpu.cpp:236-243
tc_status_t validate(tc_context* ctx, const tc_buffer* b, size_t min_bytes) {
    if (!ctx || !b || !b->dptr) return TC_ERR_INVALID_ARG;
    if (b->owner != ctx) return TC_ERR_INVALID_ARG;
    if (min_bytes > b->bytes) return TC_ERR_INVALID_SHAPE;
    return TC_OK;
}

bool staged(const tc_buffer* b) { return b->kind == BUF_WRAP_HOST || b->kind == BUF_HOST_SHADOW; }
bool managed(const tc_buffer* b) { return b->kind == BUF_MANAGED || b->kind == BUF_WRAP_MANAGED; }

// Scratch of the dense fused GEMV (partial sums of the K ranges, one ticket counter per column
// strip), one per CUDA stream: calls on a stream are ordered, calls on different streams must not
// share it.  Grown on demand, freed when the context goes.
struct DenseScratch { float* f = nullptr; size_t nf = 0; int* c = nullptr; size_t nc = 0; void* norm = nullptr; size_t norm_bytes = 0;
                      void* dq = nullptr; size_t dq_bytes = 0; };
std::mutex g_dense_mutex;
std::unordered_map<cudaStream_t, DenseScratch> g_dense;

void dense_scratch_for(tc_context* ctx, cudaStream_t st, tcb::DenseNormGemvArgs* a) {
    size_t nf = 0, nc = 0;
    tcb::dense_norm_gemv_scratch(a->M, a->N, a->K, ctx->sm_count, &nf, &nc);
    std::lock_guard<std::mutex> lock(g_dense_mutex);
    if (g_dense.size() > 32 && g_dense.find(st) == g_dense.end()) {
        // many short-lived streams: start over rather than keep scratch for streams that are gone
        cudaDeviceSynchronize();
        for (auto& kv : g_dense) {
            if (kv.second.f) cudaFree(kv.second.f);
            if (kv.second.c) cudaFree(kv.second.c);
            if (kv.second.norm) cudaFree(kv.second.norm);
            if (kv.second.dq) cudaFree(kv.second.dq);
        }
        g_dense.clear();
    }
    DenseScratch& d = g_dense[st];
    if (d.nf < nf || d.nc < nc) {
        cudaStreamSynchronize(st);        // an earlier call on this stream may still use the old one
        if (d.f) cudaFree(d.f);
        if (d.c) cudaFree(d.c);
        d.f = nullptr; d.c = nullptr; d.nf = 0; d.nc = 0;
        const size_t wf = nf + nf / 2, wc = nc * 2;
        if (cudaMalloc(reinterpret_cast<void**>(&d.f), wf * sizeof(float)) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void**>(&d.c), wc * sizeof(int)) != cudaSuccess ||
            cudaMemset(d.c, 0, wc * sizeof(int)) != cudaSuccess) {
            (void)cudaGetLastError();
            if (d.f) cudaFree(d.f);
            if (d.c) cudaFree(d.c);
            d.f = nullptr; d.c = nullptr; d.nf = 0; d.nc = 0;
            return;                        // the launcher falls back to the kernel that needs none
        }
        d.nf = wf;
        d.nc = wc;
    }
    a->scratch = d.f; a->scratch_floats = d.nf; a->counters = d.c; a->counters_n = d.nc;
}
// Room for the normalised rows of the batched fused RMSNorm GEMV (the tensor-core kernel reads them as
// plain fp16 activations).
// Whether the call is prefill-sized: its weights are dequantised once and multiplied as a GEMM.
bool dequant_gemm_wanted(const tcb::GemvQArgs& a) {
    return a.M >= tcb::gemm_min_rows(a.fmt) && !a.x_f32 && !a.y_f32 && a.K % 32 == 0 &&
           static_cast<size_t>(a.N) * a.K * 2 <= (static_cast<size_t>(3) << 29);      // at most 1.5 GB of scratch
}
size_t norm_scratch_need(const tcb::GemvQArgs& a) {
    if (!a.gamma || a.x_f32) return 0;
    if (dequant_gemm_wanted(a)) return static_cast<size_t>(a.M) * a.K * 2 + static_cast<size_t>(a.M) * 4;
    if (a.fmt != 0 || !tcb::batched_tc_rows(a.M, a.N, a.K) || a.K % 256 != 0) return 0;
    const size_t rows = a.M < 32 ? a.M : 32;
    return rows * static_cast<size_t>(a.K) * 2 + rows * 4;
}
void norm_scratch_for(cudaStream_t st, size_t need, tcb::GemvQArgs* a) {
    if (need == 0) return;
    std::lock_guard<std::mutex> lock(g_dense_mutex);
    DenseScratch& d = g_dense[st];
    if (d.norm_bytes < need) {
        cudaStreamSynchronize(st);        // an earlier call on this stream may still use the old one
        if (d.norm) cudaFree(d.norm);
        d.norm = nullptr;
        d.norm_bytes = 0;
        const size_t want = need > (1u << 20) ? need + need / 2 : (1u << 20);
        if (cudaMalloc(&d.norm, want) != cudaSuccess) {
            (void)cudaGetLastError();
            d.norm = nullptr;
            return;                        // the launcher then uses the kernels that need no scratch
        }
        d.norm_bytes = want;
    }
    a->norm_scratch = d.norm;
    a->norm_scratch_bytes = d.norm_bytes;
}
// Room for the normalised rows of a dense fused norm + GEMV call with five rows or more.
void dense_norm_rows_for(cudaStream_t st, tcb::DenseNormGemvArgs* a) {
    if (a->M < 5) return;
    tcb::GemvQArgs tmp;
    norm_scratch_for(st, static_cast<size_t>(a->M) * a->K * 2 + static_cast<size_t>(a->M) * 8, &tmp);
    a->norm_scratch = tmp.norm_scratch;
    a->norm_scratch_bytes = tmp.norm_scratch_bytes;
}
// Room for the weights as fp16 of a prefill-sized quantized GEMV on this stream (grown on demand; a
// call that finds none keeps the kernels that stream the blocks).
void dequant_scratch_for(cudaStream_t st, size_t need, tcb::GemvQArgs* a) {
    if (need == 0) return;
    std::lock_guard<std::mutex> lock(g_dense_mutex);
    DenseScratch& d = g_dense[st];
    if (d.dq_bytes < need) {
        cudaStreamSynchronize(st);        // an earlier call on this stream may still use the old one
        if (d.dq) cudaFree(d.dq);
        d.dq = nullptr;
        d.dq_bytes = 0;
        if (cudaMalloc(&d.dq, need) != cudaSuccess) {
            (void)cudaGetLastError();
            d.dq = nullptr;
            return;
        }
        d.dq_bytes = need;
    }
    a->dequant_scratch = d.dq;
    a->dequant_scratch_bytes = d.dq_bytes;
}
size_t dequant_scratch_need(const tcb::GemvQArgs& a) {
    return dequant_gemm_wanted(a) ? static_cast<size_t>(a.N) * a.K * 2 : 0;
}
void free_dense_scratch() {
    std::lock_guard<std::mutex> lock(g_dense_mutex);
    for (auto& kv : g_dense) {
        if (kv.second.f) cudaFree(kv.second.f);
        if (kv.second.c) cudaFree(kv.second.c);
        if (kv.second.norm) cudaFree(kv.second.norm);
        if (kv.second.dq) cudaFree(kv.second.dq);
    }
    g_dense.clear();
}

LaunchEnv make_env(tc_context* ctx, bool allow_pdl) {
    LaunchEnv e;
    e.sm_count = ctx->sm_count;
    e.smem_optin = ctx->smem_optin;
    e.pdl = allow_pdl && ctx->pdl;
    e.variant = g_variant.load();
    e.err_word = ctx->err_dev;
    return e;
}

// Makes `bytes` of an input buffer current on the device before a kernel reads it.
cudaError_t prepare_input(tc_context* ctx, tc_buffer* b, size_t bytes, cudaStream_t st) {
    if (staged(b)) return cudaMemcpyAsync(b->dptr, b->hptr, bytes, cudaMemcpyHostToDevice, st);
    if (managed(b) && b->prefetch_hint) {
        b->prefetch_hint = false;
        if (ctx->managed_ok) (void)cudaMemPrefetchAsync(b->dptr, b->bytes, ctx->device, st);
        (void)cudaGetLastError();  // a refused hint is not an error: pages fault in on demand
    }
    return cudaSuccess;
}
cudaError_t prepare_output(tc_context* ctx, tc_buffer* b, cudaStream_t st) {
    if (managed(b) && b->prefetch_hint) {
        b->prefetch_hint = false;
        if (ctx->managed_ok) (void)cudaMemPrefetchAsync(b->dptr, b->bytes, ctx->device, st);
        (void)cudaGetLastError();
    }
    return cudaSuccess;
}
cudaError_t finish_output(tc_buffer* b, size_t bytes, cudaStream_t st) {
    if (staged(b)) return cudaMemcpyAsync(b->hptr, b->dptr, bytes, cudaMemcpyDeviceToHost, st);
    return cudaSuccess;
}

tc_status_t check_device_error(tc_context* ctx) {
    if (ctx->err_host && *reinterpret_cast<volatile uint32_t*>(ctx->err_host) != 0) {
        return TC_ERR_INTERNAL;  // left set; tcx_take_device_error reads and clears it
    }
    return TC_OK;
}

cudaError_t bind_device(tc_context* ctx) { return cudaSetDevice(ctx->device); }

tc_status_t setup_device(tc_context* ctx, int device) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return TC_ERR_NO_DEVICE;
    if (prop.major != 10) return TC_ERR_NO_DEVICE;  // kernels are built for sm_100a only
    if (cudaSetDevice(device) != cudaSuccess) return TC_ERR_NO_DEVICE;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    int optin = 0;
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    ctx->smem_optin = optin;
    int mm = 0, cma = 0;
    cudaDeviceGetAttribute(&mm, cudaDevAttrManagedMemory, device);
    cudaDeviceGetAttribute(&cma, cudaDevAttrConcurrentManagedAccess, device);
    ctx->managed_ok = (mm != 0) && (cma != 0) && env_flag("TC_MANAGED_MAP", true);

    std::memset(&ctx->info, 0, sizeof(ctx->info));
    ctx->info.family = TC_FAMILY_UNKNOWN;
    std::strncpy(ctx->info.name, "cuda", sizeof(ctx->info.name) - 1);
    ctx->info.max_buffer_bytes = prop.totalGlobalMem;
    ctx->info.recommended_working_set_bytes = prop.totalGlobalMem;
    ctx->info.max_threadgroup_memory = static_cast<uint32_t>(optin);
    ctx->info.max_threads_per_threadgroup = static_cast<uint32_t>(prop.maxThreadsPerBlock);
    ctx->info.thread_execution_width = static_cast<uint32_t>(prop.warpSize);
    ctx->info.unified_memory = false;
    ctx->info.supports_fp64_native = true;

    if (cudaStreamCreateWithFlags(&ctx->stream0, cudaStreamNonBlocking) != cudaSuccess)
        return TC_ERR_INTERNAL;
    if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->err_host), sizeof(uint32_t),
                      cudaHostAllocMapped) != cudaSuccess)
        return TC_ERR_ALLOC;
    *ctx->err_host = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->err_dev), ctx->err_host, 0) !=
        cudaSuccess)
        return TC_ERR_INTERNAL;
    if (tcb::init_gemv_kernels(optin) != cudaSuccess) return TC_ERR_INTERNAL;
    return TC_OK;
}

void teardown_device(tc_context* ctx) {
    if (ctx->stream0) cudaStreamDestroy(ctx->stream0);
    if (ctx->err_host) cudaFreeHost(ctx->err_host);
    if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
    free_dense_scratch();
    ctx->attn_scratch = nullptr;
    ctx->attn_scratch_floats = 0;
    ctx->stream0 = nullptr;
    ctx->err_host = nullptr;
    ctx->err_dev = nullptr;
}

uint64_t fnv1a(uint64_t h, const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Strings
// ---------------------------------------------------------------------------------------
extern "C" const int tensorcore_abi_version = 1;

extern "C" const char* tc_version(void) { return "tensorcore 0.1.22"; }

extern "C" const char* tc_status_string(tc_status_t s) {
    switch (s) {
        case TC_OK: return "ok";
        case TC_ERR_NOT_INITIALIZED: return "context not initialized";
        case TC_ERR_ALREADY_INITIALIZED: return "context already initialized";
        case TC_ERR_NO_DEVICE: return "no Metal device available";
        case TC_ERR_UNSUPPORTED_FAMILY: return "operation unsupported on this GPU family";
        case TC_ERR_UNSUPPORTED_DTYPE: return "dtype unsupported on this GPU family";
        case TC_ERR_INVALID_SHAPE: return "invalid tensor shape";
        case TC_ERR_INVALID_ARG: return "invalid argument";
        case TC_ERR_ALLOC: return "allocation failure";
        case TC_ERR_KERNEL_NOT_FOUND: return "kernel not in metallib";
        case TC_ERR_PIPELINE: return "MTLComputePipelineState creation failed";
        case TC_ERR_DISPATCH: return "command-buffer dispatch failed";
        case TC_ERR_INTERNAL: return "internal error";
    }
    return "unknown status";
}

extern "C" const char* tc_dtype_name(tc_dtype_t d) {
    static const char* const names[] = {"f16", "bf16", "f32", "i8", "i32",
                                        "f64", "sf64", "df64", "fp24", "fp53"};
    const int i = static_cast<int>(d);
    return (i >= 0 && i < 10) ? names[i] : "?";
}

extern "C" const char* tc_backend_name(tc_backend_t b) {
    static const char* const names[] = {"none", "simdgroup_matrix", "tensorops_m5", "mps",
                                        "accelerate_cpu", "sf64_emulated", "ozaki_ii",
                                        "portable_cpu", "metal_compute", "cuda", "hip"};
    const int i = static_cast<int>(b);
    return (i >= 0 && i <= 10) ? names[i] : "?";
}

extern "C" tc_backend_t tc_last_backend(void) { return t_last_backend; }
extern "C" const char* tc_cuda_last_kernel_name(void) { return t_last_kernel; }

// ---------------------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tc_init(tc_context** out_ctx) {
    if (!out_ctx) return TC_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (g_ctx) {
        g_ctx->ref.fetch_add(1);
        *out_ctx = g_ctx;
        return TC_ERR_ALREADY_INITIALIZED;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return TC_ERR_NO_DEVICE;
    }
    int device = 0;
    if (const char* v = std::getenv("TC_CUDA_DEVICE")) device = std::atoi(v);
    else if (cudaGetDevice(&device) != cudaSuccess) device = 0;
    if (device < 0 || device >= count) return TC_ERR_NO_DEVICE;

    tc_context* ctx = new (std::nothrow) tc_context();
    if (!ctx) return TC_ERR_ALLOC;
    ctx->ref.store(1);
    ctx->stream0 = nullptr;
    ctx->err_host = nullptr;
    ctx->err_dev = nullptr;
    ctx->attn_scratch = nullptr;
    ctx->attn_scratch_floats = 0;
    if (const char* v = std::getenv("TC_GEMV_VARIANT")) (void)tcx_set_gemv_variant(v);
    ctx->mega_on = env_flag("TC_MEGA", true);
    ctx->pdl = env_flag("TC_PDL", true);
    ctx->graphs = env_flag("TC_STREAM_GRAPH", true);
    const tc_status_t st = setup_device(ctx, device);
    if (st != TC_OK) {
        teardown_device(ctx);
        delete ctx;
        return st;
    }
    g_ctx = ctx;
    *out_ctx = ctx;
    return TC_OK;
}

extern "C" tc_status_t tc_shutdown(tc_context* ctx) {
    if (!ctx) return TC_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (ctx != g_ctx) return TC_ERR_INVALID_ARG;
    if (ctx->ref.fetch_sub(1) > 1) return TC_OK;
    g_ctx = nullptr;
    bind_device(ctx);
    cudaDeviceSynchronize();
    teardown_device(ctx);
    delete ctx;
    return TC_OK;
}

extern "C" tc_status_t tc_device_info_get(tc_context* ctx, tc_device_info* out_info) {
    if (!ctx || !out_info) return TC_ERR_INVALID_ARG;
    *out_info = ctx->info;
    return TC_OK;
}

// --- tc_cuda_* ---------------------------------------------------------------------------
static bool fill_cuda_info(int index, tc_cuda_device_info* out) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || index >= count) {
        (void)cudaGetLastError();
        return false;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, index) != cudaSuccess) return false;
    std::memset(out, 0, sizeof(*out));
    std::strncpy(out->device_name, prop.name, sizeof(out->device_name) - 1);
    std::snprintf(out->compute_capability, sizeof(out->compute_capability), "%d.%d", prop.major,
                  prop.minor);
    out->major = prop.major;
    out->minor = prop.minor;
    out->global_memory_bytes = prop.totalGlobalMem;
    out->shared_memory_per_block = prop.sharedMemPerBlock;
    out->multiprocessor_count = static_cast<uint32_t>(prop.multiProcessorCount);
    out->max_threads_per_block = static_cast<uint32_t>(prop.maxThreadsPerBlock);
    out->warp_size = static_cast<uint32_t>(prop.warpSize);
    out->supports_fp16 = (prop.major > 5) || (prop.major == 5 && prop.minor >= 3);
    out->supports_bf16 = prop.major >= 8;
    out->supports_int8_tensor_core = (prop.major > 7) || (prop.major == 7 && prop.minor >= 2);
    out->supports_tf32 = prop.major >= 8;
    out->unified_memory = prop.integrated != 0;
    return true;
}

extern "C" tc_status_t tc_cuda_init(tc_context* ctx) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    return TC_OK;  // tc_init already bound the device
}

extern "C" int tc_cuda_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return count;
}

extern "C" tc_status_t tc_cuda_device_at(int index, tc_cuda_device_info* out_info) {
    if (index < 0 || !out_info) return TC_ERR_INVALID_ARG;
    return fill_cuda_info(index, out_info) ? TC_OK : TC_ERR_INVALID_ARG;
}

extern "C" tc_status_t tc_cuda_select_device(tc_context* ctx, int index) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (index < 0 || index >= tc_cuda_device_count()) return TC_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (index == ctx->device) return from_cuda(bind_device(ctx), TC_ERR_INTERNAL);
    // Buffers and streams created on the old device keep working only there; like the
    // reference, switching is meant to happen before any allocation.
    bind_device(ctx);
    cudaDeviceSynchronize();
    teardown_device(ctx);
    return setup_device(ctx, index);
}

// ---------------------------------------------------------------------------------------
// Buffers
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tc_buffer_alloc(tc_context* ctx, size_t bytes, tc_buffer** out) {
    if (!ctx || !out || bytes == 0) return TC_ERR_INVALID_ARG;
    tc_buffer* b = new (std::nothrow) tc_buffer();
    if (!b) return TC_ERR_ALLOC;
    bind_device(ctx);
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess || !p) {
        (void)cudaGetLastError();
        delete b;
        return TC_ERR_ALLOC;
    }
    b->dptr = p;
    b->hptr = nullptr;
    b->bytes = bytes;
    b->owner = ctx;
    b->kind = BUF_DEVICE;
    b->prefetch_hint = false;
    *out = b;
    return TC_OK;
}

extern "C" tc_status_t tc_buffer_from_ptr(tc_context* ctx, void* ptr, size_t bytes,
                                          tc_buffer** out) {
    if (!ctx || !ptr || !out || bytes == 0) return TC_ERR_INVALID_ARG;
    tc_buffer* b = new (std::nothrow) tc_buffer();
    if (!b) return TC_ERR_ALLOC;
    bind_device(ctx);
    cudaPointerAttributes at;
    std::memset(&at, 0, sizeof(at));
    cudaMemoryType type = cudaMemoryTypeUnregistered;
    if (cudaPointerGetAttributes(&at, ptr) == cudaSuccess) type = at.type;
    else (void)cudaGetLastError();
    b->bytes = bytes;
    b->owner = ctx;
    b->prefetch_hint = false;
    b->hptr = nullptr;
    if (type == cudaMemoryTypeDevice) {
        b->kind = BUF_WRAP_DEVICE;
        b->dptr = ptr;
    } else if (type == cudaMemoryTypeManaged) {
        b->kind = BUF_WRAP_MANAGED;
        b->dptr = ptr;
        b->prefetch_hint = true;
    } else {
        void* mirror = nullptr;
        if (cudaMalloc(&mirror, bytes) != cudaSuccess || !mirror) {
            (void)cudaGetLastError();
            delete b;
            return TC_ERR_ALLOC;
        }
        b->kind = BUF_WRAP_HOST;
        b->dptr = mirror;
        b->hptr = ptr;
    }
    *out = b;
    return TC_OK;
}

extern "C" tc_status_t tc_buffer_free(tc_context* ctx, tc_buffer* buf) {
    if (!ctx || !buf || buf->owner != ctx) return TC_ERR_INVALID_ARG;
    bind_device(ctx);
    switch (buf->kind) {
        case BUF_DEVICE:
        case BUF_MANAGED:
        case BUF_WRAP_HOST:
            if (buf->dptr) cudaFree(buf->dptr);  // cudaFree waits for work that uses the memory
            break;
        case BUF_HOST_SHADOW:
            if (buf->dptr) cudaFree(buf->dptr);
            if (buf->hptr) cudaFreeHost(buf->hptr);
            break;
        default:
            break;
    }
    buf->dptr = nullptr;
    buf->owner = nullptr;
    delete buf;
    return TC_OK;
}

// The reference contract: the pointer is stable for the buffer's life and there is no unmap
// (include/tensorcore/device.h:59-62).  A device buffer is converted once, on its first map,
// to managed memory, which the driver keeps coherent page by page; its contents are carried
// over.  Later maps only note that the host may have written, so that the next operation can
// move the pages back in one prefetch instead of by demand faults.
extern "C" tc_status_t tc_buffer_map(tc_buffer* buf, void** out_ptr) {
    if (!buf || !buf->dptr || !out_ptr) return TC_ERR_INVALID_ARG;
    tc_context* ctx = buf->owner;
    if (!ctx) return TC_ERR_INVALID_ARG;
    switch (buf->kind) {
        case BUF_MANAGED:
        case BUF_WRAP_MANAGED:
            buf->prefetch_hint = true;
            *out_ptr = buf->dptr;
            return TC_OK;
        case BUF_WRAP_HOST:
        case BUF_HOST_SHADOW:
            *out_ptr = buf->hptr;
            return TC_OK;
        case BUF_WRAP_DEVICE:
            return TC_ERR_INVALID_ARG;
        case BUF_DEVICE:
            break;
    }
    bind_device(ctx);
    if (cudaDeviceSynchronize() != cudaSuccess) return TC_ERR_INTERNAL;
    if (ctx->managed_ok) {
        void* m = nullptr;
        if (cudaMallocManaged(&m, buf->bytes, cudaMemAttachGlobal) != cudaSuccess || !m) {
            (void)cudaGetLastError();
            return TC_ERR_ALLOC;
        }
        if (cudaMemcpy(m, buf->dptr, buf->bytes, cudaMemcpyDeviceToDevice) != cudaSuccess) {
            cudaFree(m);
            return TC_ERR_INTERNAL;
        }
        (void)cudaMemAdvise(m, buf->bytes, cudaMemAdviseSetPreferredLocation, ctx->device);
        (void)cudaGetLastError();
        cudaFree(buf->dptr);
        buf->dptr = m;
        buf->kind = BUF_MANAGED;
        buf->prefetch_hint = true;
        *out_ptr = m;
        return TC_OK;
    }
    void* h = nullptr;
    if (cudaHostAlloc(&h, buf->bytes, cudaHostAllocDefault) != cudaSuccess || !h) {
        (void)cudaGetLastError();
        return TC_ERR_ALLOC;
    }
    if (cudaMemcpy(h, buf->dptr, buf->bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaFreeHost(h);
        return TC_ERR_INTERNAL;
    }
    buf->hptr = h;
    buf->kind = BUF_HOST_SHADOW;
    *out_ptr = h;
    return TC_OK;
}

extern "C" size_t tc_buffer_size(const tc_buffer* buf) { return buf ? buf->bytes : 0; }

extern "C" tc_status_t tcx_buffer_upload(tc_buffer* buf, size_t offset, const void* src,
                                         size_t bytes) {
    if (!buf || !buf->dptr || !src || !buf->owner) return TC_ERR_INVALID_ARG;
    if (offset > buf->bytes || bytes > buf->bytes - offset) return TC_ERR_INVALID_SHAPE;
    tc_context* ctx = buf->owner;
    bind_device(ctx);
    if (staged(buf)) std::memcpy(static_cast<uint8_t*>(buf->hptr) + offset, src, bytes);
    // A plain cudaMemcpy from pageable memory may return while the DMA into device memory is
    // still in flight, ordered only against the legacy default stream - and the operations of
    // this library run on non-blocking streams.  Copy on the context's stream and wait for it:
    // when this returns the bytes are in place for any stream.
    cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(buf->dptr) + offset, src, bytes,
                                    cudaMemcpyHostToDevice, ctx->stream0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream0);
    return from_cuda(e, TC_ERR_INTERNAL);
}

extern "C" tc_status_t tcx_buffer_download(const tc_buffer* buf, size_t offset, void* dst,
                                           size_t bytes) {
    if (!buf || !buf->dptr || !dst || !buf->owner) return TC_ERR_INVALID_ARG;
    if (offset > buf->bytes || bytes > buf->bytes - offset) return TC_ERR_INVALID_SHAPE;
    tc_context* ctx = buf->owner;
    bind_device(ctx);
    cudaError_t e = cudaMemcpyAsync(dst, static_cast<const uint8_t*>(buf->dptr) + offset, bytes,
                                    cudaMemcpyDeviceToHost, ctx->stream0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream0);
    return from_cuda(e, TC_ERR_INTERNAL);
}

extern "C" tc_status_t tcx_buffer_device_ptr(const tc_buffer* buf, void** out_dptr) {
    if (!buf || !out_dptr) return TC_ERR_INVALID_ARG;
    *out_dptr = buf->dptr;
    return TC_OK;
}

// ---------------------------------------------------------------------------------------
// Streams
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tc_stream_create(tc_context* ctx, tc_stream** out) {
    if (!ctx || !out) return TC_ERR_INVALID_ARG;
    tc_stream* s = new (std::nothrow) tc_stream();
    if (!s) return TC_ERR_ALLOC;
    bind_device(ctx);
    if (cudaStreamCreateWithFlags(&s->s, cudaStreamNonBlocking) != cudaSuccess) {
        (void)cudaGetLastError();
        delete s;
        return TC_ERR_INTERNAL;
    }
    s->owner = ctx;
    *out = s;
    return TC_OK;
}

namespace { void free_decode_site(DecodeSite& d); }

static void drop_graphs(tc_stream* s) {
    for (auto& kv : s->cache)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    s->cache.clear();
}

extern "C" tc_status_t tc_stream_destroy(tc_context* ctx, tc_stream* s) {
    if (!ctx || !s || s->owner != ctx) return TC_ERR_INVALID_ARG;
    bind_device(ctx);
    cudaStreamSynchronize(s->s);
    drop_graphs(s);
    free_decode_site(s->site);
    cudaStreamDestroy(s->s);
    delete s;
    return TC_OK;
}

namespace {

cudaError_t launch_recorded(tc_context* ctx, const RecordedOp& op, cudaStream_t st, bool pdl,
                            int* launches, const char** name) {
    LaunchEnv env = make_env(ctx, pdl);
    return tcb::launch_gemv_q(op.a, env, st, launches, name);
}

constexpr int kMegaMaxOps = 1024;
constexpr size_t kMegaFlagBytes = 256;

void free_decode_site(DecodeSite& d) {
    for (int r = 0; r < d.n_ranks; ++r) {
        if (r == d.rank || d.n_ranks <= 1) continue;
        if (d.peer_pool[r]) cudaIpcCloseMemHandle(d.peer_pool[r]);
        if (d.peer_counter[r]) cudaIpcCloseMemHandle(d.peer_counter[r]);
    }
    if (d.host) cudaFreeHost(d.host);
    if (d.maps_host) cudaFreeHost(d.maps_host);
    if (d.dev) cudaFree(d.dev);
    if (d.maps_dev) cudaFree(d.maps_dev);
    if (d.pool) cudaFree(d.pool);
    if (d.counter) cudaFree(d.counter);
    d = DecodeSite();
}

// After a launch that gave up on a bounded wait the counter and the accumulators hold arbitrary
// values: start over from zero.
void reset_decode_site(DecodeSite& d) {
    if (d.n_ranks > 1) return;   // tensor parallel: the ranks must agree on a restart (tcx_stream_tp_reset)
    if (d.counter) cudaMemset(d.counter, 0, kMegaFlagBytes);
    if (d.pool) cudaMemset(d.pool, 0, d.pool_floats * sizeof(float));
    d.base = 0;
}

bool alloc_decode_site_tables(DecodeSite& d) {
    if (d.host) return true;
    if (cudaHostAlloc(reinterpret_cast<void**>(&d.host), kMegaMaxOps * sizeof(tcb::MegaOp), cudaHostAllocDefault) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&d.dev), kMegaMaxOps * sizeof(tcb::MegaOp)) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void**>(&d.maps_host), kMegaMaxOps * tcb::kDecodeMapBytes, cudaHostAllocDefault) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&d.maps_dev), kMegaMaxOps * tcb::kDecodeMapBytes) != cudaSuccess ||
        (d.counter == nullptr && (cudaMalloc(reinterpret_cast<void**>(&d.counter), kMegaFlagBytes) != cudaSuccess ||
                                  cudaMemset(d.counter, 0, kMegaFlagBytes) != cudaSuccess))) {
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

// Tries to run the whole recorded list as ONE persistent launch (Q4_0, M = 1 lists: a decode
// token).  Returns cudaErrorNotSupported when the list does not qualify; nothing has been
// enqueued in that case.
cudaError_t submit_as_persistent_launch(tc_stream* s, int* launches, const char** name) {
    tc_context* ctx = s->owner;
    const size_t n = s->pending.size();
    if (!ctx->mega_on || !s->persistent || n < 2 || n > static_cast<size_t>(kMegaMaxOps)) return cudaErrorNotSupported;
    for (const RecordedOp& op : s->pending)
        if (op.kind != OP_GEMV_Q || op.a.fmt != tcb::FMT_Q4_0 || op.a.M != 1) return cudaErrorNotSupported;
    DecodeSite& d = s->site;
    if (d.n_ranks > 1) return cudaErrorNotSupported;   // tensor-parallel lists go through tcx_stream_decode_tp
    s->args.resize(n);
    for (size_t i = 0; i < n; ++i) s->args[i] = s->pending[i].a;
    cudaError_t e = cudaSuccess;
    // The same list as last time (a decode loop records the same token over and over): the table
    // on the device, its tensor maps and the plan are still good.
    const bool replay = d.uploaded == static_cast<int>(n) && s->planned.size() == n &&
                        std::memcmp(s->planned.data(), s->args.data(), n * sizeof(tcb::GemvQArgs)) == 0;
    if (replay) {
        tcb::DecodeDevice dev;
        dev.ops = d.dev; dev.maps = d.maps_dev; dev.pool = d.pool; dev.counter = d.counter; dev.base = d.base;
        e = tcb::launch_decode(d.host, d.plan, dev, make_env(ctx, false), s->s);
        if (e == cudaSuccess) {
            tcb::decode_advance(d.plan, ctx->sm_count, 1, &d.base);
            *launches += 1;
            *name = "q4_0_decode_persistent_sm100";
            return e;
        }
        (void)cudaGetLastError();
        s->planned.clear();
        d.uploaded = 0;
        return e == cudaErrorCooperativeLaunchTooLarge ? cudaErrorNotSupported : e;
    }
    s->planned.clear();
    s->table.resize(n);
    s->spans.resize(5 * n);
    tcb::DecodePlan plan;
    e = tcb::plan_decode(s->args.data(), nullptr, static_cast<int>(n), s->spans.data(),
                                     s->table.data(), &plan, 0);
    if (e != cudaSuccess) return cudaErrorNotSupported;
    if (!alloc_decode_site_tables(d)) {
        free_decode_site(d);
        return cudaErrorNotSupported;
    }
    if (plan.pool_floats > d.pool_floats) {
        // a larger accumulator pool: the stream's earlier launches must be done with the old one
        e = cudaStreamSynchronize(s->s);
        if (e != cudaSuccess) return e;
        if (d.pool) cudaFree(d.pool);
        d.pool = nullptr;
        d.pool_floats = 0;
        const size_t want = plan.pool_floats + plan.pool_floats / 2;
        if (cudaMalloc(reinterpret_cast<void**>(&d.pool), want * sizeof(float)) != cudaSuccess ||
            cudaMemset(d.pool, 0, want * sizeof(float)) != cudaSuccess) {
            (void)cudaGetLastError();
            if (d.pool) cudaFree(d.pool);
            d.pool = nullptr;
            return cudaErrorNotSupported;
        }
        d.pool_floats = want;
    }
    const bool same = d.uploaded == static_cast<int>(n) &&
                      std::memcmp(d.host, s->table.data(), n * sizeof(tcb::MegaOp)) == 0;
    if (!same) {
        // the pinned staging copy may still be read by an earlier upload on this stream, and the
        // device copies by an earlier launch
        e = cudaStreamSynchronize(s->s);
        if (e != cudaSuccess) return e;
        std::memcpy(d.host, s->table.data(), n * sizeof(tcb::MegaOp));
        e = tcb::encode_decode_maps(d.host, static_cast<int>(n), d.maps_host);
        if (e != cudaSuccess) { d.uploaded = 0; return cudaErrorNotSupported; }
        e = cudaMemcpyAsync(d.dev, d.host, n * sizeof(tcb::MegaOp), cudaMemcpyHostToDevice, s->s);
        if (e != cudaSuccess) return e;
        e = cudaMemcpyAsync(d.maps_dev, d.maps_host, n * tcb::kDecodeMapBytes, cudaMemcpyHostToDevice, s->s);
        if (e != cudaSuccess) return e;
        d.uploaded = static_cast<int>(n);
    }
    d.plan = plan;
    tcb::DecodeDevice dev;
    dev.ops = d.dev; dev.maps = d.maps_dev; dev.pool = d.pool; dev.counter = d.counter; dev.base = d.base;
    e = tcb::launch_decode(d.host, plan, dev, make_env(ctx, false), s->s);
    if (e == cudaErrorCooperativeLaunchTooLarge) { (void)cudaGetLastError(); return cudaErrorNotSupported; }
    if (e == cudaErrorNotSupported) return e;
    if (e == cudaSuccess) {
        tcb::decode_advance(plan, ctx->sm_count, 1, &d.base);
        *launches += 1;
        *name = "q4_0_decode_persistent_sm100";
        s->planned = s->args;
    }
    return e;
}

// Submits the recorded operations.  Lists without host-staged buffers are replayed as a CUDA
// graph from the second time the identical list (same kernels, pointers and shapes) is seen;
// the first submission of a list, and lists that need staging copies, launch directly.
tc_status_t submit_pending(tc_stream* s) {
    tc_context* ctx = s->owner;
    if (s->pending.empty()) return TC_OK;
    bind_device(ctx);
    bool any_staged = false;
    uint64_t sig = 1469598103934665603ull;
    tcb::GemvQArgs scratch_of;          // the stream's scratch for normalised rows, sized for the widest operation
    {
        size_t need = 0, dq = 0;
        for (const RecordedOp& op : s->pending) {
            const size_t n = norm_scratch_need(op.a);
            need = n > need ? n : need;
            const size_t q = dequant_scratch_need(op.a);
            dq = q > dq ? q : dq;
        }
        norm_scratch_for(s->s, need, &scratch_of);
        dequant_scratch_for(s->s, dq, &scratch_of);
    }
    for (RecordedOp& op : s->pending) {
        op.a.norm_scratch = scratch_of.norm_scratch;
        op.a.norm_scratch_bytes = scratch_of.norm_scratch_bytes;
        op.a.dequant_scratch = scratch_of.dequant_scratch;
        op.a.dequant_scratch_bytes = scratch_of.dequant_scratch_bytes;
        // Device addresses are resolved now, not when the operation was recorded: a first
        // tc_buffer_map between the two moves a buffer to managed storage.
        op.a.X = op.X->dptr;
        op.a.W = static_cast<const uint8_t*>(op.W->dptr);
        op.a.Y = op.Y->dptr;
        op.a.gamma = op.gamma ? op.gamma->dptr : nullptr;
        tc_buffer* bufs[4] = {op.X, op.W, op.Y, op.gamma};
        for (tc_buffer* b : bufs)
            if (b && staged(b)) any_staged = true;
        sig = fnv1a(sig, &op.kind, sizeof(op.kind));
        sig = fnv1a(sig, &op.a, sizeof(op.a));
    }
    const int variant = g_variant.load();
    sig = fnv1a(sig, &variant, sizeof(variant));

    cudaError_t e = cudaSuccess;
    // Host-visible inputs first (staging copies or prefetch hints), outside any graph.
    for (RecordedOp& op : s->pending) {
        if (e == cudaSuccess) e = prepare_input(ctx, op.X, op.x_bytes, s->s);
        if (e == cudaSuccess) e = prepare_input(ctx, op.W, op.w_bytes, s->s);
        if (e == cudaSuccess && op.gamma) e = prepare_input(ctx, op.gamma, op.g_bytes, s->s);
        if (e == cudaSuccess) e = prepare_output(ctx, op.Y, s->s);
    }
    if (e != cudaSuccess) { s->pending.clear(); return from_cuda(e, TC_ERR_DISPATCH); }

    const char* name = t_last_kernel;
    int launches = 0;
    bool done = false;
    if (!any_staged) {
        const cudaError_t me = submit_as_persistent_launch(s, &launches, &name);
        if (me == cudaSuccess) done = true;
        else if (me != cudaErrorNotSupported) e = me;
        else (void)cudaGetLastError();
    }
    if (!done && e == cudaSuccess && ctx->graphs && !any_staged && s->pending.size() > 1) {
        CachedGraph& cg = s->cache[sig];
        if (cg.exec) {
            e = cudaGraphLaunch(cg.exec, s->s);
            launches = cg.kernels;
            done = true;
        } else if (cg.seen >= 1) {
            cudaGraph_t graph = nullptr;
            e = cudaStreamBeginCapture(s->s, cudaStreamCaptureModeThreadLocal);
            if (e == cudaSuccess) {
                cudaError_t le = cudaSuccess;
                int k = 0;
                for (size_t i = 0; i < s->pending.size() && le == cudaSuccess; ++i)
                    le = launch_recorded(ctx, s->pending[i], s->s, i > 0, &k, &name);
                e = cudaStreamEndCapture(s->s, &graph);
                if (le != cudaSuccess) e = le;
                if (e == cudaSuccess && graph) {
                    e = cudaGraphInstantiate(&cg.exec, graph, 0);
                    if (e == cudaSuccess) {
                        cg.kernels = k;
                        e = cudaGraphLaunch(cg.exec, s->s);
                        launches = k;
                        done = true;
                    } else {
                        cg.exec = nullptr;
                    }
                }
                if (graph) cudaGraphDestroy(graph);
            }
            if (!done) {  // capture or instantiation refused: fall through to direct launches
                (void)cudaGetLastError();
                e = cudaSuccess;
                cg.seen = -1000000;  // do not try again for this list
            }
        }
        if (!done) cg.seen += 1;
        if (s->cache.size() > 64) {  // bound the cache: drop everything but keep working
            if (!done) { drop_graphs(s); }
        }
    }
    if (!done) {
        for (size_t i = 0; i < s->pending.size() && e == cudaSuccess; ++i)
            e = launch_recorded(ctx, s->pending[i], s->s, i > 0, &launches, &name);
    }
    if (e == cudaSuccess && any_staged) {
        for (RecordedOp& op : s->pending)
            if (e == cudaSuccess) e = finish_output(op.Y, op.y_bytes, s->s);
    }
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    s->pending.clear();
    return from_cuda(e, TC_ERR_DISPATCH);
}

}  // namespace

extern "C" tc_status_t tcx_stream_flush(tc_stream* s) {
    if (!s) return TC_ERR_INVALID_ARG;
    return submit_pending(s);
}

extern "C" tc_status_t tc_stream_sync(tc_stream* s) {
    if (!s) return TC_ERR_INVALID_ARG;
    tc_status_t st = submit_pending(s);
    const cudaError_t e = cudaStreamSynchronize(s->s);
    if (st == TC_OK) st = from_cuda(e, TC_ERR_DISPATCH);
    if (st == TC_OK) st = check_device_error(s->owner);
    if (st != TC_OK) reset_decode_site(s->site);
    return st;
}

// ---------------------------------------------------------------------------------------
// Tensor-parallel decode: one process per GPU, every rank runs the same list on its shard and
// row-parallel results are summed / row-sharded results gathered inside the persistent kernel by
// adding into every rank's accumulators over NVLink (see include/tensorcore_b200.h).
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tcx_stream_tp_export(tc_stream* s, size_t pool_floats, void* handles_out) {
    if (!s || !handles_out || pool_floats == 0) return TC_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "two handles fill the 128-byte record");
    DecodeSite& d = s->site;
    if (d.pool || d.n_ranks > 1) return TC_ERR_INVALID_ARG;     // before the stream's first decode launch only
    bind_device(s->owner);
    if (cudaMalloc(reinterpret_cast<void**>(&d.pool), pool_floats * sizeof(float)) != cudaSuccess ||
        cudaMemset(d.pool, 0, pool_floats * sizeof(float)) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&d.counter), kMegaFlagBytes) != cudaSuccess ||
        cudaMemset(d.counter, 0, kMegaFlagBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return TC_ERR_ALLOC;
    }
    d.pool_floats = pool_floats;
    cudaIpcMemHandle_t* h = static_cast<cudaIpcMemHandle_t*>(handles_out);
    if (cudaIpcGetMemHandle(&h[0], d.pool) != cudaSuccess || cudaIpcGetMemHandle(&h[1], d.counter) != cudaSuccess) {
        (void)cudaGetLastError();
        return TC_ERR_INTERNAL;
    }
    return from_cuda(cudaDeviceSynchronize(), TC_ERR_INTERNAL);
}

extern "C" tc_status_t tcx_stream_tp_connect(tc_stream* s, int n_ranks, int rank, const void* all_handles) {
    if (!s || !all_handles || n_ranks < 2 || n_ranks > tcb::kDecodeMaxRanks || rank < 0 || rank >= n_ranks)
        return TC_ERR_INVALID_ARG;
    DecodeSite& d = s->site;
    if (!d.pool || !d.counter || d.n_ranks > 1) return TC_ERR_INVALID_ARG;
    bind_device(s->owner);
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(all_handles);
    for (int r = 0; r < n_ranks; ++r) {
        if (r == rank) {
            d.peer_pool[r] = d.pool;
            d.peer_counter[r] = d.counter;
            continue;
        }
        void *pp = nullptr, *pc = nullptr;
        if (cudaIpcOpenMemHandle(&pp, h[2 * r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
            cudaIpcOpenMemHandle(&pc, h[2 * r + 1], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            return TC_ERR_INTERNAL;
        }
        d.peer_pool[r] = static_cast<float*>(pp);
        d.peer_counter[r] = static_cast<unsigned long long*>(pc);
    }
    d.n_ranks = n_ranks;
    d.rank = rank;
    return TC_OK;
}

extern "C" tc_status_t tcx_stream_decode_tp(tc_stream* s, const tcx_decode_tp_op* ops, int n_ops) {
    if (!s || !ops || n_ops <= 0) return TC_ERR_INVALID_ARG;
    if (n_ops > kMegaMaxOps) return TC_ERR_INVALID_SHAPE;
    tc_context* ctx = s->owner;
    DecodeSite& d = s->site;
    if (!d.pool || !d.counter) return TC_ERR_INVALID_ARG;     // tcx_stream_tp_export first
    bind_device(ctx);
    const size_t n = static_cast<size_t>(n_ops);
    s->args.resize(n);
    d.tp_ops.resize(n);
    for (size_t i = 0; i < n; ++i) {
        const tcx_decode_op& o = ops[i].op;
        if (!o.W || !o.X || !o.Y || o.N <= 0 || o.K <= 0) return TC_ERR_INVALID_ARG;
        if ((o.x_dtype != TC_DTYPE_F16 && o.x_dtype != TC_DTYPE_F32) || (o.y_dtype != TC_DTYPE_F16 && o.y_dtype != TC_DTYPE_F32))
            return TC_ERR_UNSUPPORTED_DTYPE;
        tcb::GemvQArgs a;
        std::memset(&a, 0, sizeof(a));
        a.W = static_cast<const uint8_t*>(o.W); a.X = o.X; a.Y = o.Y; a.gamma = o.gamma;
        a.fmt = tcb::FMT_Q4_0; a.M = 1; a.N = o.N; a.K = o.K;
        a.x_f32 = o.x_dtype == TC_DTYPE_F32; a.y_f32 = o.y_dtype == TC_DTYPE_F32; a.eps = o.eps;
        s->args[i] = a;
        tcb::DecodeTpOp t;
        t.peers = ops[i].peers != 0 && d.n_ranks > 1;
        t.y_row0 = ops[i].y_row0; t.y_rows = ops[i].y_rows; t.layout_rows = ops[i].layout_rows;
        t.expect = ops[i].expect;
        d.tp_ops[i] = t;
    }
    cudaError_t e = cudaSuccess;
    const bool replay = d.uploaded == n_ops && s->planned.size() == n &&
                        std::memcmp(s->planned.data(), s->args.data(), n * sizeof(tcb::GemvQArgs)) == 0;
    if (!replay) {
        s->planned.clear();
        s->table.resize(n);
        s->spans.resize(5 * n);
        tcb::DecodePlan plan;
        e = tcb::plan_decode(s->args.data(), d.tp_ops.data(), n_ops, s->spans.data(), s->table.data(), &plan,
                             d.pool_floats, d.n_ranks);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return TC_ERR_INVALID_SHAPE; }
        if (!alloc_decode_site_tables(d)) return TC_ERR_ALLOC;
        e = cudaStreamSynchronize(s->s);
        if (e != cudaSuccess) return from_cuda(e, TC_ERR_DISPATCH);
        std::memcpy(d.host, s->table.data(), n * sizeof(tcb::MegaOp));
        e = tcb::encode_decode_maps(d.host, n_ops, d.maps_host);
        if (e != cudaSuccess) { d.uploaded = 0; (void)cudaGetLastError(); return TC_ERR_INVALID_SHAPE; }
        e = cudaMemcpyAsync(d.dev, d.host, n * sizeof(tcb::MegaOp), cudaMemcpyHostToDevice, s->s);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(d.maps_dev, d.maps_host, n * tcb::kDecodeMapBytes, cudaMemcpyHostToDevice, s->s);
        if (e != cudaSuccess) return from_cuda(e, TC_ERR_DISPATCH);
        d.uploaded = n_ops;
        d.plan = plan;
        s->planned = s->args;
    }
    tcb::DecodeDevice dev;
    dev.ops = d.dev; dev.maps = d.maps_dev; dev.pool = d.pool; dev.counter = d.counter; dev.base = d.base;
    dev.n_ranks = d.n_ranks; dev.rank = d.rank;
    for (int r = 0; r < d.n_ranks; ++r) { dev.peer_pool[r] = d.peer_pool[r]; dev.peer_counter[r] = d.peer_counter[r]; }
    e = tcb::launch_decode(d.host, d.plan, dev, make_env(ctx, false), s->s);
    if (e == cudaErrorNotSupported || e == cudaErrorCooperativeLaunchTooLarge) { (void)cudaGetLastError(); return TC_ERR_INVALID_SHAPE; }
    if (e == cudaSuccess) {
        tcb::decode_advance(d.plan, ctx->sm_count, d.n_ranks, &d.base);
        g_launches.fetch_add(1);
        t_last_kernel = d.n_ranks > 1 ? "q4_0_decode_persistent_tp_sm100" : "q4_0_decode_persistent_sm100";
    }
    return record("tcx_stream_decode_tp", from_cuda(e, TC_ERR_DISPATCH));
}

extern "C" tc_status_t tcx_stream_set_persistent(tc_stream* s, int enable) {
    if (!s) return TC_ERR_INVALID_ARG;
    s->persistent = enable != 0;
    return TC_OK;
}

extern "C" tc_status_t tcx_stream_cuda_handle(const tc_stream* s, void** out) {
    if (!s || !out) return TC_ERR_INVALID_ARG;
    *out = static_cast<void*>(s->s);
    return TC_OK;
}

// ---------------------------------------------------------------------------------------
// Quantized operations
// ---------------------------------------------------------------------------------------
extern "C" size_t tc_quantized_size(tc_quant_t fmt, int N, int K) {
    if (N <= 0 || K <= 0 || K % 32 != 0) return 0;
    const size_t nblocks = static_cast<size_t>(K / 32);
    if (fmt == TC_QUANT_Q4_0) return static_cast<size_t>(N) * nblocks * 18u;
    if (fmt == TC_QUANT_Q8_0) return static_cast<size_t>(N) * nblocks * 34u;
    return 0;
}

extern "C" tc_status_t tc_quantize_weights(tc_context* ctx, const tc_buffer* W_fp16,
                                           tc_buffer* W_quant, tc_quant_t fmt, int N, int K) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!W_fp16 || !W_quant || N <= 0 || K <= 0 || K % 32 != 0) return TC_ERR_INVALID_ARG;
    size_t in_bytes = 0;
    if (!matrix_bytes(N, K, 2, &in_bytes)) return TC_ERR_INVALID_ARG;
    const size_t out_bytes = tc_quantized_size(fmt, N, K);
    if (out_bytes == 0) return TC_ERR_INVALID_ARG;
    tc_status_t st = validate(ctx, W_fp16, in_bytes);
    if (st != TC_OK) return st;
    st = validate(ctx, W_quant, out_bytes);
    if (st != TC_OK) return st;
    if ((reinterpret_cast<uintptr_t>(W_fp16->dptr) & 15u) != 0) return TC_ERR_INVALID_ARG;

    bind_device(ctx);
    tc_buffer* in = const_cast<tc_buffer*>(W_fp16);
    cudaStream_t s0 = ctx->stream0;
    cudaError_t e = prepare_input(ctx, in, in_bytes, s0);
    if (e == cudaSuccess) e = prepare_output(ctx, W_quant, s0);
    int launches = 0;
    const char* name = "none";
    if (e == cudaSuccess)
        e = tcb::launch_quantize(in->dptr, W_quant->dptr, static_cast<int>(fmt), N, K,
                                 make_env(ctx, false), s0, &launches, &name);
    if (e == cudaSuccess) e = finish_output(W_quant, out_bytes, s0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s0);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    return record("tc_quantize_weights", from_cuda(e, TC_ERR_DISPATCH));
}

namespace {

struct GemvCall {
    tc_context* ctx;
    const tc_buffer* X;
    const tc_buffer* gamma;  // null unless fused
    const tc_buffer* W;
    tc_buffer* Y;
    tc_quant_t fmt;
    int M, N, K;
    float eps;
    tc_dtype_t xd, yd;
    bool fused;
};

// Argument checks in the reference's order (lib/ops/quantized_cpu.cpp:171-177, 243-250),
// then either a direct launch + wait (stream == null) or a recording on the stream.
tc_status_t gemv_common(const GemvCall& c, tc_stream* stream, const char* opname) {
    if (!c.ctx) return TC_ERR_NOT_INITIALIZED;
    if (!c.X || !c.W || !c.Y || (c.fused && !c.gamma) || c.M <= 0 || c.N <= 0 || c.K <= 0 ||
        c.K % 32 != 0)
        return TC_ERR_INVALID_ARG;
    if ((c.xd != TC_DTYPE_F16 && c.xd != TC_DTYPE_F32) ||
        (c.yd != TC_DTYPE_F16 && c.yd != TC_DTYPE_F32))
        return TC_ERR_UNSUPPORTED_DTYPE;
    const size_t xs = c.xd == TC_DTYPE_F32 ? 4 : 2, ys = c.yd == TC_DTYPE_F32 ? 4 : 2;
    size_t xb = 0, yb = 0, gb = 0;
    if (!matrix_bytes(c.M, c.K, xs, &xb) || !matrix_bytes(c.M, c.N, ys, &yb))
        return TC_ERR_INVALID_ARG;
    const size_t wb = tc_quantized_size(c.fmt, c.N, c.K);
    if (wb == 0) return TC_ERR_INVALID_ARG;
    tc_status_t st = validate(c.ctx, c.X, xb);
    if (st != TC_OK) return st;
    st = validate(c.ctx, c.W, wb);
    if (st != TC_OK) return st;
    st = validate(c.ctx, c.Y, yb);
    if (st != TC_OK) return st;
    if (c.fused) {
        if (!matrix_bytes(1, c.K, xs, &gb)) return TC_ERR_INVALID_ARG;
        st = validate(c.ctx, c.gamma, gb);
        if (st != TC_OK) return st;
    }
    if (stream && stream->owner != c.ctx) return TC_ERR_INVALID_ARG;

    RecordedOp op;
    op.kind = OP_GEMV_Q;
    op.X = const_cast<tc_buffer*>(c.X);
    op.W = const_cast<tc_buffer*>(c.W);
    op.Y = c.Y;
    op.gamma = c.fused ? const_cast<tc_buffer*>(c.gamma) : nullptr;
    op.x_bytes = xb; op.w_bytes = wb; op.y_bytes = yb; op.g_bytes = gb;
    std::memset(&op.a, 0, sizeof(op.a));  // padding bytes take part in the list signature
    op.a.W = static_cast<const uint8_t*>(c.W->dptr);
    op.a.X = c.X->dptr;
    op.a.Y = c.Y->dptr;
    op.a.gamma = c.fused ? c.gamma->dptr : nullptr;
    op.a.fmt = static_cast<int>(c.fmt);
    op.a.M = c.M; op.a.N = c.N; op.a.K = c.K;
    op.a.x_f32 = c.xd == TC_DTYPE_F32;
    op.a.y_f32 = c.yd == TC_DTYPE_F32;
    op.a.eps = c.eps;

    if (stream) {
        stream->pending.push_back(op);
        return record(opname, TC_OK);
    }
    tc_context* ctx = c.ctx;
    bind_device(ctx);
    cudaStream_t s0 = ctx->stream0;
    cudaError_t e = prepare_input(ctx, op.X, xb, s0);
    if (e == cudaSuccess) e = prepare_input(ctx, op.W, wb, s0);
    if (e == cudaSuccess && op.gamma) e = prepare_input(ctx, op.gamma, gb, s0);
    if (e == cudaSuccess) e = prepare_output(ctx, op.Y, s0);
    int launches = 0;
    const char* name = "none";
    if (e == cudaSuccess) norm_scratch_for(s0, norm_scratch_need(op.a), &op.a);
    if (e == cudaSuccess) dequant_scratch_for(s0, dequant_scratch_need(op.a), &op.a);
    if (e == cudaSuccess) e = launch_recorded(ctx, op, s0, false, &launches, &name);
    if (e == cudaSuccess) e = finish_output(op.Y, yb, s0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s0);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    tc_status_t out = from_cuda(e, TC_ERR_DISPATCH);
    if (out == TC_OK) out = check_device_error(ctx);
    return record(opname, out);
}

}  // namespace

extern "C" tc_status_t tc_gemv_quantized(tc_context* ctx, const tc_buffer* X,
                                         const tc_buffer* W_quant, tc_buffer* Y, tc_quant_t fmt,
                                         int M, int N, int K) {
    GemvCall c{ctx, X, nullptr, W_quant, Y, fmt, M, N, K, 0.f, TC_DTYPE_F16, TC_DTYPE_F16, false};
    return gemv_common(c, nullptr, "tc_gemv_quantized");
}

extern "C" tc_status_t tc_gemv_quantized_async(tc_context* ctx, const tc_buffer* X,
                                               const tc_buffer* W_quant, tc_buffer* Y,
                                               tc_quant_t fmt, int M, int N, int K,
                                               tc_stream* stream) {
    if (!stream) return TC_ERR_INVALID_ARG;
    GemvCall c{ctx, X, nullptr, W_quant, Y, fmt, M, N, K, 0.f, TC_DTYPE_F16, TC_DTYPE_F16, false};
    return gemv_common(c, stream, "tc_gemv_quantized_async");
}

extern "C" tc_status_t tc_fused_rmsnorm_gemv_quantized(tc_context* ctx, const tc_buffer* X,
                                                       const tc_buffer* gamma,
                                                       const tc_buffer* W_quant, tc_buffer* Y,
                                                       tc_quant_t fmt, int M, int N, int K,
                                                       float eps) {
    GemvCall c{ctx, X, gamma, W_quant, Y, fmt, M, N, K, eps, TC_DTYPE_F16, TC_DTYPE_F16, true};
    return gemv_common(c, nullptr, "tc_fused_rmsnorm_gemv_quantized");
}

extern "C" tc_status_t tcx_gemv_quantized_ex(tc_context* ctx, const tc_buffer* X,
                                             const tc_buffer* W_quant, tc_buffer* Y,
                                             tc_quant_t fmt, int M, int N, int K,
                                             tc_dtype_t x_dtype, tc_dtype_t y_dtype,
                                             tc_stream* stream) {
    GemvCall c{ctx, X, nullptr, W_quant, Y, fmt, M, N, K, 0.f, x_dtype, y_dtype, false};
    return gemv_common(c, stream, "tcx_gemv_quantized_ex");
}

extern "C" tc_status_t tcx_fused_rmsnorm_gemv_quantized_ex(
    tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma, const tc_buffer* W_quant,
    tc_buffer* Y, tc_quant_t fmt, int M, int N, int K, float eps, tc_dtype_t x_dtype,
    tc_dtype_t y_dtype, tc_stream* stream) {
    GemvCall c{ctx, X, gamma, W_quant, Y, fmt, M, N, K, eps, x_dtype, y_dtype, true};
    return gemv_common(c, stream, "tcx_fused_rmsnorm_gemv_quantized_ex");
}

// ---------------------------------------------------------------------------------------
// Fused norm + dense fp16 GEMV
// ---------------------------------------------------------------------------------------
static tc_status_t dense_common(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma,
                                const tc_buffer* beta, bool layernorm, const tc_buffer* W,
                                tc_buffer* Y, int M, int N, int K, float eps, const char* opname) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !gamma || (layernorm && !beta) || !W || !Y || M <= 0 || N <= 0 || K <= 0)
        return TC_ERR_INVALID_ARG;
    size_t xb = 0, gb = 0, wb = 0, yb = 0;
    if (!matrix_bytes(M, K, 2, &xb) || !matrix_bytes(1, K, 2, &gb) ||
        !matrix_bytes(K, N, 2, &wb) || !matrix_bytes(M, N, 2, &yb))
        return TC_ERR_INVALID_ARG;
    tc_status_t st = validate(ctx, X, xb);
    if (st != TC_OK) return st;
    st = validate(ctx, gamma, gb);
    if (st != TC_OK) return st;
    if (layernorm) {
        st = validate(ctx, beta, gb);
        if (st != TC_OK) return st;
    }
    st = validate(ctx, W, wb);
    if (st != TC_OK) return st;
    st = validate(ctx, Y, yb);
    if (st != TC_OK) return st;

    bind_device(ctx);
    cudaStream_t s0 = ctx->stream0;
    tc_buffer* bx = const_cast<tc_buffer*>(X);
    tc_buffer* bg = const_cast<tc_buffer*>(gamma);
    tc_buffer* bb = layernorm ? const_cast<tc_buffer*>(beta) : nullptr;
    tc_buffer* bw = const_cast<tc_buffer*>(W);
    cudaError_t e = prepare_input(ctx, bx, xb, s0);
    if (e == cudaSuccess) e = prepare_input(ctx, bg, gb, s0);
    if (e == cudaSuccess && bb) e = prepare_input(ctx, bb, gb, s0);
    if (e == cudaSuccess) e = prepare_input(ctx, bw, wb, s0);
    if (e == cudaSuccess) e = prepare_output(ctx, Y, s0);
    tcb::DenseNormGemvArgs a;
    a.X = bx->dptr; a.gamma = bg->dptr; a.beta = bb ? bb->dptr : nullptr; a.W = bw->dptr;
    a.Y = Y->dptr; a.M = M; a.N = N; a.K = K; a.eps = eps;
    int launches = 0;
    const char* name = "none";
    if (e == cudaSuccess) {
        dense_scratch_for(ctx, s0, &a);
        dense_norm_rows_for(s0, &a);
        e = tcb::launch_dense_norm_gemv(a, make_env(ctx, false), s0, &launches, &name);
    }
    if (e == cudaSuccess) e = finish_output(Y, yb, s0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s0);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    return record(opname, from_cuda(e, TC_ERR_DISPATCH));
}

extern "C" tc_status_t tc_fused_rmsnorm_gemv(tc_context* ctx, const tc_buffer* X,
                                             const tc_buffer* gamma, const tc_buffer* W,
                                             tc_buffer* Y, int M, int N, int K, float eps) {
    return dense_common(ctx, X, gamma, nullptr, false, W, Y, M, N, K, eps, "tc_fused_rmsnorm_gemv");
}

extern "C" tc_status_t tc_fused_layernorm_gemv(tc_context* ctx, const tc_buffer* X,
                                               const tc_buffer* gamma, const tc_buffer* beta,
                                               const tc_buffer* W, tc_buffer* Y, int M, int N,
                                               int K, float eps) {
    return dense_common(ctx, X, gamma, beta, true, W, Y, M, N, K, eps, "tc_fused_layernorm_gemv");
}

// ---------------------------------------------------------------------------------------
// The operations between the GEMVs of a decode step
// ---------------------------------------------------------------------------------------
namespace {

struct StepIo { tc_buffer* b; size_t bytes; bool write; };

// Validates (reference order: lib/ops/training_cpu.cpp:132-141), makes inputs current, runs
// `launch` on the context's stream, copies staged results back and waits.
template <typename Launch>
tc_status_t run_step_op(tc_context* ctx, const char* opname, const char* kname, StepIo* io, int n_io, Launch launch) {
    for (int i = 0; i < n_io; ++i) {
        const tc_status_t st = validate(ctx, io[i].b, io[i].bytes);
        if (st != TC_OK) return st;
    }
    bind_device(ctx);
    cudaStream_t s0 = ctx->stream0;
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < n_io && e == cudaSuccess; ++i)
        e = io[i].write ? prepare_output(ctx, io[i].b, s0) : prepare_input(ctx, io[i].b, io[i].bytes, s0);
    if (e == cudaSuccess) e = launch(s0);
    for (int i = 0; i < n_io && e == cudaSuccess; ++i)
        if (io[i].write) e = finish_output(io[i].b, io[i].bytes, s0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s0);
    g_launches.fetch_add(1);
    t_last_kernel = kname;
    return record(opname, from_cuda(e, TC_ERR_DISPATCH));
}

tc_buffer* mut(const tc_buffer* b) { return const_cast<tc_buffer*>(b); }

}  // namespace

extern "C" tc_status_t tc_rmsnorm_forward(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma,
                                          tc_buffer* Y, tc_buffer* rstd_out, int N, int D, float eps) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !gamma || !Y || !rstd_out || N <= 0 || D <= 0) return TC_ERR_INVALID_ARG;
    const size_t nd = static_cast<size_t>(N) * D * 2;
    StepIo io[] = {{mut(X), nd, false}, {mut(gamma), static_cast<size_t>(D) * 2, false}, {Y, nd, true},
                   {rstd_out, static_cast<size_t>(N) * 4, true}};
    return run_step_op(ctx, "tc_rmsnorm_forward", "rmsnorm_forward_sm100", io, 4, [&](cudaStream_t st) {
        return tcb::launch_norm_forward(X->dptr, gamma->dptr, nullptr, Y->dptr, nullptr,
                                        static_cast<float*>(rstd_out->dptr), N, D, eps, st);
    });
}

extern "C" tc_status_t tc_layernorm_forward(tc_context* ctx, const tc_buffer* X, const tc_buffer* gamma,
                                            const tc_buffer* beta, tc_buffer* Y, tc_buffer* mean_out,
                                            tc_buffer* rstd_out, int N, int D, float eps) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !gamma || !beta || !Y || !mean_out || !rstd_out || N <= 0 || D <= 0) return TC_ERR_INVALID_ARG;
    const size_t nd = static_cast<size_t>(N) * D * 2, d2 = static_cast<size_t>(D) * 2, n4 = static_cast<size_t>(N) * 4;
    StepIo io[] = {{mut(X), nd, false}, {mut(gamma), d2, false}, {mut(beta), d2, false}, {Y, nd, true},
                   {mean_out, n4, true}, {rstd_out, n4, true}};
    return run_step_op(ctx, "tc_layernorm_forward", "layernorm_forward_sm100", io, 6, [&](cudaStream_t st) {
        return tcb::launch_norm_forward(X->dptr, gamma->dptr, beta->dptr, Y->dptr,
                                        static_cast<float*>(mean_out->dptr),
                                        static_cast<float*>(rstd_out->dptr), N, D, eps, st);
    });
}

extern "C" tc_status_t tc_swiglu_forward(tc_context* ctx, const tc_buffer* gate, const tc_buffer* up,
                                         tc_buffer* out, int n) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!gate || !up || !out || n <= 0) return TC_ERR_INVALID_ARG;
    const size_t b = static_cast<size_t>(n) * 2;
    StepIo io[] = {{mut(gate), b, false}, {mut(up), b, false}, {out, b, true}};
    return run_step_op(ctx, "tc_swiglu_forward", "swiglu_forward_sm100", io, 3, [&](cudaStream_t st) {
        return tcb::launch_swiglu(gate->dptr, up->dptr, out->dptr, n, st);
    });
}

extern "C" tc_status_t tc_rope_forward(tc_context* ctx, tc_buffer* X, const tc_buffer* cos_t,
                                       const tc_buffer* sin_t, int batch, int heads, int seq, int head_dim) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !cos_t || !sin_t || batch <= 0 || heads <= 0 || seq <= 0 || head_dim <= 0 || head_dim % 2 != 0)
        return TC_ERR_INVALID_ARG;
    const size_t xb = static_cast<size_t>(batch) * heads * seq * head_dim * 2;
    const size_t tb = static_cast<size_t>(seq) * (head_dim / 2) * 4;
    // X is read and written in place: make it current as an input, copy it back as an output
    StepIo io[] = {{X, xb, false}, {mut(cos_t), tb, false}, {mut(sin_t), tb, false}, {X, xb, true}};
    return run_step_op(ctx, "tc_rope_forward", "rope_forward_sm100", io, 4, [&](cudaStream_t st) {
        return tcb::launch_rope(X->dptr, static_cast<const float*>(cos_t->dptr),
                                static_cast<const float*>(sin_t->dptr), batch, heads, seq, head_dim, st);
    });
}

// Attention forward for decode (include/tensorcore/attention.h:54-69; checks in the order of
// lib/ops/attention_cpu.cpp:138-151).  Any seq_q is accepted, but the kernel is a streaming pass
// per query row: it is meant for the one to few rows of a decode step.
extern "C" tc_status_t tc_attention_forward(tc_context* ctx, const tc_attention_desc* d, const tc_buffer* Q,
                                            const tc_buffer* K, const tc_buffer* V, tc_buffer* O, tc_buffer* LSE) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!d || !Q || !K || !V || !O) return TC_ERR_INVALID_ARG;
    if (d->batch <= 0 || d->heads <= 0 || d->seq_q <= 0 || d->seq_kv <= 0 || d->head_dim <= 0) return TC_ERR_INVALID_ARG;
    if (d->io_dtype != TC_DTYPE_F16 || d->accum_dtype != TC_DTYPE_F32) return TC_ERR_UNSUPPORTED_DTYPE;
    if (d->return_lse && !LSE) return TC_ERR_INVALID_ARG;
    const int Hkv = d->kv_heads > 0 ? d->kv_heads : d->heads;
    if (Hkv <= 0 || d->heads % Hkv != 0) return TC_ERR_INVALID_ARG;
    if (d->head_dim > 128) return TC_ERR_INVALID_SHAPE;
    const int B = d->batch, Hq = d->heads, Sq = d->seq_q, Sk = d->seq_kv, D = d->head_dim;
    const float scale = d->softmax_scale > 0 ? d->softmax_scale : 1.0f / std::sqrt(static_cast<float>(D));
    const size_t qb = static_cast<size_t>(B) * Hq * Sq * D * 2, kb = static_cast<size_t>(B) * Hkv * Sk * D * 2;
    const size_t lb = static_cast<size_t>(B) * Hq * Sq * 4;
    StepIo io[6] = {{mut(Q), qb, false}, {mut(K), kb, false}, {mut(V), kb, false}, {O, qb, true}, {LSE, lb, true}, {nullptr, 0, false}};
    const int n_io = LSE ? 5 : 4;
    bind_device(ctx);
    // scratch for the partial softmax states of a row's key chunks, and the ALiBi slopes
    int chunks = 1;
    const long long rows = static_cast<long long>(B) * Hq * Sq;
    if (rows > 0x7fffffffLL) return TC_ERR_INVALID_SHAPE;
    size_t want = tcb::attention_scratch_floats(B, Hq, Hkv, Sq, Sk, D, ctx->sm_count, &chunks);
    const size_t slope_at = want;
    if (d->alibi_slopes) want += static_cast<size_t>(Hq);
    if (want > ctx->attn_scratch_floats) {
        cudaStreamSynchronize(ctx->stream0);
        if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
    free_dense_scratch();
        ctx->attn_scratch = nullptr;
        ctx->attn_scratch_floats = 0;
        if (cudaMalloc(reinterpret_cast<void**>(&ctx->attn_scratch), want * sizeof(float)) != cudaSuccess) {
            (void)cudaGetLastError();
            return record("tc_attention_forward", TC_ERR_ALLOC);
        }
        ctx->attn_scratch_floats = want;
    }
    float* slopes_dev = nullptr;
    if (d->alibi_slopes) {
        slopes_dev = ctx->attn_scratch + slope_at;
        // a small copy from caller memory: staged by the runtime before the call returns
        if (cudaMemcpyAsync(slopes_dev, d->alibi_slopes, static_cast<size_t>(Hq) * sizeof(float),
                            cudaMemcpyHostToDevice, ctx->stream0) != cudaSuccess)
            return record("tc_attention_forward", TC_ERR_DISPATCH);
    }
    int launched = 0;
    const tc_status_t st = run_step_op(ctx, "tc_attention_forward", "attention_decode_sm100", io, n_io, [&](cudaStream_t s0) {
        return tcb::launch_attention_forward(Q->dptr, K->dptr, V->dptr, O->dptr,
                                             LSE ? static_cast<float*>(LSE->dptr) : nullptr,
                                             chunks > 1 ? ctx->attn_scratch : nullptr, slopes_dev, B, Hq, Hkv, Sq, Sk,
                                             D, scale, d->causal, d->window_size, ctx->sm_count, s0, &launched);
    });
    if (launched > 1) g_launches.fetch_add(static_cast<uint64_t>(launched - 1));
    return st;
}

// The same on raw device pointers, asynchronous on the caller's stream (no ALiBi: its slopes would
// have to be staged from host memory).  The scratch for the key chunks belongs to the context:
// launches on different streams must not overlap.
extern "C" tc_status_t tcx_raw_attention_forward(tc_context* ctx, const tc_attention_desc* d, const void* Q,
                                                 const void* K, const void* V, void* O, void* LSE,
                                                 void* cuda_stream) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!d || !Q || !K || !V || !O) return TC_ERR_INVALID_ARG;
    if (d->batch <= 0 || d->heads <= 0 || d->seq_q <= 0 || d->seq_kv <= 0 || d->head_dim <= 0) return TC_ERR_INVALID_ARG;
    if (d->io_dtype != TC_DTYPE_F16 || d->accum_dtype != TC_DTYPE_F32) return TC_ERR_UNSUPPORTED_DTYPE;
    if (d->alibi_slopes) return TC_ERR_UNSUPPORTED_FAMILY;
    const int Hkv = d->kv_heads > 0 ? d->kv_heads : d->heads;
    if (Hkv <= 0 || d->heads % Hkv != 0) return TC_ERR_INVALID_ARG;
    if (d->head_dim > 128) return TC_ERR_INVALID_SHAPE;
    const long long rows = static_cast<long long>(d->batch) * d->heads * d->seq_q;
    if (rows > 0x7fffffffLL) return TC_ERR_INVALID_SHAPE;
    bind_device(ctx);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    int chunks = 1;
    const size_t want = tcb::attention_scratch_floats(d->batch, d->heads, Hkv, d->seq_q, d->seq_kv, d->head_dim,
                                                       ctx->sm_count, &chunks);
    if (want > ctx->attn_scratch_floats) {
        cudaDeviceSynchronize();
        if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
        ctx->attn_scratch = nullptr;
        ctx->attn_scratch_floats = 0;
        if (cudaMalloc(reinterpret_cast<void**>(&ctx->attn_scratch), want * sizeof(float)) != cudaSuccess) {
            (void)cudaGetLastError();
            return record("tcx_raw_attention_forward", TC_ERR_ALLOC);
        }
        ctx->attn_scratch_floats = want;
    }
    const float scale = d->softmax_scale > 0 ? d->softmax_scale : 1.0f / std::sqrt(static_cast<float>(d->head_dim));
    int launched = 0;
    const cudaError_t e = tcb::launch_attention_forward(Q, K, V, O, static_cast<float*>(LSE),
                                                        chunks > 1 ? ctx->attn_scratch : nullptr, nullptr, d->batch,
                                                        d->heads, Hkv, d->seq_q, d->seq_kv, d->head_dim, scale, d->causal,
                                                        d->window_size, ctx->sm_count, st, &launched);
    g_launches.fetch_add(static_cast<uint64_t>(launched));
    t_last_kernel = "attention_decode_sm100";
    return record("tcx_raw_attention_forward", from_cuda(e, TC_ERR_DISPATCH));
}

// The recorded form runs at once, as the reference's CPU backend does (attention_cpu.cpp:280-291).
extern "C" tc_status_t tc_attention_forward_async(tc_context* ctx, const tc_attention_desc* d, const tc_buffer* Q,
                                                  const tc_buffer* K, const tc_buffer* V, tc_buffer* O,
                                                  tc_buffer* LSE, tc_stream* stream) {
    if (!stream) return TC_ERR_INVALID_ARG;
    return tc_attention_forward(ctx, d, Q, K, V, O, LSE);
}

// tc_gemm and tc_gemm_batched (include/tensorcore/gemm.h:45-72; checks as in lib/ops/gemm_cpu.cpp:768-810):
// `batch` products of the same shape, the matrices of consecutive products stride_* elements apart.
static tc_status_t gemm_impl(tc_context* ctx, const tc_gemm_desc* d, const tc_buffer* A, const tc_buffer* B,
                             tc_buffer* C, int batch, long long stride_a, long long stride_b, long long stride_c,
                             const char* opname) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!d || !A || !B || !C || d->M <= 0 || d->N <= 0 || d->K <= 0 || batch <= 0) return TC_ERR_INVALID_ARG;
    const bool f16 = d->a_dtype == TC_DTYPE_F16 && d->b_dtype == TC_DTYPE_F16 && d->c_dtype == TC_DTYPE_F16;
    const bool bf16 = d->a_dtype == TC_DTYPE_BF16 && d->b_dtype == TC_DTYPE_BF16 && d->c_dtype == TC_DTYPE_BF16;
    if ((!f16 && !bf16) || d->accum_dtype != TC_DTYPE_F32) return TC_ERR_UNSUPPORTED_DTYPE;
    if (batch > 1 && (stride_a <= 0 || stride_b <= 0 || stride_c <= 0)) return TC_ERR_INVALID_SHAPE;
    const bool ta = d->transpose_a;
    const bool tb = d->transpose_b;
    // defaults as in lib/ops/gemm_cpu.cpp (effective_ldb): N for B as given, K for B transposed
    const int lda = d->lda ? d->lda : (ta ? d->M : d->K), ldb = d->ldb ? d->ldb : (tb ? d->K : d->N), ldc = d->ldc ? d->ldc : d->N;
    if (lda < (ta ? d->M : d->K) || ldb < (tb ? d->K : d->N) || ldc < d->N) return TC_ERR_INVALID_ARG;
    const size_t a1 = ta ? static_cast<size_t>(d->K - 1) * lda + d->M : static_cast<size_t>(d->M - 1) * lda + d->K;
    const size_t b1 = tb ? static_cast<size_t>(d->N - 1) * ldb + d->K : static_cast<size_t>(d->K - 1) * ldb + d->N;
    const size_t c1 = static_cast<size_t>(d->M - 1) * ldc + d->N;
    if (batch > 1 && (static_cast<size_t>(stride_a) < a1 || static_cast<size_t>(stride_b) < b1 || static_cast<size_t>(stride_c) < c1))
        return TC_ERR_INVALID_SHAPE;
    const size_t nb1 = static_cast<size_t>(batch - 1);
    const size_t ab = (nb1 * static_cast<size_t>(batch > 1 ? stride_a : 0) + a1) * 2;
    const size_t bb = (nb1 * static_cast<size_t>(batch > 1 ? stride_b : 0) + b1) * 2;
    const size_t cb = (nb1 * static_cast<size_t>(batch > 1 ? stride_c : 0) + c1) * 2;
    // beta != 0 reads C as well
    StepIo io[] = {{mut(A), ab, false}, {mut(B), bb, false}, {C, cb, false}, {C, cb, true}};
    bool unsupported = false;
    // A handful of rows (a decode step) takes the row kernel, which adds in the reference's k order;
    // anything larger the tensor cores, when the tiled copies can describe the operands.
    const bool few_rows = d->M <= 4 && !ta && !tb && f16;
    const char* used = few_rows ? "gemm_f16_rows_sm100" : "gemm_f16_tcgen05_sm100";
    int launched = 0;
    const tc_status_t st = run_step_op(ctx, opname, used, io, 4, [&](cudaStream_t s) {
        for (int i = 0; i < batch; ++i) {
            const uint8_t* pa = static_cast<const uint8_t*>(A->dptr) + static_cast<size_t>(i) * (batch > 1 ? stride_a : 0) * 2;
            const uint8_t* pb = static_cast<const uint8_t*>(B->dptr) + static_cast<size_t>(i) * (batch > 1 ? stride_b : 0) * 2;
            uint8_t* pc = static_cast<uint8_t*>(C->dptr) + static_cast<size_t>(i) * (batch > 1 ? stride_c : 0) * 2;
            cudaError_t e = cudaErrorNotSupported;
            if (!few_rows)
                e = tcb::launch_gemm_f16_tc(pa, pb, pc, d->M, d->N, d->K, lda, ldb, ldc, tb, d->alpha, d->beta,
                                            make_env(ctx, false), s, bf16, ta);
            if (e == cudaErrorNotSupported && !ta && !tb && f16) {
                used = "gemm_f16_rows_sm100";
                e = tcb::launch_gemm_f16_rows(pa, pb, pc, d->M, d->N, d->K, lda, ldb, ldc, d->alpha, d->beta, s);
            }
            if (e == cudaErrorNotSupported) { unsupported = true; return cudaSuccess; }
            if (e != cudaSuccess) return e;
            ++launched;
        }
        return cudaSuccess;
    });
    if (launched > 1) g_launches.fetch_add(static_cast<uint64_t>(launched - 1));
    t_last_kernel = used;
    return unsupported ? TC_ERR_UNSUPPORTED_FAMILY : st;
}

extern "C" tc_status_t tc_gemm(tc_context* ctx, const tc_gemm_desc* d, const tc_buffer* A,
                               const tc_buffer* B, tc_buffer* C) {
    return gemm_impl(ctx, d, A, B, C, 1, 0, 0, 0, "tc_gemm");
}

extern "C" tc_status_t tc_gemm_batched(tc_context* ctx, const tc_gemm_batched_desc* bd, const tc_buffer* A,
                                       const tc_buffer* B, tc_buffer* C) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!bd) return TC_ERR_INVALID_ARG;
    return gemm_impl(ctx, &bd->base, A, B, C, bd->batch, bd->stride_a, bd->stride_b, bd->stride_c, "tc_gemm_batched");
}

// include/tensorcore/gemm.h:52-58.  The recorded form runs at once (as the reference's CPU backend does).
extern "C" tc_status_t tc_gemm_async(tc_context* ctx, const tc_gemm_desc* d, const tc_buffer* A,
                                     const tc_buffer* B, tc_buffer* C, tc_stream* stream) {
    if (!stream) return TC_ERR_INVALID_ARG;
    return tc_gemm(ctx, d, A, B, C);
}

// ---------------------------------------------------------------------------------------
// Collectives (include/tensorcore/distributed.h:51-87) over NCCL, one process per GPU
// ---------------------------------------------------------------------------------------
struct tc_dist_ctx {
    tc_context* ctx;
    tcb::DistComm* comm;
};

namespace {
tc_status_t dist_status(int rc) {
    switch (rc) {
        case 0: return TC_OK;
        case -1: return TC_ERR_INVALID_ARG;
        case -2: return TC_ERR_UNSUPPORTED_FAMILY;    // no NCCL library on this machine
        case -3: return TC_ERR_DISPATCH;              // the ranks did not find each other
        default: return TC_ERR_INTERNAL;
    }
}
size_t dist_elem(tc_dtype_t t) { return t == TC_DTYPE_F16 ? 2 : (t == TC_DTYPE_F32 ? 4 : 0); }

template <typename Launch>
tc_status_t run_collective(tc_dist_ctx* d, const char* opname, StepIo* io, int n_io, Launch launch) {
    tc_context* ctx = d->ctx;
    for (int i = 0; i < n_io; ++i) {
        const tc_status_t st = validate(ctx, io[i].b, io[i].bytes);
        if (st != TC_OK) return st;
    }
    bind_device(ctx);
    cudaStream_t s0 = ctx->stream0;
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < n_io && e == cudaSuccess; ++i)
        e = io[i].write ? prepare_output(ctx, io[i].b, s0) : prepare_input(ctx, io[i].b, io[i].bytes, s0);
    if (e != cudaSuccess) return from_cuda(e, TC_ERR_DISPATCH);
    const int rc = launch(s0);
    if (rc != 0) return dist_status(rc);
    for (int i = 0; i < n_io && e == cudaSuccess; ++i)
        if (io[i].write) e = finish_output(io[i].b, io[i].bytes, s0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s0);
    return record(opname, from_cuda(e, TC_ERR_DISPATCH));
}
}  // namespace

extern "C" tc_status_t tc_dist_init(tc_context* tc, tc_dist_backend_t backend, int world_size, int rank,
                                    const char* rendezvous_url, tc_dist_ctx** out) {
    if (!tc) return TC_ERR_NOT_INITIALIZED;
    if (!out || world_size < 1 || rank < 0 || rank >= world_size) return TC_ERR_INVALID_ARG;
    if (backend != TC_DIST_SINGLE && backend != TC_DIST_RING && backend != TC_DIST_GLOO) return TC_ERR_INVALID_ARG;
    if (backend == TC_DIST_SINGLE && world_size != 1) return TC_ERR_INVALID_ARG;
    if (world_size > 1 && !rendezvous_url) return TC_ERR_INVALID_ARG;
    bind_device(tc);
    tc_dist_ctx* d = new (std::nothrow) tc_dist_ctx();
    if (!d) return TC_ERR_ALLOC;
    d->ctx = tc;
    d->comm = nullptr;
    const int rc = tcb::dist_create(world_size, rank, rendezvous_url, &d->comm);
    if (rc != 0) { delete d; return dist_status(rc); }
    *out = d;
    return TC_OK;
}

extern "C" tc_status_t tc_dist_finalize(tc_dist_ctx* d) {
    if (!d) return TC_ERR_INVALID_ARG;
    bind_device(d->ctx);
    cudaStreamSynchronize(d->ctx->stream0);
    tcb::dist_destroy(d->comm);
    delete d;
    return TC_OK;
}

extern "C" int tc_dist_world_size(const tc_dist_ctx* d) { return d ? tcb::dist_world(d->comm) : 0; }
extern "C" int tc_dist_rank(const tc_dist_ctx* d) { return d ? tcb::dist_rank(d->comm) : 0; }

extern "C" tc_status_t tc_allreduce(tc_dist_ctx* d, tc_buffer* buf, size_t num_elements, tc_dtype_t dtype,
                                    tc_reduce_op_t op) {
    if (!d || !buf || num_elements == 0) return TC_ERR_INVALID_ARG;
    if (dist_elem(dtype) == 0) return TC_ERR_UNSUPPORTED_DTYPE;
    StepIo io[] = {{buf, num_elements * dist_elem(dtype), false}, {buf, num_elements * dist_elem(dtype), true}};
    return run_collective(d, "tc_allreduce", io, 2, [&](cudaStream_t st) {
        return tcb::dist_allreduce(d->comm, buf->dptr, num_elements, static_cast<int>(dtype), static_cast<int>(op), st);
    });
}

extern "C" tc_status_t tc_broadcast(tc_dist_ctx* d, tc_buffer* buf, size_t num_elements, tc_dtype_t dtype, int root) {
    if (!d || !buf || num_elements == 0) return TC_ERR_INVALID_ARG;
    if (dist_elem(dtype) == 0) return TC_ERR_UNSUPPORTED_DTYPE;
    StepIo io[] = {{buf, num_elements * dist_elem(dtype), false}, {buf, num_elements * dist_elem(dtype), true}};
    return run_collective(d, "tc_broadcast", io, 2, [&](cudaStream_t st) {
        return tcb::dist_broadcast(d->comm, buf->dptr, num_elements, static_cast<int>(dtype), root, st);
    });
}

extern "C" tc_status_t tc_allgather(tc_dist_ctx* d, const tc_buffer* in, tc_buffer* out,
                                    size_t num_elements_per_rank, tc_dtype_t dtype) {
    if (!d || !in || !out || num_elements_per_rank == 0) return TC_ERR_INVALID_ARG;
    if (dist_elem(dtype) == 0) return TC_ERR_UNSUPPORTED_DTYPE;
    const size_t per = num_elements_per_rank * dist_elem(dtype);
    StepIo io[] = {{mut(in), per, false}, {out, per * static_cast<size_t>(tcb::dist_world(d->comm)), true}};
    return run_collective(d, "tc_allgather", io, 2, [&](cudaStream_t st) {
        return tcb::dist_allgather(d->comm, in->dptr, out->dptr, num_elements_per_rank, static_cast<int>(dtype), st);
    });
}

extern "C" tc_status_t tc_barrier(tc_dist_ctx* d) {
    if (!d) return TC_ERR_INVALID_ARG;
    bind_device(d->ctx);
    const int rc = tcb::dist_barrier(d->comm, d->ctx->stream0);
    if (rc != 0) return dist_status(rc);
    return from_cuda(cudaStreamSynchronize(d->ctx->stream0), TC_ERR_DISPATCH);
}

// ---------------------------------------------------------------------------------------
// Raw device-pointer launches
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tcx_raw_quantize_weights(tc_context* ctx, const void* W_fp16,
                                                void* W_quant, tc_quant_t fmt, int N, int K,
                                                void* cuda_stream) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!W_fp16 || !W_quant || tc_quantized_size(fmt, N, K) == 0) return TC_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(W_fp16) & 15u) != 0) return TC_ERR_INVALID_ARG;
    int launches = 0;
    const char* name = "none";
    const cudaError_t e = tcb::launch_quantize(W_fp16, W_quant, static_cast<int>(fmt), N, K,
                                               make_env(ctx, false),
                                               static_cast<cudaStream_t>(cuda_stream), &launches,
                                               &name);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    return record("tcx_raw_quantize_weights", from_cuda(e, TC_ERR_DISPATCH));
}

static tc_status_t raw_gemv(tc_context* ctx, const void* X, const void* gamma, bool fused,
                            const void* W, void* Y, tc_quant_t fmt, int M, int N, int K, float eps,
                            tc_dtype_t xd, tc_dtype_t yd, void* cuda_stream, const char* opname) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !W || !Y || (fused && !gamma) || M <= 0 || tc_quantized_size(fmt, N, K) == 0)
        return TC_ERR_INVALID_ARG;
    if ((xd != TC_DTYPE_F16 && xd != TC_DTYPE_F32) || (yd != TC_DTYPE_F16 && yd != TC_DTYPE_F32))
        return TC_ERR_UNSUPPORTED_DTYPE;
    tcb::GemvQArgs a;
    a.W = static_cast<const uint8_t*>(W);
    a.X = X; a.Y = Y; a.gamma = fused ? gamma : nullptr;
    a.fmt = static_cast<int>(fmt); a.M = M; a.N = N; a.K = K;
    a.x_f32 = xd == TC_DTYPE_F32; a.y_f32 = yd == TC_DTYPE_F32; a.eps = eps;
    norm_scratch_for(static_cast<cudaStream_t>(cuda_stream), norm_scratch_need(a), &a);
    dequant_scratch_for(static_cast<cudaStream_t>(cuda_stream), dequant_scratch_need(a), &a);
    int launches = 0;
    const char* name = "none";
    const cudaError_t e = tcb::launch_gemv_q(a, make_env(ctx, true),
                                             static_cast<cudaStream_t>(cuda_stream), &launches,
                                             &name);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    return record(opname, from_cuda(e, TC_ERR_DISPATCH));
}

extern "C" tc_status_t tcx_raw_gemv_quantized(tc_context* ctx, const void* X, const void* W_quant,
                                              void* Y, tc_quant_t fmt, int M, int N, int K,
                                              tc_dtype_t x_dtype, tc_dtype_t y_dtype,
                                              void* cuda_stream) {
    return raw_gemv(ctx, X, nullptr, false, W_quant, Y, fmt, M, N, K, 0.f, x_dtype, y_dtype,
                    cuda_stream, "tcx_raw_gemv_quantized");
}

extern "C" tc_status_t tcx_raw_fused_rmsnorm_gemv_quantized(
    tc_context* ctx, const void* X, const void* gamma, const void* W_quant, void* Y,
    tc_quant_t fmt, int M, int N, int K, float eps, tc_dtype_t x_dtype, tc_dtype_t y_dtype,
    void* cuda_stream) {
    return raw_gemv(ctx, X, gamma, true, W_quant, Y, fmt, M, N, K, eps, x_dtype, y_dtype,
                    cuda_stream, "tcx_raw_fused_rmsnorm_gemv_quantized");
}

extern "C" tc_status_t tcx_raw_fused_norm_gemv_f16(tc_context* ctx, const void* X,
                                                   const void* gamma, const void* beta,
                                                   const void* W, void* Y, int M, int N, int K,
                                                   float eps, void* cuda_stream) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!X || !gamma || !W || !Y || M <= 0 || N <= 0 || K <= 0) return TC_ERR_INVALID_ARG;
    tcb::DenseNormGemvArgs a;
    a.X = X; a.gamma = gamma; a.beta = beta; a.W = W; a.Y = Y;
    a.M = M; a.N = N; a.K = K; a.eps = eps;
    int launches = 0;
    const char* name = "none";
    dense_scratch_for(ctx, static_cast<cudaStream_t>(cuda_stream), &a);
    dense_norm_rows_for(static_cast<cudaStream_t>(cuda_stream), &a);
    const cudaError_t e = tcb::launch_dense_norm_gemv(a, make_env(ctx, true),
                                                      static_cast<cudaStream_t>(cuda_stream),
                                                      &launches, &name);
    g_launches.fetch_add(static_cast<uint64_t>(launches));
    t_last_kernel = name;
    return record("tcx_raw_fused_norm_gemv_f16", from_cuda(e, TC_ERR_DISPATCH));
}

// ---------------------------------------------------------------------------------------
// Decode launch without allocation (see include/tensorcore_b200.h)
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tcx_raw_decode_q4_static(tc_context* ctx, const tcx_decode_op* ops,
                                                int n_ops, void* cuda_stream) {
    if (!ctx) return TC_ERR_NOT_INITIALIZED;
    if (!ops || n_ops <= 0) return TC_ERR_INVALID_ARG;
    if (n_ops > TCX_DECODE_STATIC_MAX_OPS) {
        if (trace_enabled())
            std::fprintf(stderr, "[tensorcore] tcx_raw_decode_q4_static: %d operations exceed the "
                         "static scratch capacity of %d\n", n_ops, TCX_DECODE_STATIC_MAX_OPS);
        return TC_ERR_INVALID_SHAPE;
    }
    tcb::GemvQArgs args[TCX_DECODE_STATIC_MAX_OPS];
    for (int i = 0; i < n_ops; ++i) {
        const tcx_decode_op& o = ops[i];
        if (!o.W || !o.X || !o.Y || o.N <= 0 || o.K <= 0 || o.K % 32 != 0) return TC_ERR_INVALID_ARG;
        if ((o.x_dtype != TC_DTYPE_F16 && o.x_dtype != TC_DTYPE_F32) ||
            (o.y_dtype != TC_DTYPE_F16 && o.y_dtype != TC_DTYPE_F32))
            return TC_ERR_UNSUPPORTED_DTYPE;
        if (o.K % 256 != 0) return TC_ERR_INVALID_SHAPE;   // the persistent kernel's domain
        tcb::GemvQArgs& a = args[i];
        a.W = static_cast<const uint8_t*>(o.W);
        a.X = o.X; a.Y = o.Y; a.gamma = o.gamma;
        a.fmt = tcb::FMT_Q4_0; a.M = 1; a.N = o.N; a.K = o.K;
        a.x_f32 = o.x_dtype == TC_DTYPE_F32; a.y_f32 = o.y_dtype == TC_DTYPE_F32; a.eps = o.eps;
    }
    bind_device(ctx);
    const cudaError_t e = tcb::launch_gemv_q4_decode_static(args, n_ops, make_env(ctx, false),
                                                            static_cast<cudaStream_t>(cuda_stream));
    if (e == cudaErrorNotSupported) {   // the launcher's own domain checks; CUDA errors map below
        (void)cudaGetLastError();
        return TC_ERR_INVALID_SHAPE;
    }
    if (e == cudaSuccess) {
        g_launches.fetch_add(1);
        t_last_kernel = "q4_0_decode_persistent_static_sm100";
    }
    return record("tcx_raw_decode_q4_static", from_cuda(e, TC_ERR_DISPATCH));
}

// ---------------------------------------------------------------------------------------
// Diagnostics
// ---------------------------------------------------------------------------------------
extern "C" tc_status_t tcx_set_gemv_variant(const char* name) {
    if (!name) return TC_ERR_INVALID_ARG;
    int v = -1;
    if (!std::strcmp(name, "auto")) v = tcb::VARIANT_AUTO;
    else if (!std::strcmp(name, "simt")) v = tcb::VARIANT_SIMT;
    else if (!std::strcmp(name, "stream")) v = tcb::VARIANT_STREAM;
    else if (!std::strcmp(name, "tc")) v = tcb::VARIANT_TC;
    else if (!std::strcmp(name, "generic")) v = tcb::VARIANT_GENERIC;
    if (v < 0) return TC_ERR_INVALID_ARG;
    g_variant.store(v);
    return TC_OK;
}

extern "C" uint32_t tcx_take_device_error(tc_context* ctx) {
    if (!ctx || !ctx->err_host) return 0;
    const uint32_t v = *reinterpret_cast<volatile uint32_t*>(ctx->err_host);
    *reinterpret_cast<volatile uint32_t*>(ctx->err_host) = 0;
    return v;
}

extern "C" uint64_t tcx_launch_count(void) { return g_launches.load(); }

// Used by gguf.cpp: a device buffer filled from host memory through a pinned staging ring.
extern "C" tc_status_t tcb_buffer_from_host_bytes(tc_context* ctx, const void* src, size_t bytes,
                                                  tc_buffer** out) {
    if (!ctx || !src || !out || bytes == 0) return TC_ERR_INVALID_ARG;
    tc_buffer* b = nullptr;
    tc_status_t st = tc_buffer_alloc(ctx, bytes, &b);
    if (st != TC_OK) return st;
    // Two pinned slots: the CPU fills one while the copy engine drains the other.
    static std::mutex ring_mutex;
    static void* slots[2] = {nullptr, nullptr};
    static cudaEvent_t done[2] = {nullptr, nullptr};
    static const size_t kSlot = 32u << 20;
    std::lock_guard<std::mutex> lock(ring_mutex);
    for (int i = 0; i < 2; ++i) {
        if (!slots[i]) {
            if (cudaHostAlloc(&slots[i], kSlot, cudaHostAllocDefault) != cudaSuccess ||
                cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess) {
                (void)cudaGetLastError();
                tc_buffer_free(ctx, b);
                return TC_ERR_ALLOC;
            }
        }
    }
    cudaError_t e = cudaSuccess;
    size_t off = 0;
    int slot = 0;
    while (off < bytes && e == cudaSuccess) {
        const size_t n = (bytes - off) < kSlot ? (bytes - off) : kSlot;
        e = cudaEventSynchronize(done[slot]);  // slot free again (no-op before first use)
        if (e != cudaSuccess) break;
        std::memcpy(slots[slot], static_cast<const uint8_t*>(src) + off, n);
        e = cudaMemcpyAsync(static_cast<uint8_t*>(b->dptr) + off, slots[slot], n,
                            cudaMemcpyHostToDevice, ctx->stream0);
        if (e == cudaSuccess) e = cudaEventRecord(done[slot], ctx->stream0);
        off += n;
        slot ^= 1;
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream0);
    if (e != cudaSuccess) {
        tc_buffer_free(ctx, b);
        return from_cuda(e, TC_ERR_INTERNAL);
    }
    *out = b;
    return TC_OK;
}
