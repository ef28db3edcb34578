// Decode harness: drives the GEMV sequence of a Llama-shaped decode step through the public
// C ABI of libtensorcore.so (tc_gemv_quantized_async / tcx_*_ex + tc_stream_sync), the way the
// reference's bench/bench_inference_7b.c drives the reference library: every projection of
// every layer is recorded on one stream and the stream is synchronised once per token.
//
// It exists so that the timed loop runs in compiled code (225 recorded calls per 7B token cost
// well under a microsecond each here; the same loop in Python would cost more than the GPU
// work).  It links only against the public ABI and the CUDA runtime (for events); it contains
// no kernels and no arithmetic.
#include "../../../include/tensorcore_b200.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

extern "C" {

typedef struct {
    int n_layers, d_model, d_ff, d_kv, vocab;
    int M;       // sequences decoded together
    int fmt;     // tc_quant_t of all projection matrices
    tc_buffer** wq;      // [n_layers] each [d_model x d_model]
    tc_buffer** wk;      // [n_layers] each [d_kv x d_model]
    tc_buffer** wv;      // [n_layers]
    tc_buffer** wo;      // [n_layers] [d_model x d_model]
    tc_buffer** wgate;   // [n_layers] [d_ff x d_model]
    tc_buffer** wup;     // [n_layers]
    tc_buffer** wdown;   // [n_layers] [d_model x d_ff]
    tc_buffer** attn_norm;  // [n_layers] fp16 [d_model] (may be NULL when mode 0 is used only)
    tc_buffer** ffn_norm;   // [n_layers]
    tc_buffer* out_norm;    // fp16 [d_model]
    tc_buffer* lm_head;     // [vocab x d_model], may be NULL (the reference bench has none)
} tch_model_desc;

typedef struct tch_session {
    tc_context* ctx;
    tch_model_desc d;
    std::vector<tc_buffer*> wq, wk, wv, wo, wgate, wup, wdown, attn_norm, ffn_norm;
    tc_stream* stream;
    tc_buffer *x[3], *q, *k, *v, *o, *gate, *up, *logits;   // x[0]: step input, x[1..2]: hidden
    cudaEvent_t ev0, ev1;
} tch_session;

static void copy_list(std::vector<tc_buffer*>& dst, tc_buffer** src, int n) {
    dst.clear();
    if (src) dst.assign(src, src + n);
}

void tch_session_destroy(tch_session* s) {
    if (!s) return;
    tc_buffer* bufs[] = {s->x[0], s->x[1], s->x[2], s->q, s->k, s->v, s->o, s->gate, s->up, s->logits};
    for (tc_buffer* b : bufs)
        if (b) tc_buffer_free(s->ctx, b);
    if (s->stream) tc_stream_destroy(s->ctx, s->stream);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    delete s;
}

// Activations are fp16 [M, width].  Returns a tc_status_t.
int tch_session_create(tc_context* ctx, const tch_model_desc* d, tch_session** out) {
    if (!ctx || !d || !out || d->n_layers <= 0 || d->M <= 0) return TC_ERR_INVALID_ARG;
    tch_session* s = new (std::nothrow) tch_session();
    if (!s) return TC_ERR_ALLOC;
    s->ctx = ctx;
    s->d = *d;
    const int L = d->n_layers;
    copy_list(s->wq, d->wq, L); copy_list(s->wk, d->wk, L); copy_list(s->wv, d->wv, L);
    copy_list(s->wo, d->wo, L); copy_list(s->wgate, d->wgate, L); copy_list(s->wup, d->wup, L);
    copy_list(s->wdown, d->wdown, L); copy_list(s->attn_norm, d->attn_norm, L);
    copy_list(s->ffn_norm, d->ffn_norm, L);
    s->stream = nullptr;
    s->ev0 = s->ev1 = nullptr;
    tc_buffer** slots[] = {&s->x[0], &s->x[1], &s->x[2], &s->q, &s->k, &s->v, &s->o, &s->gate,
                           &s->up, &s->logits};
    const size_t widths[] = {(size_t)d->d_model, (size_t)d->d_model, (size_t)d->d_model,
                             (size_t)d->d_model,
                             (size_t)d->d_kv, (size_t)d->d_kv, (size_t)d->d_model,
                             (size_t)d->d_ff, (size_t)d->d_ff,
                             (size_t)(d->vocab > 0 ? d->vocab : 1)};
    for (tc_buffer** p : slots) *p = nullptr;
    int st = TC_OK;
    for (int i = 0; i < 10 && st == TC_OK; ++i)
        st = tc_buffer_alloc(ctx, widths[i] * (size_t)d->M * 2, slots[i]);
    if (st == TC_OK) st = tc_stream_create(ctx, &s->stream);
    if (st == TC_OK && (cudaEventCreate(&s->ev0) != cudaSuccess ||
                        cudaEventCreate(&s->ev1) != cudaSuccess))
        st = TC_ERR_INTERNAL;
    if (st != TC_OK) { tch_session_destroy(s); return st; }
    *out = s;
    return TC_OK;
}

tc_buffer* tch_session_x(tch_session* s) { return s ? s->x[0] : nullptr; }
tc_buffer* tch_session_logits(tch_session* s) { return s ? s->logits : nullptr; }
tc_buffer* tch_session_hidden(tch_session* s, int which) { return s ? s->x[1 + (which & 1)] : nullptr; }

// One projection.  mode 0: tc_gemv_quantized_async (the reference entry point).
// mode 1 with gamma: RMSNorm prologue fused into the GEMV (tcx_fused_rmsnorm_gemv_quantized_ex).
static int proj(tch_session* s, int mode, tc_buffer* x, tc_buffer* gamma, tc_buffer* w,
                tc_buffer* y, int N, int K) {
    const tc_quant_t fmt = (tc_quant_t)s->d.fmt;
    if (mode == 1 && gamma)
        return tcx_fused_rmsnorm_gemv_quantized_ex(s->ctx, x, gamma, w, y, fmt, s->d.M, N, K, 1e-5f,
                                                   TC_DTYPE_F16, TC_DTYPE_F16, s->stream);
    return tc_gemv_quantized_async(s->ctx, x, w, y, fmt, s->d.M, N, K, s->stream);
}

// Records one token's projections.  The step input x[0] is only read; the hidden state then
// ping-pongs between x[1] and x[2]; the
// attention mix and the SwiGLU gate, which lie outside this path, are stood in for by feeding
// the q projection to o_proj and the gate projection to down_proj, so that every GEMV reads
// the output of an earlier one (a true dependency chain) with the real shapes.
static int record_token(tch_session* s, int mode) {
    const tch_model_desc& d = s->d;
    int st = TC_OK;
    int cur = 0;   // index into x[]: layer l reads x[cur], writes x[nxt]
    for (int l = 0; l < d.n_layers && st == TC_OK; ++l) {
        const int nxt = (cur == 1) ? 2 : 1;
        tc_buffer* an = s->attn_norm.empty() ? nullptr : s->attn_norm[l];
        tc_buffer* fn = s->ffn_norm.empty() ? nullptr : s->ffn_norm[l];
        st = proj(s, mode, s->x[cur], an, s->wq[l], s->q, d.d_model, d.d_model);
        if (st == TC_OK) st = proj(s, mode, s->x[cur], an, s->wk[l], s->k, d.d_kv, d.d_model);
        if (st == TC_OK) st = proj(s, mode, s->x[cur], an, s->wv[l], s->v, d.d_kv, d.d_model);
        if (st == TC_OK) st = proj(s, 0, s->q, nullptr, s->wo[l], s->o, d.d_model, d.d_model);
        if (st == TC_OK) st = proj(s, mode, s->o, fn, s->wgate[l], s->gate, d.d_ff, d.d_model);
        if (st == TC_OK) st = proj(s, mode, s->o, fn, s->wup[l], s->up, d.d_ff, d.d_model);
        if (st == TC_OK) st = proj(s, 0, s->gate, nullptr, s->wdown[l], s->x[nxt], d.d_model, d.d_ff);
        cur = nxt;
    }
    if (st == TC_OK && d.lm_head)
        st = proj(s, mode, s->x[cur], d.out_norm, d.lm_head, s->logits, d.vocab, d.d_model);
    return st;
}

// Runs `tokens` decode steps.  e2e != 0: every step first copies the step's input hidden state
// from host_x (caller memory, pinned for the benchmark) into the device and afterwards copies
// the logits back to host_logits.  Timing: *gpu_ms = CUDA-event time on the stream over all
// steps, *wall_ms = host clock over the same loop (both include the copies in e2e mode).
int tch_session_run(tch_session* s, int tokens, int mode, int e2e, const void* host_x,
                    void* host_logits, float* gpu_ms, double* wall_ms) {
    if (!s || tokens <= 0) return TC_ERR_INVALID_ARG;
    if (e2e && (!host_x || !host_logits || !s->d.lm_head)) return TC_ERR_INVALID_ARG;
    void* cs = nullptr;
    int st = tcx_stream_cuda_handle(s->stream, &cs);
    if (st != TC_OK) return st;
    cudaStream_t stream = (cudaStream_t)cs;
    const size_t xb = (size_t)s->d.d_model * s->d.M * 2;
    const size_t lb = (size_t)(s->d.vocab > 0 ? s->d.vocab : 1) * s->d.M * 2;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return TC_ERR_INTERNAL;
    const auto t0 = std::chrono::steady_clock::now();
    cudaEventRecord(s->ev0, stream);
    for (int t = 0; t < tokens && st == TC_OK; ++t) {
        if (e2e) st = tcx_buffer_upload(s->x[0], 0, host_x, xb);
        if (st == TC_OK) st = record_token(s, mode);
        if (st == TC_OK) st = tc_stream_sync(s->stream);
        if (st == TC_OK && e2e) st = tcx_buffer_download(s->logits, 0, host_logits, lb);
    }
    cudaEventRecord(s->ev1, stream);
    if (cudaStreamSynchronize(stream) != cudaSuccess && st == TC_OK) st = TC_ERR_INTERNAL;
    const auto t1 = std::chrono::steady_clock::now();
    if (gpu_ms) { *gpu_ms = 0.f; cudaEventElapsedTime(gpu_ms, s->ev0, s->ev1); }
    if (wall_ms) *wall_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    return st;
}

// Single-matrix benchmark: `iters` GEMVs recorded on one stream, rotating over `copies`
// distinct weight buffers (so that with copies * bytes > L2 every launch streams from HBM),
// one synchronisation at the end.  fused != 0 uses the RMSNorm-fused entry point.
// persistent == 0: one kernel per operation (graph replay) even where the list would qualify for
// the persistent decode kernel.
int tch_gemv_bench(tc_context* ctx, tc_buffer** weights, int copies, tc_buffer* x,
                   tc_buffer* gamma, tc_buffer* y, int fmt, int M, int N, int K, int x_dtype,
                   int y_dtype, int fused, int iters, int persistent, float* gpu_ms) {
    if (!ctx || !weights || copies <= 0 || iters <= 0) return TC_ERR_INVALID_ARG;
    tc_stream* s = nullptr;
    int st = tc_stream_create(ctx, &s);
    if (st != TC_OK) return st;
    tcx_stream_set_persistent(s, persistent);
    void* cs = nullptr;
    tcx_stream_cuda_handle(s, &cs);
    cudaStream_t stream = (cudaStream_t)cs;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int rep = 0; rep < 3 && st == TC_OK; ++rep) {  // rep 0,1: warm-up (and graph build)
        if (rep == 2) cudaEventRecord(e0, stream);
        for (int i = 0; i < iters && st == TC_OK; ++i) {
            tc_buffer* w = weights[i % copies];
            if (fused)
                st = tcx_fused_rmsnorm_gemv_quantized_ex(ctx, x, gamma, w, y, (tc_quant_t)fmt, M, N,
                                                         K, 1e-5f, (tc_dtype_t)x_dtype,
                                                         (tc_dtype_t)y_dtype, s);
            else
                st = tcx_gemv_quantized_ex(ctx, x, w, y, (tc_quant_t)fmt, M, N, K,
                                           (tc_dtype_t)x_dtype, (tc_dtype_t)y_dtype, s);
        }
        if (st == TC_OK) st = tcx_stream_flush(s);
        if (rep == 2) cudaEventRecord(e1, stream);
        if (st == TC_OK) st = tc_stream_sync(s);
    }
    if (gpu_ms) { *gpu_ms = 0.f; if (st == TC_OK) cudaEventElapsedTime(gpu_ms, e0, e1); }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    tc_stream_destroy(ctx, s);
    return st;
}

// The dense fused norm + GEMV operations (fp16 W[K,N]): `iters` raw launches back to back on one
// CUDA stream, rotating over `copies` weight matrices.  beta == NULL: RMSNorm, else LayerNorm.
int tch_dense_bench(tc_context* ctx, tc_buffer** weights, int copies, tc_buffer* x, tc_buffer* gamma,
                    tc_buffer* beta, tc_buffer* y, int M, int N, int K, int iters, float* gpu_ms) {
    if (!ctx || !weights || copies <= 0 || iters <= 0 || !x || !gamma || !y) return TC_ERR_INVALID_ARG;
    cudaStream_t stream;
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return TC_ERR_INTERNAL;
    void *px, *pg, *pb = nullptr, *py;
    tcx_buffer_device_ptr(x, &px); tcx_buffer_device_ptr(gamma, &pg); tcx_buffer_device_ptr(y, &py);
    if (beta) tcx_buffer_device_ptr(beta, &pb);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int st = TC_OK;
    for (int rep = 0; rep < 2 && st == TC_OK; ++rep) {
        if (rep == 1) cudaEventRecord(e0, stream);
        for (int i = 0; i < iters && st == TC_OK; ++i) {
            void* pw;
            tcx_buffer_device_ptr(weights[i % copies], &pw);
            st = tcx_raw_fused_norm_gemv_f16(ctx, px, pg, pb, pw, py, M, N, K, 1e-5f, stream);
        }
        if (rep == 1) cudaEventRecord(e1, stream);
        if (cudaStreamSynchronize(stream) != cudaSuccess && st == TC_OK) st = TC_ERR_INTERNAL;
    }
    if (gpu_ms) { *gpu_ms = 0.f; if (st == TC_OK) cudaEventElapsedTime(gpu_ms, e0, e1); }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(stream);
    return st;
}

// Decode attention: `iters` launches of one query row per head over `copies` distinct K/V caches
// (so that they stream from HBM), event-timed on one stream.
int tch_attention_bench(tc_context* ctx, tc_buffer* q, tc_buffer** ks, tc_buffer** vs, int copies, tc_buffer* o,
                        int batch, int heads, int kv_heads, int seq_kv, int head_dim, int iters, float* gpu_ms) {
    if (!ctx || !q || !ks || !vs || !o || copies <= 0 || iters <= 0) return TC_ERR_INVALID_ARG;
    cudaStream_t stream;
    if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return TC_ERR_INTERNAL;
    tc_attention_desc d;
    std::memset(&d, 0, sizeof(d));
    d.batch = batch; d.heads = heads; d.seq_q = 1; d.seq_kv = seq_kv; d.head_dim = head_dim;
    d.io_dtype = TC_DTYPE_F16; d.accum_dtype = TC_DTYPE_F32; d.kv_heads = kv_heads;
    void *pq, *po;
    tcx_buffer_device_ptr(q, &pq); tcx_buffer_device_ptr(o, &po);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int st = TC_OK;
    for (int rep = 0; rep < 2 && st == TC_OK; ++rep) {
        if (rep == 1) cudaEventRecord(e0, stream);
        for (int i = 0; i < iters && st == TC_OK; ++i) {
            void *pk, *pv;
            tcx_buffer_device_ptr(ks[i % copies], &pk);
            tcx_buffer_device_ptr(vs[i % copies], &pv);
            st = tcx_raw_attention_forward(ctx, &d, pq, pk, pv, po, nullptr, stream);
        }
        if (rep == 1) cudaEventRecord(e1, stream);
        if (cudaStreamSynchronize(stream) != cudaSuccess && st == TC_OK) st = TC_ERR_INTERNAL;
    }
    if (gpu_ms) { *gpu_ms = 0.f; if (st == TC_OK) cudaEventElapsedTime(gpu_ms, e0, e1); }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaStreamDestroy(stream);
    return st;
}

}  // extern "C"
