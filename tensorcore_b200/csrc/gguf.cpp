// GGUF v3 reader and device loader.
//
// Behaviour follows the reference reader (lib/io/gguf.c): read-only mmap of the file, header
// magic 'GGUF' and version 3 required, metadata key/value table (scalars, strings, arrays),
// tensor table (<= 4 dims, all non-zero), tensor data starting at the next multiple of
// general.alignment (default 32), every tensor range checked against the file size.  Storage
// types F32, F16, Q4_0, Q4_1, Q8_0 and BF16 are loadable; anything else is reported as
// TC_GGUF_TYPE_UNSUPPORTED with n_bytes 0 and skipped by the bulk loader.
//
// What differs from the reference is the destination: tensor bytes are copied from the file
// mapping through a pinned staging ring directly into device memory (tcb_buffer_from_host_bytes
// in runtime.cu); no host-visible copy of the weights is kept.
#include "../../include/tensorcore_b200.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <climits>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

extern "C" tc_status_t tcb_buffer_from_host_bytes(tc_context* ctx, const void* src, size_t bytes,
                                                  tc_buffer** out);

namespace {

enum ValueType : uint32_t {
    VT_U8 = 0, VT_I8 = 1, VT_U16 = 2, VT_I16 = 3, VT_U32 = 4, VT_I32 = 5, VT_F32 = 6,
    VT_BOOL = 7, VT_STRING = 8, VT_ARRAY = 9, VT_U64 = 10, VT_I64 = 11, VT_F64 = 12,
};

size_t scalar_size(uint32_t t) {
    switch (t) {
        case VT_U8: case VT_I8: case VT_BOOL: return 1;
        case VT_U16: case VT_I16: return 2;
        case VT_U32: case VT_I32: case VT_F32: return 4;
        case VT_U64: case VT_I64: case VT_F64: return 8;
        default: return 0;
    }
}

struct MetaValue {
    std::string key;
    uint32_t type = 0;
    uint8_t raw[8] = {0};          // scalar payload, little-endian as in the file
    std::string str;               // VT_STRING
    uint32_t elem_type = 0;        // VT_ARRAY
    uint64_t count = 0;
    const uint8_t* array_data = nullptr;  // into the mapping
};

struct Cursor {
    const uint8_t* base;
    size_t pos;
    size_t size;
    bool take(void* dst, size_t n) {
        if (pos > size || n > size - pos) return false;
        std::memcpy(dst, base + pos, n);
        pos += n;
        return true;
    }
    bool skip(size_t n) {
        if (pos > size || n > size - pos) return false;
        pos += n;
        return true;
    }
    bool string_view(const char** p, uint64_t* n) {
        uint64_t len = 0;
        if (!take(&len, 8)) return false;
        if (pos > size || len > size - pos) return false;
        *p = reinterpret_cast<const char*>(base + pos);
        *n = len;
        pos += static_cast<size_t>(len);
        return true;
    }
};

bool read_value(Cursor& c, uint32_t type, MetaValue& v) {
    v.type = type;
    const size_t ss = scalar_size(type);
    if (ss) return c.take(v.raw, ss);
    if (type == VT_STRING) {
        const char* p; uint64_t n;
        if (!c.string_view(&p, &n)) return false;
        v.str.assign(p, static_cast<size_t>(n));
        return true;
    }
    if (type == VT_ARRAY) {
        uint32_t et; uint64_t n;
        if (!c.take(&et, 4) || !c.take(&n, 8)) return false;
        v.elem_type = et;
        v.count = n;
        v.array_data = c.base + c.pos;
        if (et == VT_STRING) {
            for (uint64_t i = 0; i < n; ++i) {
                const char* p; uint64_t sn;
                if (!c.string_view(&p, &sn)) return false;
            }
            return true;
        }
        const size_t es = scalar_size(et);
        if (es == 0) return false;
        if (c.pos > c.size || n > (c.size - c.pos) / es) return false;
        return c.skip(static_cast<size_t>(n) * es);
    }
    return false;
}

tc_gguf_type_t storage_type(uint32_t ggml) {
    switch (ggml) {
        case 0: return TC_GGUF_TYPE_F32;
        case 1: return TC_GGUF_TYPE_F16;
        case 2: return TC_GGUF_TYPE_Q4_0;
        case 3: return TC_GGUF_TYPE_Q4_1;
        case 8: return TC_GGUF_TYPE_Q8_0;
        case 30: return TC_GGUF_TYPE_BF16;
        default: return TC_GGUF_TYPE_UNSUPPORTED;
    }
}

// Bytes of n elements in a storage type; false when the count does not fit the block size or
// overflows.  Unsupported types have size 0 (lib/io/gguf.c:311-339).
bool storage_bytes(tc_gguf_type_t t, uint64_t n, size_t* out) {
    uint64_t per = 0, blk = 1;
    switch (t) {
        case TC_GGUF_TYPE_F32: per = 4; break;
        case TC_GGUF_TYPE_F16: case TC_GGUF_TYPE_BF16: per = 2; break;
        case TC_GGUF_TYPE_Q4_0: per = 18; blk = 32; break;
        case TC_GGUF_TYPE_Q4_1: per = 20; blk = 32; break;
        case TC_GGUF_TYPE_Q8_0: per = 34; blk = 32; break;
        default: *out = 0; return true;
    }
    if (n % blk != 0) return false;
    const uint64_t units = n / blk;
    if (units > SIZE_MAX / per) return false;
    *out = static_cast<size_t>(units * per);
    return true;
}

int64_t scalar_i64(const uint8_t* p, uint32_t t, int64_t dflt, bool allow_bool) {
    switch (t) {
        case VT_U8: return *p;
        case VT_I8: return static_cast<int8_t>(*p);
        case VT_U16: { uint16_t v; std::memcpy(&v, p, 2); return v; }
        case VT_I16: { int16_t v; std::memcpy(&v, p, 2); return v; }
        case VT_U32: { uint32_t v; std::memcpy(&v, p, 4); return v; }
        case VT_I32: { int32_t v; std::memcpy(&v, p, 4); return v; }
        case VT_U64: { uint64_t v; std::memcpy(&v, p, 8); return static_cast<int64_t>(v); }
        case VT_I64: { int64_t v; std::memcpy(&v, p, 8); return v; }
        case VT_BOOL: return allow_bool ? *p : dflt;
        default: return dflt;
    }
}

double scalar_f64(const uint8_t* p, uint32_t t, double dflt, bool allow_bool) {
    switch (t) {
        case VT_F32: { float v; std::memcpy(&v, p, 4); return v; }
        case VT_F64: { double v; std::memcpy(&v, p, 8); return v; }
        case VT_U64: { uint64_t v; std::memcpy(&v, p, 8); return static_cast<double>(v); }
        case VT_BOOL: return allow_bool ? static_cast<double>(*p) : dflt;
        case VT_U8: case VT_I8: case VT_U16: case VT_I16: case VT_U32: case VT_I32: case VT_I64:
            return static_cast<double>(scalar_i64(p, t, 0, false));
        default: return dflt;
    }
}

}  // namespace

struct tc_gguf_file {
    int fd = -1;
    void* map = nullptr;
    size_t map_size = 0;
    uint32_t version = 0;
    uint32_t alignment = 32;
    uint64_t data_offset = 0;
    std::vector<MetaValue> meta;
    std::vector<std::string> names;            // tensor names (stable storage)
    std::vector<tc_gguf_tensor_info> tensors;

    const MetaValue* find(const char* key) const {
        if (!key) return nullptr;
        for (const MetaValue& m : meta)
            if (m.key == key) return &m;
        return nullptr;
    }
};

struct LoadedTensor {
    std::string name;
    tc_gguf_loaded_tensor_info info;
};

struct tc_gguf_loaded_model {
    std::vector<std::unique_ptr<LoadedTensor>> tensors;
    uint64_t skipped = 0;
};

extern "C" void tc_gguf_close(tc_gguf_file* f) {
    if (!f) return;
    if (f->map && f->map != MAP_FAILED) munmap(f->map, f->map_size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

extern "C" tc_status_t tc_gguf_open(const char* path, tc_gguf_file** out) {
    if (!path || !out) return TC_ERR_INVALID_ARG;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return TC_ERR_INTERNAL;
    struct stat st;
    if (fstat(fd, &st) < 0 || st.st_size <= 0) { close(fd); return TC_ERR_INTERNAL; }
    void* map = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) { close(fd); return TC_ERR_INTERNAL; }

    tc_gguf_file* f = new (std::nothrow) tc_gguf_file();
    if (!f) { munmap(map, static_cast<size_t>(st.st_size)); close(fd); return TC_ERR_ALLOC; }
    f->fd = fd;
    f->map = map;
    f->map_size = static_cast<size_t>(st.st_size);

    Cursor c{static_cast<const uint8_t*>(map), 0, f->map_size};
    uint32_t magic = 0;
    uint64_t n_tensors = 0, n_kv = 0;
    bool ok = c.take(&magic, 4) && magic == 0x46554747u && c.take(&f->version, 4) &&
              f->version == 3 && c.take(&n_tensors, 8) && c.take(&n_kv, 8);
    // Each KV needs at least 12 bytes and each tensor entry at least 24: reject counts that
    // cannot fit before reserving memory for them.
    if (ok && (n_kv > f->map_size / 12 || n_tensors > f->map_size / 24)) ok = false;
    if (ok) {
        f->meta.reserve(static_cast<size_t>(n_kv));
        for (uint64_t i = 0; ok && i < n_kv; ++i) {
            MetaValue v;
            const char* kp; uint64_t kn; uint32_t vt = 0;
            ok = c.string_view(&kp, &kn) && c.take(&vt, 4);
            if (!ok) break;
            v.key.assign(kp, static_cast<size_t>(kn));
            ok = read_value(c, vt, v);
            if (!ok) break;
            if (v.key == "general.alignment" && v.type == VT_U32) {
                uint32_t a; std::memcpy(&a, v.raw, 4);
                f->alignment = a;
            }
            f->meta.push_back(std::move(v));
        }
    }
    if (ok && f->alignment == 0) ok = false;
    if (ok) {
        f->names.reserve(static_cast<size_t>(n_tensors));
        f->tensors.reserve(static_cast<size_t>(n_tensors));
        for (uint64_t i = 0; ok && i < n_tensors; ++i) {
            const char* np; uint64_t nn; uint32_t nd = 0, gt = 0;
            tc_gguf_tensor_info ti;
            std::memset(&ti, 0, sizeof(ti));
            ok = c.string_view(&np, &nn) && c.take(&nd, 4) && nd <= 4;
            if (!ok) break;
            uint64_t elems = 1;
            for (uint32_t d = 0; ok && d < nd; ++d) {
                ok = c.take(&ti.dims[d], 8) && ti.dims[d] != 0 && elems <= UINT64_MAX / ti.dims[d];
                if (ok) elems *= ti.dims[d];
            }
            ok = ok && c.take(&gt, 4) && c.take(&ti.offset, 8);
            if (!ok) break;
            ti.n_dims = static_cast<int32_t>(nd);
            ti.type = storage_type(gt);
            ok = storage_bytes(ti.type, elems, &ti.n_bytes);
            if (!ok) break;
            f->names.emplace_back(np, static_cast<size_t>(nn));
            f->tensors.push_back(ti);
        }
    }
    if (ok) {
        const uint64_t a = f->alignment;
        const uint64_t pad = (a - (c.pos % a)) % a;
        f->data_offset = c.pos + pad;
        ok = f->data_offset <= f->map_size;
    }
    if (ok) {
        for (size_t i = 0; ok && i < f->tensors.size(); ++i) {
            tc_gguf_tensor_info& ti = f->tensors[i];
            ti.name = f->names[i].c_str();
            ok = ti.offset <= f->map_size - f->data_offset &&
                 ti.n_bytes <= f->map_size - f->data_offset - ti.offset;
            if (ok) ti.data = static_cast<const uint8_t*>(map) + f->data_offset + ti.offset;
        }
    }
    if (!ok) { tc_gguf_close(f); return TC_ERR_INTERNAL; }
    *out = f;
    return TC_OK;
}

extern "C" uint64_t tc_gguf_tensor_count(const tc_gguf_file* f) { return f ? f->tensors.size() : 0; }
extern "C" uint64_t tc_gguf_metadata_count(const tc_gguf_file* f) { return f ? f->meta.size() : 0; }

extern "C" tc_status_t tc_gguf_get_tensor(const tc_gguf_file* f, const char* name,
                                          tc_gguf_tensor_info* out) {
    if (!f || !name || !out) return TC_ERR_INVALID_ARG;
    for (const tc_gguf_tensor_info& t : f->tensors)
        if (std::strcmp(t.name, name) == 0) { *out = t; return TC_OK; }
    return TC_ERR_INVALID_ARG;
}

extern "C" tc_status_t tc_gguf_tensor_at(const tc_gguf_file* f, uint64_t i,
                                         tc_gguf_tensor_info* out) {
    if (!f || !out || i >= f->tensors.size()) return TC_ERR_INVALID_ARG;
    *out = f->tensors[static_cast<size_t>(i)];
    return TC_OK;
}

extern "C" const char* tc_gguf_meta_get_str(const tc_gguf_file* f, const char* key) {
    if (!f || !key) return nullptr;
    for (const MetaValue& m : f->meta)
        if (m.type == VT_STRING && m.key == key) return m.str.c_str();
    return nullptr;
}

extern "C" int64_t tc_gguf_meta_get_i64(const tc_gguf_file* f, const char* key, int64_t dflt) {
    const MetaValue* m = f ? f->find(key) : nullptr;
    if (!m || scalar_size(m->type) == 0) return dflt;
    if (m->type == VT_F32 || m->type == VT_F64 || m->type == VT_BOOL) return dflt;
    return scalar_i64(m->raw, m->type, dflt, false);
}

extern "C" double tc_gguf_meta_get_f64(const tc_gguf_file* f, const char* key, double dflt) {
    const MetaValue* m = f ? f->find(key) : nullptr;
    if (!m || scalar_size(m->type) == 0 || m->type == VT_BOOL) return dflt;
    return scalar_f64(m->raw, m->type, dflt, false);
}

extern "C" uint64_t tc_gguf_meta_array_count(const tc_gguf_file* f, const char* key) {
    const MetaValue* m = f ? f->find(key) : nullptr;
    return (m && m->type == VT_ARRAY) ? m->count : 0;
}

extern "C" tc_status_t tc_gguf_meta_array_get_str(const tc_gguf_file* f, const char* key,
                                                  uint64_t index, const char** out_ptr,
                                                  size_t* out_len) {
    if (!out_ptr || !out_len) return TC_ERR_INVALID_ARG;
    *out_ptr = nullptr;
    *out_len = 0;
    const MetaValue* m = f ? f->find(key) : nullptr;
    if (!m || m->type != VT_ARRAY || m->elem_type != VT_STRING || index >= m->count)
        return TC_ERR_INVALID_ARG;
    const uint8_t* base = static_cast<const uint8_t*>(f->map);
    Cursor c{m->array_data, 0, f->map_size - static_cast<size_t>(m->array_data - base)};
    const char* p = nullptr;
    uint64_t n = 0;
    for (uint64_t i = 0; i <= index; ++i)
        if (!c.string_view(&p, &n)) return TC_ERR_INTERNAL;
    *out_ptr = p;
    *out_len = static_cast<size_t>(n);
    return TC_OK;
}

extern "C" int64_t tc_gguf_meta_array_get_i64(const tc_gguf_file* f, const char* key,
                                              uint64_t index, int64_t dflt) {
    const MetaValue* m = f ? f->find(key) : nullptr;
    if (!m || m->type != VT_ARRAY || index >= m->count) return dflt;
    const size_t es = scalar_size(m->elem_type);
    if (es == 0) return dflt;
    return scalar_i64(m->array_data + index * es, m->elem_type, dflt, true);
}

extern "C" double tc_gguf_meta_array_get_f64(const tc_gguf_file* f, const char* key,
                                             uint64_t index, double dflt) {
    const MetaValue* m = f ? f->find(key) : nullptr;
    if (!m || m->type != VT_ARRAY || index >= m->count) return dflt;
    const size_t es = scalar_size(m->elem_type);
    if (es == 0) return dflt;
    return scalar_f64(m->array_data + index * es, m->elem_type, dflt, true);
}

extern "C" tc_status_t tc_gguf_get_llama_config(const tc_gguf_file* f, tc_gguf_llama_config* out) {
    if (!f || !out) return TC_ERR_INVALID_ARG;
    const char* arch = tc_gguf_meta_get_str(f, "general.architecture");
    if (!arch || std::strcmp(arch, "llama") != 0) return TC_ERR_INVALID_ARG;
    std::memset(out, 0, sizeof(*out));
    out->context_length = tc_gguf_meta_get_i64(f, "llama.context_length", 0);
    out->embedding_length = tc_gguf_meta_get_i64(f, "llama.embedding_length", 0);
    out->feed_forward_length = tc_gguf_meta_get_i64(f, "llama.feed_forward_length", 0);
    out->block_count = tc_gguf_meta_get_i64(f, "llama.block_count", 0);
    out->attention_head_count = tc_gguf_meta_get_i64(f, "llama.attention.head_count", 0);
    out->attention_head_count_kv =
        tc_gguf_meta_get_i64(f, "llama.attention.head_count_kv", out->attention_head_count);
    out->rope_dimension_count = tc_gguf_meta_get_i64(f, "llama.rope.dimension_count", 0);
    out->vocab_size = static_cast<int64_t>(tc_gguf_meta_array_count(f, "tokenizer.ggml.tokens"));
    out->rms_norm_epsilon = tc_gguf_meta_get_f64(f, "llama.attention.layer_norm_rms_epsilon", 1e-5);
    out->rope_freq_base = tc_gguf_meta_get_f64(f, "llama.rope.freq_base", 10000.0);
    out->rope_freq_scale = tc_gguf_meta_get_f64(f, "llama.rope.freq_scale", 1.0);
    return TC_OK;
}

static tc_status_t tensor_to_device(tc_context* ctx, const tc_gguf_tensor_info& ti,
                                    tc_buffer** out) {
    *out = nullptr;
    if (!ti.data || ti.n_bytes == 0 || ti.type == TC_GGUF_TYPE_UNSUPPORTED)
        return TC_ERR_UNSUPPORTED_DTYPE;
    return tcb_buffer_from_host_bytes(ctx, ti.data, ti.n_bytes, out);
}

extern "C" tc_status_t tc_gguf_tensor_to_buffer(tc_context* ctx, const tc_gguf_file* f,
                                                const char* name, tc_buffer** out_buffer) {
    if (!ctx || !f || !name || !out_buffer) return TC_ERR_INVALID_ARG;
    *out_buffer = nullptr;
    tc_gguf_tensor_info ti;
    const tc_status_t st = tc_gguf_get_tensor(f, name, &ti);
    if (st != TC_OK) return st;
    return tensor_to_device(ctx, ti, out_buffer);
}

// lib/io/gguf.c:766-817: a 2-D Q4_0/Q8_0 tensor with dims[0] = K (multiple of 32), dims[1] = N
// and exactly tc_quantized_size bytes is the [N,K] operand of tc_gemv_quantized.
static tc_status_t matrix_info(int32_t n_dims, const uint64_t* dims, tc_gguf_type_t type,
                               size_t n_bytes, tc_buffer* buffer,
                               tc_gguf_quantized_matrix_info* out) {
    std::memset(out, 0, sizeof(*out));
    tc_quant_t q;
    if (type == TC_GGUF_TYPE_Q4_0) q = TC_QUANT_Q4_0;
    else if (type == TC_GGUF_TYPE_Q8_0) q = TC_QUANT_Q8_0;
    else return TC_ERR_UNSUPPORTED_DTYPE;
    if (n_dims != 2 || dims[0] == 0 || dims[1] == 0 || dims[0] > static_cast<uint64_t>(INT_MAX) ||
        dims[1] > static_cast<uint64_t>(INT_MAX) || dims[0] % 32 != 0)
        return TC_ERR_INVALID_SHAPE;
    const int K = static_cast<int>(dims[0]), N = static_cast<int>(dims[1]);
    const size_t want = tc_quantized_size(q, N, K);
    if (want == 0 || want != n_bytes) return TC_ERR_INVALID_SHAPE;
    out->N = N;
    out->K = K;
    out->gguf_type = type;
    out->quant_type = q;
    out->n_bytes = n_bytes;
    out->buffer = buffer;
    return TC_OK;
}

extern "C" tc_status_t tc_gguf_tensor_quantized_matrix_info(const tc_gguf_tensor_info* t,
                                                            tc_gguf_quantized_matrix_info* out) {
    if (!t || !out) return TC_ERR_INVALID_ARG;
    return matrix_info(t->n_dims, t->dims, t->type, t->n_bytes, nullptr, out);
}

extern "C" tc_status_t tc_gguf_loaded_tensor_quantized_matrix_info(
    const tc_gguf_loaded_tensor_info* t, tc_gguf_quantized_matrix_info* out) {
    if (!t || !out) return TC_ERR_INVALID_ARG;
    return matrix_info(t->n_dims, t->dims, t->type, t->n_bytes, t->buffer, out);
}

extern "C" void tc_gguf_loaded_model_free(tc_context* ctx, tc_gguf_loaded_model* model) {
    if (!model) return;
    for (auto& t : model->tensors)
        if (ctx && t->info.buffer) tc_buffer_free(ctx, t->info.buffer);
    delete model;
}

extern "C" tc_status_t tc_gguf_load_supported_tensors(tc_context* ctx, const tc_gguf_file* f,
                                                      tc_gguf_loaded_model** out_model) {
    if (!ctx || !f || !out_model) return TC_ERR_INVALID_ARG;
    *out_model = nullptr;
    tc_gguf_loaded_model* model = new (std::nothrow) tc_gguf_loaded_model();
    if (!model) return TC_ERR_ALLOC;
    for (const tc_gguf_tensor_info& src : f->tensors) {
        if (!src.data || src.n_bytes == 0 || src.type == TC_GGUF_TYPE_UNSUPPORTED) {
            model->skipped++;
            continue;
        }
        std::unique_ptr<LoadedTensor> lt(new (std::nothrow) LoadedTensor());
        if (!lt) { tc_gguf_loaded_model_free(ctx, model); return TC_ERR_ALLOC; }
        lt->name = src.name ? src.name : "";
        std::memset(&lt->info, 0, sizeof(lt->info));
        lt->info.n_dims = src.n_dims;
        for (int d = 0; d < src.n_dims && d < 4; ++d) lt->info.dims[d] = src.dims[d];
        lt->info.type = src.type;
        lt->info.offset = src.offset;
        lt->info.n_bytes = src.n_bytes;
        const tc_status_t st = tensor_to_device(ctx, src, &lt->info.buffer);
        if (st != TC_OK) { tc_gguf_loaded_model_free(ctx, model); return st; }
        lt->info.name = lt->name.c_str();
        model->tensors.push_back(std::move(lt));
    }
    *out_model = model;
    return TC_OK;
}

extern "C" uint64_t tc_gguf_loaded_tensor_count(const tc_gguf_loaded_model* m) {
    return m ? m->tensors.size() : 0;
}
extern "C" uint64_t tc_gguf_loaded_skipped_tensor_count(const tc_gguf_loaded_model* m) {
    return m ? m->skipped : 0;
}

extern "C" tc_status_t tc_gguf_loaded_tensor_at(const tc_gguf_loaded_model* m, uint64_t i,
                                                tc_gguf_loaded_tensor_info* out) {
    if (!m || !out || i >= m->tensors.size()) return TC_ERR_INVALID_ARG;
    *out = m->tensors[static_cast<size_t>(i)]->info;
    return TC_OK;
}

extern "C" tc_status_t tc_gguf_loaded_get_tensor(const tc_gguf_loaded_model* m, const char* name,
                                                 tc_gguf_loaded_tensor_info* out) {
    if (!m || !name || !out) return TC_ERR_INVALID_ARG;
    for (const auto& t : m->tensors)
        if (t->name == name) { *out = t->info; return TC_OK; }
    return TC_ERR_INVALID_ARG;
}
