// GGUF reader (host code only; see include/ullm_gguf.h for the rules it follows and the
// reference lines they come from).
#include "../../include/ullm_gguf.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <memory>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

constexpr uint32_t GGUF_MAGIC = 0x46554747u; // "GGUF" little-endian
constexpr uint64_t DEFAULT_ALIGNMENT = 32;

enum : uint32_t { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

struct Failure {
    int code;
    std::string msg;
};
[[noreturn]] void fail(int code, const char *fmt, ...) {
    char buf[256];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw Failure{code, buf};
}

// bounds-checked little-endian cursor (crates/ullm-gguf/src/reader.rs)
struct Cursor {
    const uint8_t *buf;
    size_t len, pos = 0;
    const uint8_t *take(size_t n) {
        if (n > len - pos) fail(ULLM_GGUF_ERR_FORMAT, "unexpected end of file");
        const uint8_t *p = buf + pos;
        pos += n;
        return p;
    }
    template <typename T> T get() {
        T v;
        memcpy(&v, take(sizeof(T)), sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (n > len - pos) fail(ULLM_GGUF_ERR_FORMAT, "unexpected end of file");
        const uint8_t *p = take((size_t)n);
        return std::string((const char *)p, (size_t)n);
    }
};

struct Value {
    uint32_t type = T_U8, elem_type = T_U8;
    uint64_t u = 0;  // integers (sign-extended like the reference's `as u64`) and bool
    double f = 0;    // floats
    std::string s;
    std::vector<Value> items;
    bool is_int() const { return type <= T_I32 || type == T_BOOL || type == T_U64 || type == T_I64; }
    bool is_float() const { return type == T_F32 || type == T_F64; }
};

Value read_value(Cursor &r, uint32_t type) {
    Value v;
    v.type = type;
    switch (type) {
    case T_U8: v.u = r.get<uint8_t>(); break;
    case T_I8: v.u = (uint64_t)(int64_t)r.get<int8_t>(); break;
    case T_U16: v.u = r.get<uint16_t>(); break;
    case T_I16: v.u = (uint64_t)(int64_t)r.get<int16_t>(); break;
    case T_U32: v.u = r.get<uint32_t>(); break;
    case T_I32: v.u = (uint64_t)(int64_t)r.get<int32_t>(); break;
    case T_F32: v.f = r.get<float>(); break;
    case T_BOOL: v.u = r.get<uint8_t>() != 0; break;
    case T_STRING: v.s = r.str(); break;
    case T_U64: v.u = r.get<uint64_t>(); break;
    case T_I64: v.u = (uint64_t)r.get<int64_t>(); break;
    case T_F64: v.f = r.get<double>(); break;
    case T_ARRAY: {
        v.elem_type = r.get<uint32_t>();
        if (v.elem_type == T_ARRAY) fail(ULLM_GGUF_ERR_FORMAT, "nested GGUF arrays are not supported");
        const uint64_t n = r.get<uint64_t>();
        v.items.reserve((size_t)(n < (1u << 16) ? n : (1u << 16))); // a corrupt count must not reserve the world
        for (uint64_t i = 0; i < n; ++i) v.items.push_back(read_value(r, v.elem_type));
        break;
    }
    default: fail(ULLM_GGUF_ERR_FORMAT, "unknown GGUF value type id %u", type);
    }
    return v;
}

// ggml type id -> (weights per block, bytes per block); 0 = not a type the reference maps
bool block_geometry(uint32_t id, uint64_t &block, uint64_t &bytes) {
    switch (id) {
    case 0: block = 1, bytes = 4; return true;      // F32
    case 1: block = 1, bytes = 2; return true;      // F16
    case 2: block = 32, bytes = 18; return true;    // Q4_0
    case 3: block = 32, bytes = 20; return true;    // Q4_1
    case 6: block = 32, bytes = 22; return true;    // Q5_0
    case 7: block = 32, bytes = 24; return true;    // Q5_1
    case 8: block = 32, bytes = 34; return true;    // Q8_0
    case 10: block = 256, bytes = 84; return true;  // Q2_K
    case 11: block = 256, bytes = 110; return true; // Q3_K
    case 12: block = 256, bytes = 144; return true; // Q4_K
    case 13: block = 256, bytes = 176; return true; // Q5_K
    case 14: block = 256, bytes = 210; return true; // Q6_K
    case 15: block = 256, bytes = 292; return true; // Q8_K
    case 30: block = 1, bytes = 2; return true;     // BF16
    default: return false;
    }
}

struct Tensor {
    std::string name;
    uint32_t dtype = 0;
    std::vector<uint64_t> shape; // outermost first
    uint64_t offset = 0, nbytes = 0;
};

} // namespace

struct ullm_gguf {
    const uint8_t *base = nullptr;
    size_t len = 0;
    bool mapped = false;
    std::vector<uint8_t> owned;
    uint32_t version = 0;
    uint64_t alignment = DEFAULT_ALIGNMENT, data_start = 0;
    std::map<std::string, Value> meta; // ordered like the reference's BTreeMap
    std::vector<const std::string *> meta_keys;
    std::vector<Tensor> tensors;
    std::map<std::string, size_t> by_name;
    std::string arch;

    ~ullm_gguf() {
        if (mapped && base) munmap((void *)base, len);
    }
    const Value *find(const char *key) const {
        auto it = meta.find(key);
        return it == meta.end() ? nullptr : &it->second;
    }
    void parse() {
        Cursor r{base, len};
        const uint32_t magic = r.get<uint32_t>();
        if (magic != GGUF_MAGIC) fail(ULLM_GGUF_ERR_FORMAT, "not a GGUF file (bad magic 0x%08x)", magic);
        version = r.get<uint32_t>();
        if (version != 2 && version != 3) fail(ULLM_GGUF_ERR_UNSUPPORTED, "GGUF version %u (only 2 and 3 are supported)", version);
        const uint64_t n_tensors = r.get<uint64_t>(), n_meta = r.get<uint64_t>();
        for (uint64_t i = 0; i < n_meta; ++i) {
            std::string key = r.str();
            const uint32_t type = r.get<uint32_t>();
            meta[key] = read_value(r, type); // a repeated key keeps the last value, as a map insert does
        }
        struct Raw {
            Tensor t;
            uint64_t rel;
        };
        std::vector<Raw> raws;
        for (uint64_t i = 0; i < n_tensors; ++i) {
            Raw rw;
            rw.t.name = r.str();
            const uint32_t nd = r.get<uint32_t>();
            if (nd > 8) fail(ULLM_GGUF_ERR_FORMAT, "tensor '%s' has %u dimensions", rw.t.name.c_str(), nd);
            for (uint32_t d = 0; d < nd; ++d) rw.t.shape.push_back(r.get<uint64_t>());
            rw.t.dtype = r.get<uint32_t>();
            uint64_t blk, bytes;
            if (!block_geometry(rw.t.dtype, blk, bytes)) fail(ULLM_GGUF_ERR_UNSUPPORTED, "ggml tensor type id %u is not yet supported", rw.t.dtype);
            rw.rel = r.get<uint64_t>();
            raws.push_back(std::move(rw));
        }
        if (const Value *a = find("general.alignment"))
            if (a->is_int()) alignment = a->u;
        if (alignment < 1) alignment = 1;
        const uint64_t info_end = r.pos;
        // an alignment beyond the file (a negative i32 read as u64, say) would wrap the round-up below
        if (alignment > len) fail(ULLM_GGUF_ERR_FORMAT, "general.alignment %llu exceeds the file size", (unsigned long long)alignment);
        data_start = (info_end + alignment - 1) / alignment * alignment;
        for (Raw &rw : raws) {
            Tensor &t = rw.t;
            // fastest-varying dimension first on disk -> outermost first here
            std::vector<uint64_t> rev(t.shape.rbegin(), t.shape.rend());
            t.shape.swap(rev);
            uint64_t n = 1, blk, bytes;
            for (uint64_t d : t.shape) {
                if (d != 0 && n > UINT64_MAX / d) fail(ULLM_GGUF_ERR_FORMAT, "tensor '%s': element count overflow", t.name.c_str());
                n *= d;
            }
            block_geometry(t.dtype, blk, bytes);
            if (n % blk) fail(ULLM_GGUF_ERR_FORMAT, "element count %llu is not a multiple of block size %llu", (unsigned long long)n, (unsigned long long)blk);
            t.nbytes = n / blk * bytes;
            t.offset = data_start + rw.rel;
            if (t.offset < data_start || t.offset + t.nbytes < t.offset) fail(ULLM_GGUF_ERR_FORMAT, "tensor offset overflow");
            if (t.offset + t.nbytes > len) fail(ULLM_GGUF_ERR_FORMAT, "tensor '%s' extends past end of file", t.name.c_str());
            by_name[t.name] = tensors.size(); // a repeated name keeps the last record
            tensors.push_back(std::move(t));
        }
        for (auto &kv : meta) meta_keys.push_back(&kv.first);
        if (const Value *a = find("general.architecture"))
            if (a->type == T_STRING) arch = a->s;
    }
};

namespace {

void put_err(char *err, size_t cap, const char *msg) {
    if (err && cap) snprintf(err, cap, "%s", msg);
}

int finish(std::unique_ptr<ullm_gguf> g, ullm_gguf **out, char *err, size_t cap) {
    try {
        g->parse();
    } catch (const Failure &f) {
        put_err(err, cap, f.msg.c_str());
        return f.code;
    } catch (const std::bad_alloc &) {
        put_err(err, cap, "out of memory while reading the GGUF directory");
        return ULLM_GGUF_ERR_FORMAT;
    }
    *out = g.release();
    return ULLM_GGUF_OK;
}

void fill(const ullm_gguf *g, const Tensor &t, ullm_gguf_tensor *o) {
    memset(o, 0, sizeof *o);
    o->name = t.name.c_str(), o->dtype = (int)t.dtype, o->n_dims = (uint32_t)t.shape.size();
    for (size_t i = 0; i < t.shape.size(); ++i) o->shape[i] = t.shape[i];
    o->offset = t.offset, o->nbytes = t.nbytes, o->data = g->base + t.offset;
}

} // namespace

extern "C" {

int ullm_gguf_open(const char *path, ullm_gguf **out, char *err, size_t err_cap) {
    if (!path || !out) return ULLM_GGUF_ERR_INVALID;
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        put_err(err, err_cap, "cannot open the file");
        return ULLM_GGUF_ERR_IO;
    }
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        put_err(err, err_cap, "cannot stat the file");
        return ULLM_GGUF_ERR_IO;
    }
    if (st.st_size <= 0) {
        close(fd);
        put_err(err, err_cap, st.st_size == 0 ? "unexpected end of file" : "cannot stat the file");
        return st.st_size == 0 ? ULLM_GGUF_ERR_FORMAT : ULLM_GGUF_ERR_IO;
    }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) {
        put_err(err, err_cap, "cannot map the file");
        return ULLM_GGUF_ERR_IO;
    }
    std::unique_ptr<ullm_gguf> g(new (std::nothrow) ullm_gguf);
    if (!g) {
        munmap(m, (size_t)st.st_size);
        return ULLM_GGUF_ERR_IO;
    }
    g->base = (const uint8_t *)m, g->len = (size_t)st.st_size, g->mapped = true;
    return finish(std::move(g), out, err, err_cap);
}

int ullm_gguf_from_bytes(const void *bytes, size_t len, ullm_gguf **out, char *err, size_t err_cap) {
    if (!out || (len && !bytes)) return ULLM_GGUF_ERR_INVALID;
    *out = nullptr;
    std::unique_ptr<ullm_gguf> g(new (std::nothrow) ullm_gguf);
    if (!g) return ULLM_GGUF_ERR_IO;
    g->owned.assign((const uint8_t *)bytes, (const uint8_t *)bytes + len);
    g->base = g->owned.data(), g->len = len;
    return finish(std::move(g), out, err, err_cap);
}

void ullm_gguf_close(ullm_gguf *g) { delete g; }

uint32_t ullm_gguf_version(const ullm_gguf *g) { return g ? g->version : 0; }
const char *ullm_gguf_architecture(const ullm_gguf *g) { return g ? g->arch.c_str() : ""; }
uint64_t ullm_gguf_alignment(const ullm_gguf *g) { return g ? g->alignment : 0; }
uint64_t ullm_gguf_data_start(const ullm_gguf *g) { return g ? g->data_start : 0; }

size_t ullm_gguf_tensor_count(const ullm_gguf *g) { return g ? g->tensors.size() : 0; }
int ullm_gguf_tensor_at(const ullm_gguf *g, size_t i, ullm_gguf_tensor *out) {
    if (!g || !out || i >= g->tensors.size()) return ULLM_GGUF_ERR_INVALID;
    fill(g, g->tensors[i], out);
    return ULLM_GGUF_OK;
}
int ullm_gguf_tensor_find(const ullm_gguf *g, const char *name, ullm_gguf_tensor *out) {
    if (!g || !name || !out) return ULLM_GGUF_ERR_INVALID;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return ULLM_GGUF_ERR_MISSING;
    fill(g, g->tensors[it->second], out);
    return ULLM_GGUF_OK;
}

size_t ullm_gguf_meta_count(const ullm_gguf *g) { return g ? g->meta_keys.size() : 0; }
const char *ullm_gguf_meta_key_at(const ullm_gguf *g, size_t i) { return g && i < g->meta_keys.size() ? g->meta_keys[i]->c_str() : nullptr; }
int ullm_gguf_meta_type(const ullm_gguf *g, const char *key, int *type_id, int *elem_type_id, uint64_t *array_len) {
    if (!g || !key) return ULLM_GGUF_ERR_INVALID;
    const Value *v = g->find(key);
    if (!v) return ULLM_GGUF_ERR_MISSING;
    if (type_id) *type_id = (int)v->type;
    if (elem_type_id) *elem_type_id = v->type == T_ARRAY ? (int)v->elem_type : -1;
    if (array_len) *array_len = v->type == T_ARRAY ? v->items.size() : 0;
    return ULLM_GGUF_OK;
}
int ullm_gguf_meta_u64(const ullm_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return ULLM_GGUF_ERR_INVALID;
    const Value *v = g->find(key);
    if (!v || !v->is_int()) return ULLM_GGUF_ERR_MISSING;
    *out = v->u;
    return ULLM_GGUF_OK;
}
int ullm_gguf_meta_f32(const ullm_gguf *g, const char *key, float *out) {
    if (!g || !key || !out) return ULLM_GGUF_ERR_INVALID;
    const Value *v = g->find(key);
    if (!v || !v->is_float()) return ULLM_GGUF_ERR_MISSING;
    *out = (float)v->f;
    return ULLM_GGUF_OK;
}
int ullm_gguf_meta_str(const ullm_gguf *g, const char *key, const char **s, size_t *len) {
    if (!g || !key || !s) return ULLM_GGUF_ERR_INVALID;
    const Value *v = g->find(key);
    if (!v || v->type != T_STRING) return ULLM_GGUF_ERR_MISSING;
    *s = v->s.c_str();
    if (len) *len = v->s.size();
    return ULLM_GGUF_OK;
}
static const Value *array_item(const ullm_gguf *g, const char *key, size_t i) {
    if (!g || !key) return nullptr;
    const Value *v = g->find(key);
    if (!v || v->type != T_ARRAY || i >= v->items.size()) return nullptr;
    return &v->items[i];
}
int ullm_gguf_meta_array_u64(const ullm_gguf *g, const char *key, size_t i, uint64_t *out) {
    const Value *v = array_item(g, key, i);
    if (!v || !out || !v->is_int()) return ULLM_GGUF_ERR_MISSING;
    *out = v->u;
    return ULLM_GGUF_OK;
}
int ullm_gguf_meta_array_f32(const ullm_gguf *g, const char *key, size_t i, float *out) {
    const Value *v = array_item(g, key, i);
    if (!v || !out || !v->is_float()) return ULLM_GGUF_ERR_MISSING;
    *out = (float)v->f;
    return ULLM_GGUF_OK;
}
int ullm_gguf_meta_array_str(const ullm_gguf *g, const char *key, size_t i, const char **s, size_t *len) {
    const Value *v = array_item(g, key, i);
    if (!v || !s || v->type != T_STRING) return ULLM_GGUF_ERR_MISSING;
    *s = v->s.c_str();
    if (len) *len = v->s.size();
    return ULLM_GGUF_OK;
}

int ullm_gguf_llama_params_get(const ullm_gguf *g, ullm_gguf_llama_params *out, char *err, size_t err_cap) {
    if (!g || !out) return ULLM_GGUF_ERR_INVALID;
    if (g->arch != "llama" && g->arch != "qwen2") { // lib.rs:200-209; "gemma3" needs kernels this backend does not have
        char m[160];
        snprintf(m, sizeof m, "architecture '%s' is not supported by this backend (llama, qwen2)", g->arch.c_str());
        put_err(err, err_cap, m);
        return ULLM_GGUF_ERR_UNSUPPORTED;
    }
    auto opt_u = [&](const char *suffix, uint64_t *v) {
        return ullm_gguf_meta_u64(g, (g->arch + "." + suffix).c_str(), v) == ULLM_GGUF_OK;
    };
    auto req_u = [&](const char *suffix, uint64_t *v) {
        if (opt_u(suffix, v)) return true;
        char m[160];
        snprintf(m, sizeof m, "missing metadata '%s.%s'", g->arch.c_str(), suffix);
        put_err(err, err_cap, m);
        return false;
    };
    ullm_gguf_llama_params p{};
    if (!req_u("embedding_length", &p.n_embd) || !req_u("attention.head_count", &p.n_head) || !req_u("block_count", &p.n_layer) ||
        !req_u("feed_forward_length", &p.n_ff))
        return ULLM_GGUF_ERR_FORMAT;
    if (!opt_u("attention.head_count_kv", &p.n_kv_head)) p.n_kv_head = p.n_head;
    if (!opt_u("context_length", &p.n_ctx)) p.n_ctx = 2048;
    if (p.n_ctx > 8192) p.n_ctx = 8192;
    if (!opt_u("attention.key_length", &p.head_dim)) {
        if (p.n_head == 0) {
            put_err(err, err_cap, "attention.head_count is zero");
            return ULLM_GGUF_ERR_FORMAT;
        }
        p.head_dim = p.n_embd / p.n_head;
    }
    if (ullm_gguf_meta_f32(g, (g->arch + ".rope.freq_base").c_str(), &p.rope_theta) != ULLM_GGUF_OK) p.rope_theta = 10000.0f;
    if (ullm_gguf_meta_f32(g, (g->arch + ".attention.layer_norm_rms_epsilon").c_str(), &p.eps) != ULLM_GGUF_OK) p.eps = 1e-5f;
    if (!opt_u("vocab_size", &p.vocab)) {
        int t = 0, et = 0;
        uint64_t n = 0;
        p.vocab = ullm_gguf_meta_type(g, "tokenizer.ggml.tokens", &t, &et, &n) == ULLM_GGUF_OK && t == (int)T_ARRAY ? n : 0;
    }
    *out = p;
    return ULLM_GGUF_OK;
}

} // extern "C"
