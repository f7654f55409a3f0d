// SafeTensors / MLX model-directory reader (host code only; see include/ullm_safetensors.h for the
// rules it follows and the reference lines they come from).
#include "../../include/ullm_safetensors.h"

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
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

constexpr int DT_F32 = 0, DT_F16 = 1, DT_BF16 = 30, DT_MLX_U32 = 1000; // ULLM_DTYPE_* of ullm_cuda.h

struct Failure {
    int code;
    std::string msg;
};
[[noreturn]] void fail(int code, const char *fmt, ...) {
    char buf[384];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw Failure{code, buf};
}

// ---- JSON (RFC 8259) with the readings the reference takes through serde_json ----
// Numbers keep three forms like serde_json's `Number`: a non-negative integer that fits u64, a
// negative integer that fits i64, anything else a double.  `as_u64` succeeds only for the first.
struct Json {
    enum Kind { Null, Bool, PosInt, NegInt, Float, String, Array, Object } kind = Null;
    bool b = false;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    std::string s;
    std::vector<Json> items;
    std::map<std::string, Json> members; // ascending keys, a repeated key keeps the last value

    const Json *get(const std::string &key) const {
        if (kind != Object) return nullptr;
        auto it = members.find(key);
        return it == members.end() ? nullptr : &it->second;
    }
    bool as_u64(uint64_t &out) const {
        if (kind != PosInt) return false;
        out = u;
        return true;
    }
    bool as_f64(double &out) const {
        if (kind == PosInt) out = (double)u;
        else if (kind == NegInt) out = (double)i;
        else if (kind == Float) out = f;
        else return false;
        return true;
    }
};

struct JsonParser {
    const uint8_t *p, *end;
    int depth = 0;
    [[noreturn]] void bad(const char *what) { throw std::string(what); }
    void ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool lit(const char *w) {
        const size_t n = strlen(w);
        if ((size_t)(end - p) < n || memcmp(p, w, n)) return false;
        p += n;
        return true;
    }
    unsigned hex4() {
        if (end - p < 4) bad("EOF in \\u escape");
        unsigned v = 0;
        for (int k = 0; k < 4; ++k, ++p) {
            const uint8_t c = *p;
            v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : (bad("invalid \\u escape"), 0u));
        }
        return v;
    }
    static void utf8(std::string &o, unsigned cp) {
        if (cp < 0x80) o += (char)cp;
        else if (cp < 0x800) o += (char)(0xC0 | cp >> 6), o += (char)(0x80 | (cp & 63));
        else if (cp < 0x10000) o += (char)(0xE0 | cp >> 12), o += (char)(0x80 | ((cp >> 6) & 63)), o += (char)(0x80 | (cp & 63));
        else o += (char)(0xF0 | cp >> 18), o += (char)(0x80 | ((cp >> 12) & 63)), o += (char)(0x80 | ((cp >> 6) & 63)), o += (char)(0x80 | (cp & 63));
    }
    // one UTF-8 sequence starting at p (lead byte >= 0x80) must be well formed
    void utf8_seq(std::string &o) {
        const uint8_t c = *p;
        int n = c >= 0xF0 ? 3 : c >= 0xE0 ? 2 : c >= 0xC0 ? 1 : -1;
        if (n < 0 || c > 0xF4 || end - p <= n) bad("invalid UTF-8 in string");
        unsigned cp = c & (0x3F >> n);
        for (int k = 1; k <= n; ++k) {
            if ((p[k] & 0xC0) != 0x80) bad("invalid UTF-8 in string");
            cp = cp << 6 | (p[k] & 0x3F);
        }
        static const unsigned lo[4] = {0, 0x80, 0x800, 0x10000};
        if (cp < lo[n] || cp > 0x10FFFF || (cp >= 0xD800 && cp <= 0xDFFF)) bad("invalid UTF-8 in string");
        o.append((const char *)p, n + 1);
        p += n + 1;
    }
    std::string string() { // p is just past the opening quote
        std::string o;
        for (;;) {
            if (p >= end) bad("EOF while parsing a string");
            const uint8_t c = *p;
            if (c == '"') {
                ++p;
                return o;
            }
            if (c < 0x20) bad("control character in string");
            if (c >= 0x80) {
                utf8_seq(o);
                continue;
            }
            ++p;
            if (c != '\\') {
                o += (char)c;
                continue;
            }
            if (p >= end) bad("EOF in escape");
            const uint8_t e = *p++;
            switch (e) {
            case '"': o += '"'; break;
            case '\\': o += '\\'; break;
            case '/': o += '/'; break;
            case 'b': o += '\b'; break;
            case 'f': o += '\f'; break;
            case 'n': o += '\n'; break;
            case 'r': o += '\r'; break;
            case 't': o += '\t'; break;
            case 'u': {
                unsigned cp = hex4();
                if (cp >= 0xDC00 && cp <= 0xDFFF) bad("lone trailing surrogate");
                if (cp >= 0xD800 && cp <= 0xDBFF) {
                    if (end - p < 2 || p[0] != '\\' || p[1] != 'u') bad("lone leading surrogate");
                    p += 2;
                    const unsigned lo = hex4();
                    if (lo < 0xDC00 || lo > 0xDFFF) bad("lone leading surrogate");
                    cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                }
                utf8(o, cp);
                break;
            }
            default: bad("invalid escape");
            }
        }
    }
    Json number() {
        const uint8_t *s = p;
        const bool neg = p < end && *p == '-';
        if (neg) ++p;
        if (p >= end || *p < '0' || *p > '9') bad("invalid number");
        if (*p == '0') {
            ++p;
            if (p < end && *p >= '0' && *p <= '9') bad("invalid number");
        } else
            while (p < end && *p >= '0' && *p <= '9') ++p;
        bool integral = true;
        if (p < end && *p == '.') {
            integral = false;
            ++p;
            if (p >= end || *p < '0' || *p > '9') bad("invalid number");
            while (p < end && *p >= '0' && *p <= '9') ++p;
        }
        if (p < end && (*p == 'e' || *p == 'E')) {
            integral = false;
            ++p;
            if (p < end && (*p == '+' || *p == '-')) ++p;
            if (p >= end || *p < '0' || *p > '9') bad("invalid number");
            while (p < end && *p >= '0' && *p <= '9') ++p;
        }
        const std::string tok((const char *)s, (size_t)(p - s));
        Json j;
        if (integral) {
            errno = 0;
            if (!neg) {
                const unsigned long long v = strtoull(tok.c_str(), nullptr, 10);
                if (errno == 0) {
                    j.kind = Json::PosInt, j.u = v;
                    return j;
                }
            } else {
                const long long v = strtoll(tok.c_str(), nullptr, 10);
                if (errno == 0) {
                    if (v == 0) j.kind = Json::Float, j.f = -0.0; // "-0" is the float -0.0 in serde_json
                    else j.kind = Json::NegInt, j.i = v;
                    return j;
                }
            }
        }
        j.kind = Json::Float, j.f = strtod(tok.c_str(), nullptr);
        if (!std::isfinite(j.f)) bad("number out of range");
        return j;
    }
    Json value() {
        ws();
        if (p >= end) bad("EOF while parsing a value");
        if (++depth > 128) bad("recursion limit exceeded");
        Json j;
        const uint8_t c = *p;
        if (c == '{') {
            ++p;
            j.kind = Json::Object;
            ws();
            if (p < end && *p == '}') ++p;
            else
                for (;;) {
                    ws();
                    if (p >= end || *p != '"') bad("key must be a string");
                    ++p;
                    std::string k = string();
                    ws();
                    if (p >= end || *p != ':') bad("expected ':'");
                    ++p;
                    j.members[std::move(k)] = value();
                    ws();
                    if (p < end && *p == ',') {
                        ++p;
                        continue;
                    }
                    if (p < end && *p == '}') {
                        ++p;
                        break;
                    }
                    bad("expected ',' or '}'");
                }
        } else if (c == '[') {
            ++p;
            j.kind = Json::Array;
            ws();
            if (p < end && *p == ']') ++p;
            else
                for (;;) {
                    j.items.push_back(value());
                    ws();
                    if (p < end && *p == ',') {
                        ++p;
                        continue;
                    }
                    if (p < end && *p == ']') {
                        ++p;
                        break;
                    }
                    bad("expected ',' or ']'");
                }
        } else if (c == '"') {
            ++p;
            j.kind = Json::String, j.s = string();
        } else if (c == 't') {
            if (!lit("true")) bad("expected ident");
            j.kind = Json::Bool, j.b = true;
        } else if (c == 'f') {
            if (!lit("false")) bad("expected ident");
            j.kind = Json::Bool, j.b = false;
        } else if (c == 'n') {
            if (!lit("null")) bad("expected ident");
        } else if (c == '-' || (c >= '0' && c <= '9'))
            j = number();
        else
            bad("expected value");
        --depth;
        return j;
    }
};

// serde_json::from_slice: one value, then only whitespace.  Throws std::string on a syntax error.
Json json_parse(const uint8_t *buf, size_t len) {
    JsonParser ps{buf, buf + len};
    Json j = ps.value();
    ps.ws();
    if (ps.p != ps.end) throw std::string("trailing characters");
    return j;
}

} // namespace

namespace {

struct Shard {
    const uint8_t *data = nullptr;
    size_t len = 0;
    bool mapped = false;
    std::vector<uint8_t> owned; // from_bytes keeps a copy
    Shard() = default;
    Shard(const Shard &) = delete;
    Shard &operator=(const Shard &) = delete;
    ~Shard() {
        if (mapped && data) munmap((void *)data, len);
    }
};

struct Tensor {
    std::string name;
    int dtype = 0;
    std::vector<uint64_t> shape;
    uint32_t shard = 0;
    uint64_t offset = 0;
};

size_t elem_size(int dtype) { return dtype == DT_F32 || dtype == DT_MLX_U32 ? 4 : 2; }

bool read_file(const std::string &path, std::vector<uint8_t> &out) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    uint8_t buf[1 << 16];
    size_t n;
    out.clear();
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.insert(out.end(), buf, buf + n);
    const bool ok = !ferror(f);
    fclose(f);
    return ok;
}

bool is_dir(const std::string &p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
bool exists(const std::string &p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

int parse_dtype(const std::string &s) { // lib.rs:229-241
    if (s == "F32") return DT_F32;
    if (s == "F16") return DT_F16;
    if (s == "BF16") return DT_BF16;
    if (s == "U32" || s == "I32") return DT_MLX_U32;
    fail(ULLM_ST_ERR_UNSUPPORTED, "SafeTensors dtype '%s' (only F32/F16/BF16/U32 are supported)", s.c_str());
}

} // namespace

struct ullm_st {
    std::vector<std::unique_ptr<Shard>> shards;
    std::map<std::string, Tensor> tensors;
    std::vector<const Tensor *> order; // ascending names, filled once loading is done
    Json config;                       // {} when there is no config.json
    std::string dir;                   // empty for a bare file
    bool has_dir = false;

    // add_shard, lib.rs:108-167
    void add_shard(std::unique_ptr<Shard> sh) {
        const uint32_t idx = (uint32_t)shards.size();
        const uint8_t *buf = sh->data;
        const size_t len = sh->len;
        if (len < 8) fail(ULLM_ST_ERR_FORMAT, "safetensors file too small");
        uint64_t header_len;
        memcpy(&header_len, buf, 8);
        if (header_len > len - 8) fail(ULLM_ST_ERR_FORMAT, "safetensors header out of bounds");
        const uint64_t data_start = 8 + header_len;
        Json header;
        try {
            header = json_parse(buf + 8, (size_t)header_len);
        } catch (const std::string &e) {
            fail(ULLM_ST_ERR_FORMAT, "safetensors header: %s", e.c_str());
        }
        if (header.kind != Json::Object) fail(ULLM_ST_ERR_FORMAT, "safetensors header is not an object");
        for (const auto &kv : header.members) {
            const std::string &name = kv.first;
            if (name == "__metadata__") continue;
            const Json &info = kv.second;
            const Json *dt = info.get("dtype");
            if (!dt || dt->kind != Json::String) fail(ULLM_ST_ERR_FORMAT, "tensor '%s': missing dtype", name.c_str());
            Tensor t;
            t.name = name;
            t.dtype = parse_dtype(dt->s);
            const Json *shape = info.get("shape");
            if (!shape || shape->kind != Json::Array) fail(ULLM_ST_ERR_FORMAT, "tensor '%s': missing shape", name.c_str());
            if (shape->items.size() > 8) fail(ULLM_ST_ERR_UNSUPPORTED, "tensor '%s': more than 8 dimensions", name.c_str());
            for (const Json &d : shape->items) {
                uint64_t v = 0;
                d.as_u64(v);
                t.shape.push_back(v);
            }
            const Json *offs = info.get("data_offsets");
            if (!offs || offs->kind != Json::Array) fail(ULLM_ST_ERR_FORMAT, "tensor '%s': missing data_offsets", name.c_str());
            uint64_t begin = 0;
            if (!offs->items.empty()) offs->items[0].as_u64(begin);
            t.shard = idx;
            t.offset = begin > UINT64_MAX - data_start ? UINT64_MAX : data_start + begin; // a wrapping offset lies outside every file
            tensors[name] = std::move(t);
        }
        shards.push_back(std::move(sh));
    }

    // byte_len + the bounds test of tensor_data (lib.rs:219-226, 245-252): 0 = the bytes are not all there
    uint64_t data_len(const Tensor &t) const {
        unsigned __int128 n = elem_size(t.dtype);
        for (uint64_t d : t.shape) {
            n *= d;
            if (n > (unsigned __int128)UINT64_MAX) return 0;
        }
        const Shard &sh = *shards[t.shard];
        if (t.offset > sh.len || (uint64_t)n > sh.len - t.offset) return 0;
        return (uint64_t)n;
    }
    bool empty_ok(const Tensor &t) const { // a zero-element tensor inside the file has data of length 0
        return t.offset <= shards[t.shard]->len;
    }
    void describe(const Tensor &t, ullm_st_tensor *o) const {
        memset(o, 0, sizeof *o);
        o->name = t.name.c_str(), o->dtype = t.dtype, o->n_dims = (uint32_t)t.shape.size();
        for (size_t d = 0; d < t.shape.size(); ++d) o->shape[d] = t.shape[d];
        o->shard = t.shard, o->offset = t.offset;
        o->nbytes = data_len(t);
        bool zero = false;
        for (uint64_t d : t.shape) zero = zero || d == 0;
        o->data = (o->nbytes || (zero && empty_ok(t))) ? shards[t.shard]->data + t.offset : nullptr;
    }
    void finish() {
        order.clear();
        for (const auto &kv : tensors) order.push_back(&kv.second);
    }
    const Json *walk(const char *path) const {
        const Json *j = &config;
        std::string part;
        for (const char *p = path;; ++p) {
            if (*p && *p != '.') {
                part += *p;
                continue;
            }
            if (j->kind == Json::Object) j = j->get(part);
            else if (j->kind == Json::Array && !part.empty() && part.find_first_not_of("0123456789") == std::string::npos && part.size() < 10) {
                const size_t i = (size_t)atol(part.c_str());
                j = i < j->items.size() ? &j->items[i] : nullptr;
            } else
                j = nullptr;
            if (!j || !*p) return j;
            part.clear();
        }
    }
};

namespace {

std::unique_ptr<Shard> map_file(const std::string &path) {
    // std::fs::File::open failure is reported as a format error by the reference (lib.rs:109-110);
    // a failed mapping (an empty file cannot be mapped) is an I/O error (lib.rs:112)
    const int fd = open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd < 0) fail(ULLM_ST_ERR_FORMAT, "open %s: %s", path.c_str(), strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0 || !S_ISREG(st.st_mode)) {
        close(fd);
        fail(ULLM_ST_ERR_IO, "mmap %s: not a mappable file", path.c_str());
    }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) fail(ULLM_ST_ERR_IO, "mmap %s: %s", path.c_str(), strerror(errno));
    auto sh = std::make_unique<Shard>();
    sh->data = (const uint8_t *)m, sh->len = (size_t)st.st_size, sh->mapped = true;
    return sh;
}

void open_dir(ullm_st &m, const std::string &dir) { // lib.rs:59-104
    std::vector<uint8_t> bytes;
    if (read_file(dir + "/config.json", bytes)) {
        try {
            m.config = json_parse(bytes.data(), bytes.size());
        } catch (const std::string &e) {
            fail(ULLM_ST_ERR_FORMAT, "config.json: %s", e.c_str());
        }
    }
    m.dir = dir, m.has_dir = true;
    const std::string index_path = dir + "/model.safetensors.index.json";
    if (exists(index_path)) {
        if (!read_file(index_path, bytes)) fail(ULLM_ST_ERR_IO, "read %s", index_path.c_str());
        Json index;
        try {
            index = json_parse(bytes.data(), bytes.size());
        } catch (const std::string &e) {
            fail(ULLM_ST_ERR_FORMAT, "index.json: %s", e.c_str());
        }
        const Json *map = index.get("weight_map");
        if (!map || map->kind != Json::Object) fail(ULLM_ST_ERR_FORMAT, "index.json: missing weight_map");
        std::vector<std::string> files;
        for (const auto &kv : map->members)
            if (kv.second.kind == Json::String) files.push_back(kv.second.s);
        std::sort(files.begin(), files.end());
        files.erase(std::unique(files.begin(), files.end()), files.end());
        for (const std::string &f : files) m.add_shard(map_file(dir + "/" + f));
    } else {
        const std::string single = dir + "/model.safetensors";
        if (!exists(single)) fail(ULLM_ST_ERR_FORMAT, "no model.safetensors or index.json in directory");
        m.add_shard(map_file(single));
    }
}

template <typename F> int guarded(ullm_st **out, char *err, size_t err_cap, F &&body) {
    if (err && err_cap) err[0] = 0;
    if (!out) return ULLM_ST_ERR_INVALID;
    *out = nullptr;
    try {
        std::unique_ptr<ullm_st> m(new ullm_st());
        m->config.kind = Json::Object;
        body(*m);
        m->finish();
        *out = m.release();
        return ULLM_ST_OK;
    } catch (const Failure &f) {
        if (err && err_cap) snprintf(err, err_cap, "%s", f.msg.c_str());
        return f.code;
    } catch (const std::bad_alloc &) {
        if (err && err_cap) snprintf(err, err_cap, "out of memory");
        return ULLM_ST_ERR_IO;
    }
}

template <typename F> int guarded_call(char *err, size_t err_cap, F &&body) {
    if (err && err_cap) err[0] = 0;
    try {
        body();
        return ULLM_ST_OK;
    } catch (const Failure &f) {
        if (err && err_cap) snprintf(err, err_cap, "%s", f.msg.c_str());
        return f.code;
    }
}

} // namespace

extern "C" {

int ullm_st_open(const char *path, ullm_st **out, char *err, size_t err_cap) {
    if (!path) return ULLM_ST_ERR_INVALID;
    return guarded(out, err, err_cap, [&](ullm_st &m) {
        const std::string p(path);
        if (is_dir(p)) open_dir(m, p);
        else m.add_shard(map_file(p));
    });
}

int ullm_st_from_bytes(const void *bytes, size_t len, ullm_st **out, char *err, size_t err_cap) {
    if (!bytes && len) return ULLM_ST_ERR_INVALID;
    return guarded(out, err, err_cap, [&](ullm_st &m) {
        auto sh = std::make_unique<Shard>();
        sh->owned.assign((const uint8_t *)bytes, (const uint8_t *)bytes + len);
        sh->data = sh->owned.data(), sh->len = len;
        m.add_shard(std::move(sh));
    });
}

void ullm_st_close(ullm_st *m) { delete m; }

size_t ullm_st_shard_count(const ullm_st *m) { return m ? m->shards.size() : 0; }
size_t ullm_st_tensor_count(const ullm_st *m) { return m ? m->order.size() : 0; }

int ullm_st_tensor_at(const ullm_st *m, size_t i, ullm_st_tensor *out) {
    if (!m || !out) return ULLM_ST_ERR_INVALID;
    if (i >= m->order.size()) return ULLM_ST_ERR_MISSING;
    m->describe(*m->order[i], out);
    return ULLM_ST_OK;
}

int ullm_st_tensor_find(const ullm_st *m, const char *name, ullm_st_tensor *out) {
    if (!m || !name || !out) return ULLM_ST_ERR_INVALID;
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return ULLM_ST_ERR_MISSING;
    m->describe(it->second, out);
    return ULLM_ST_OK;
}

int ullm_st_has_tensor(const ullm_st *m, const char *name) { return m && name && m->tensors.count(name) ? 1 : 0; }

int ullm_st_config_u64(const ullm_st *m, const char *path, uint64_t *out) {
    if (!m || !path || !out) return ULLM_ST_ERR_INVALID;
    const Json *j = m->walk(path);
    return j && j->as_u64(*out) ? ULLM_ST_OK : ULLM_ST_ERR_MISSING;
}

int ullm_st_config_f32(const ullm_st *m, const char *path, float *out) {
    if (!m || !path || !out) return ULLM_ST_ERR_INVALID;
    const Json *j = m->walk(path);
    double d;
    if (!j || !j->as_f64(d)) return ULLM_ST_ERR_MISSING;
    *out = (float)d;
    return ULLM_ST_OK;
}

int ullm_st_config_str(const ullm_st *m, const char *path, const char **s, size_t *len) {
    if (!m || !path || !s) return ULLM_ST_ERR_INVALID;
    const Json *j = m->walk(path);
    if (!j || j->kind != Json::String) return ULLM_ST_ERR_MISSING;
    *s = j->s.c_str();
    if (len) *len = j->s.size();
    return ULLM_ST_OK;
}

int ullm_st_has_text_config(const ullm_st *m) { return m && m->config.get("text_config") ? 1 : 0; }
int ullm_st_has_tokenizer_json(const ullm_st *m) { return m && m->has_dir && exists(m->dir + "/tokenizer.json") ? 1 : 0; }

} // extern "C"

namespace {

// one of the three tensors of an MLX linear, with the type and the element count it must have
const void *mlx_part(const ullm_st *m, const std::string &name, int dtype, uint64_t elems) {
    ullm_st_tensor t;
    if (ullm_st_tensor_find(m, name.c_str(), &t)) fail(ULLM_ST_ERR_FORMAT, "missing tensor '%s'", name.c_str());
    if (t.dtype != dtype) fail(ULLM_ST_ERR_FORMAT, "tensor '%s' is not %s", name.c_str(), dtype == DT_MLX_U32 ? "U32" : "BF16");
    if (!t.data || t.nbytes != elems * elem_size(dtype))
        fail(ULLM_ST_ERR_FORMAT, "tensor '%s': %llu bytes in the file, %llu expected", name.c_str(), (unsigned long long)t.nbytes,
             (unsigned long long)(elems * elem_size(dtype)));
    return t.data;
}

void mlx_geometry(const std::string &name, uint64_t out_dim, uint64_t in_dim, uint64_t group) {
    if (!group || !out_dim || !in_dim || in_dim % 8 || in_dim % group)
        fail(ULLM_ST_ERR_FORMAT, "'%s': [%llu, %llu] with groups of %llu is not an MLX 4-bit layout", name.c_str(), (unsigned long long)out_dim,
             (unsigned long long)in_dim, (unsigned long long)group);
    if (out_dim > (1ull << 40) / in_dim) fail(ULLM_ST_ERR_FORMAT, "'%s': matrix too large", name.c_str());
}

} // namespace

extern "C" {

int ullm_st_mlx_weight_get(const ullm_st *m, const char *name, uint64_t group, ullm_st_mlx_weight *out, char *err, size_t err_cap) {
    if (!m || !name || !out) return ULLM_ST_ERR_INVALID;
    return guarded_call(err, err_cap, [&] {
        memset(out, 0, sizeof *out);
        const std::string base(name);
        ullm_st_tensor w;
        if (ullm_st_tensor_find(m, (base + ".weight").c_str(), &w)) fail(ULLM_ST_ERR_FORMAT, "missing '%s.weight'", name);
        if (w.n_dims != 2) fail(ULLM_ST_ERR_FORMAT, "'%s.weight' is not a matrix", name);
        const uint64_t out_dim = w.shape[0], in_dim = w.shape[1] * 8; // mlx.rs:35-36
        mlx_geometry(base, out_dim, in_dim, group);
        out->weight = (const uint32_t *)mlx_part(m, base + ".weight", DT_MLX_U32, out_dim * (in_dim / 8));
        out->scales = (const uint16_t *)mlx_part(m, base + ".scales", DT_BF16, out_dim * (in_dim / group));
        out->biases = (const uint16_t *)mlx_part(m, base + ".biases", DT_BF16, out_dim * (in_dim / group));
        out->out = out_dim, out->in = in_dim, out->group = group;
    });
}

int ullm_st_mlx_experts_get(const ullm_st *m, const char *name, uint64_t n_experts, uint64_t out_dim, uint64_t in_dim, uint64_t group,
                            uint64_t expert, ullm_st_mlx_weight *out, char *err, size_t err_cap) {
    if (!m || !name || !out) return ULLM_ST_ERR_INVALID;
    return guarded_call(err, err_cap, [&] {
        memset(out, 0, sizeof *out);
        const std::string base(name);
        mlx_geometry(base, out_dim, in_dim, group);
        if (!n_experts || n_experts > (1u << 20) || expert > n_experts) fail(ULLM_ST_ERR_FORMAT, "'%s': expert %llu of %llu", name, (unsigned long long)expert, (unsigned long long)n_experts);
        const uint64_t wpe = out_dim * (in_dim / 8), spe = out_dim * (in_dim / group); // words / table entries per expert, mlx.rs:71-72
        const uint32_t *w = (const uint32_t *)mlx_part(m, base + ".weight", DT_MLX_U32, n_experts * wpe);
        const uint16_t *s = (const uint16_t *)mlx_part(m, base + ".scales", DT_BF16, n_experts * spe);
        const uint16_t *b = (const uint16_t *)mlx_part(m, base + ".biases", DT_BF16, n_experts * spe);
        const bool all = expert == n_experts;
        out->weight = w + (all ? 0 : expert * wpe), out->scales = s + (all ? 0 : expert * spe), out->biases = b + (all ? 0 : expert * spe);
        out->out = all ? n_experts * out_dim : out_dim, out->in = in_dim, out->group = group;
    });
}

int ullm_st_mlx_params_get(const ullm_st *m, ullm_st_mlx_params *out, char *err, size_t err_cap) {
    if (!m || !out) return ULLM_ST_ERR_INVALID;
    return guarded_call(err, err_cap, [&] {
        memset(out, 0, sizeof *out);
        const char *arch = "";
        ullm_st_config_str(m, "architectures.0", &arch, nullptr);
        if (strcmp(arch, "Qwen3MoeForCausalLM"))
            fail(ULLM_ST_ERR_UNSUPPORTED, "MLX architecture '%s' is not supported yet (Qwen3MoeForCausalLM)", arch); // mlx.rs:111-115
        auto req = [&](const char *k) {
            uint64_t v;
            if (ullm_st_config_u64(m, k, &v)) fail(ULLM_ST_ERR_FORMAT, "config.json: missing '%s'", k);
            return v;
        };
        auto opt = [&](const char *k, uint64_t d) {
            uint64_t v;
            return ullm_st_config_u64(m, k, &v) ? d : v;
        };
        out->group = opt("quantization.group_size", 64);
        out->n_embd = req("hidden_size");
        out->n_head = req("num_attention_heads");
        out->n_layer = req("num_hidden_layers");
        out->n_kv_head = opt("num_key_value_heads", out->n_head);
        if (!out->n_head) fail(ULLM_ST_ERR_FORMAT, "config.json: num_attention_heads is 0");
        out->head_dim = opt("head_dim", out->n_embd / out->n_head);
        out->n_experts = req("num_experts");
        out->n_experts_used = req("num_experts_per_tok");
        out->moe_inter = req("moe_intermediate_size");
        out->n_ctx = std::min<uint64_t>(opt("max_position_embeddings", 8192), 8192);
        if (ullm_st_config_f32(m, "rope_theta", &out->rope_theta)) out->rope_theta = 1000000.0f;
        if (ullm_st_config_f32(m, "rms_norm_eps", &out->eps)) out->eps = 1e-6f;
        out->vocab = req("vocab_size");
    });
}

} // extern "C"
