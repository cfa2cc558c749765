// GGUF container reader (v2 / v3, one file): the data format on the weight side of the hot path.  The file is
// memory-mapped; tensor data is handed out as pointers into the mapping, so a weight goes file -> device with one
// upload and no intermediate copy (infr_cuda_upload_at from the pointer), and q / k / v can be placed back to back in
// one device buffer for the `w_off` slices a fused-QKV Linear takes.
//
// What Gguf::open of the reference checks is checked here (crates/infr-gguf/src/lib.rs:476, :735-870): magic, version
// 2 or 3, every read bounded by the file, metadata nesting depth, general.alignment a power of two within a cap, at
// most 8 dimensions, shape products and byte sizes that do not overflow, quantised tensors a whole number of blocks
// (block geometry of :370 / the ggml type table :330-356), tensor data inside the file.  A malformed file is an
// error code and a message, never a fault.  Split models (gguf-split shard sets) are not read.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/infr_cuda.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
constexpr uint64_t kDefaultAlignment = 32, kMaxAlignment = 1u << 20;
constexpr int kMaxDepth = 64;
constexpr uint32_t kMaxDims = 8;

enum MetaType : uint32_t { kU8, kI8, kU16, kI16, kU32, kI32, kF32, kBool, kStr, kArr, kU64, kI64, kF64 };

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0;  // unsigned / bool payload
    int64_t i = 0;   // signed payload
    double f = 0;    // floating payload
    const char *str = nullptr;
    uint64_t str_len = 0;
    // arrays: element type, count, and where the elements start in the mapping
    uint32_t elem_type = 0;
    uint64_t count = 0;
    const uint8_t *arr = nullptr;
};

// (elements per block, bytes per block) of a ggml tensor type; {0, 0}: a type this reader does not know
struct BlockGeom {
    uint32_t elems, bytes;
};
BlockGeom geom_of(uint32_t t) {
    switch (t) {
        case 0: return {1, 4};       // F32
        case 1: return {1, 2};       // F16
        case 2: return {32, 18};     // Q4_0
        case 3: return {32, 20};     // Q4_1
        case 6: return {32, 22};     // Q5_0
        case 7: return {32, 24};     // Q5_1
        case 8: return {32, 34};     // Q8_0
        case 9: return {32, 36};     // Q8_1
        case 10: return {256, 84};   // Q2_K
        case 11: return {256, 110};  // Q3_K
        case 12: return {256, 144};  // Q4_K
        case 13: return {256, 176};  // Q5_K
        case 14: return {256, 210};  // Q6_K
        case 15: return {256, 292};  // Q8_K
        case 16: return {256, 66};   // IQ2_XXS
        case 17: return {256, 74};   // IQ2_XS
        case 18: return {256, 98};   // IQ3_XXS
        case 19: return {256, 50};   // IQ1_S
        case 20: return {32, 18};    // IQ4_NL
        case 21: return {256, 110};  // IQ3_S
        case 22: return {256, 82};   // IQ2_S
        case 23: return {256, 136};  // IQ4_XS
        case 24: return {1, 1};      // I8
        case 25: return {1, 2};      // I16
        case 26: return {1, 4};      // I32
        case 27: return {1, 8};      // I64
        case 28: return {1, 8};      // F64
        case 29: return {256, 56};   // IQ1_M
        case 30: return {1, 2};      // BF16
        case 34: return {256, 54};   // TQ1_0
        case 35: return {256, 66};   // TQ2_0
        case 39: return {32, 17};    // MXFP4
        case 42: return {64, 18};    // Q2_0 (ternary, one f16 scale per 64)
        default: return {0, 0};
    }
}
// the dtype code this library runs the type under, or -1
int32_t dtype_of(uint32_t t) {
    switch (t) {
        case 0: return INFR_DT_F32;
        case 1: return INFR_DT_F16;
        case 26: return INFR_DT_I32;
        case 12: return INFR_DT_Q4K;
        case 14: return INFR_DT_Q6K;
        case 42: return INFR_DT_Q2_0;
        default: return -1;
    }
}

struct Cursor {
    const uint8_t *p;
    uint64_t len, pos = 0;
    bool ok = true;
    uint64_t left() const { return len - pos; }
    template <class T>
    T get() {
        T v{};
        if (!ok || left() < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    // a GGUF string: u64 length + bytes (not NUL-terminated in the file)
    bool str(const char **s, uint64_t *n) {
        const uint64_t l = get<uint64_t>();
        if (!ok || l > left()) {
            ok = false;
            return false;
        }
        *s = reinterpret_cast<const char *>(p + pos);
        *n = l;
        pos += l;
        return true;
    }
};

uint32_t scalar_size(uint32_t t) {
    switch (t) {
        case kU8: case kI8: case kBool: return 1;
        case kU16: case kI16: return 2;
        case kU32: case kI32: case kF32: return 4;
        case kU64: case kI64: case kF64: return 8;
        default: return 0;
    }
}

}  // namespace

struct infr_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    uint64_t len = 0;
    uint32_t version = 0;
    uint64_t alignment = kDefaultAlignment, data_start = 0;
    std::vector<std::string> names;  // NUL-terminated copies of the tensor names (the file's are not)
    std::vector<infr_gguf_tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
    std::unordered_map<std::string, MetaValue> meta;
    std::vector<std::string> keys;
};

namespace {

void set_err(char *err, size_t n, const char *f, ...) {
    if (!err || !n) return;
    va_list ap;
    va_start(ap, f);
    vsnprintf(err, n, f, ap);
    va_end(ap);
}

// Reads one metadata value of type t; arrays are skipped over element by element so that every byte is bounds-checked.
bool read_value(Cursor &c, uint32_t t, MetaValue *out, int depth, std::string *why) {
    if (depth > kMaxDepth) {
        *why = "metadata nested deeper than 64 levels";
        return false;
    }
    out->type = t;
    switch (t) {
        case kU8: out->u = c.get<uint8_t>(); break;
        case kI8: out->i = c.get<int8_t>(); break;
        case kU16: out->u = c.get<uint16_t>(); break;
        case kI16: out->i = c.get<int16_t>(); break;
        case kU32: out->u = c.get<uint32_t>(); break;
        case kI32: out->i = c.get<int32_t>(); break;
        case kF32: out->f = c.get<float>(); break;
        case kBool: out->u = c.get<uint8_t>() != 0; break;
        case kU64: out->u = c.get<uint64_t>(); break;
        case kI64: out->i = c.get<int64_t>(); break;
        case kF64: out->f = c.get<double>(); break;
        case kStr:
            if (!c.str(&out->str, &out->str_len)) {
                *why = "string runs past the end of the file";
                return false;
            }
            break;
        case kArr: {
            out->elem_type = c.get<uint32_t>();
            out->count = c.get<uint64_t>();
            if (!c.ok) break;
            out->arr = c.p + c.pos;
            const uint32_t sz = scalar_size(out->elem_type);
            if (sz) {
                if (out->count > c.left() / sz) {
                    *why = "array runs past the end of the file";
                    return false;
                }
                c.pos += out->count * sz;
            } else if (out->elem_type == kStr || out->elem_type == kArr) {
                if (out->count > c.left()) {  // every element takes at least one byte
                    *why = "array count exceeds the file";
                    return false;
                }
                for (uint64_t k = 0; k < out->count; k++) {
                    MetaValue skip;
                    if (!read_value(c, out->elem_type, &skip, depth + 1, why)) return false;
                }
            } else {
                *why = "unknown array element type " + std::to_string(out->elem_type);
                return false;
            }
            break;
        }
        default: *why = "unknown value type " + std::to_string(t); return false;
    }
    if (!c.ok) {
        *why = "value runs past the end of the file";
        return false;
    }
    return true;
}

}  // namespace

extern "C" {

INFR_API int32_t infr_gguf_open(const char *path, infr_gguf **out, char *err, size_t err_len) {
    if (!path || !out) return INFR_E_INVALID;
    *out = nullptr;
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) {
        set_err(err, err_len, "GGUF: cannot open %s", path);
        return INFR_E_INVALID;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        set_err(err, err_len, "GGUF: %s is shorter than a header", path);
        close(fd);
        return INFR_E_INVALID;
    }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (m == MAP_FAILED) {
        set_err(err, err_len, "GGUF: cannot map %s", path);
        close(fd);
        return INFR_E_INVALID;
    }
    auto *g = new infr_gguf();
    g->fd = fd;
    g->map = static_cast<const uint8_t *>(m);
    g->len = (uint64_t)st.st_size;
    auto fail = [&](int32_t code, const std::string &why) {
        set_err(err, err_len, "GGUF: %s", why.c_str());
        infr_gguf_close(g);
        return code;
    };
    Cursor c{g->map, g->len};
    const uint32_t magic = c.get<uint32_t>();
    if (magic != kMagic) {
        char b[96];
        snprintf(b, sizeof b, "not a GGUF file (magic 0x%08X, expected 0x%08X)", magic, kMagic);
        return fail(INFR_E_INVALID, b);
    }
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) return fail(INFR_E_UNSUPPORTED, "unsupported GGUF version " + std::to_string(g->version) + " (supported: 2, 3)");
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    // every entry takes at least a dozen bytes: counts beyond the file are rejected before anything is reserved
    if (n_kv > c.left() / 12 || n_tensors > c.left() / 24) return fail(INFR_E_INVALID, "header counts exceed the file");
    for (uint64_t k = 0; k < n_kv; k++) {
        const char *ks;
        uint64_t kl;
        if (!c.str(&ks, &kl)) return fail(INFR_E_INVALID, "metadata key runs past the end of the file");
        const uint32_t t = c.get<uint32_t>();
        MetaValue v;
        std::string why;
        if (!c.ok || !read_value(c, t, &v, 0, &why)) return fail(INFR_E_INVALID, why.empty() ? "metadata runs past the end of the file" : why);
        std::string key(ks, kl);
        if (!g->meta.count(key)) g->keys.push_back(key);
        g->meta[key] = v;
    }
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end()) {
        const MetaValue &v = al->second;
        const bool is_int = v.type == kU8 || v.type == kU16 || v.type == kU32 || v.type == kU64 || v.type == kI8 || v.type == kI16 || v.type == kI32 || v.type == kI64;
        const uint64_t a = (v.type == kI8 || v.type == kI16 || v.type == kI32 || v.type == kI64) ? (v.i < 0 ? 0 : (uint64_t)v.i) : v.u;
        if (!is_int || a == 0 || (a & (a - 1)) || a > kMaxAlignment) return fail(INFR_E_INVALID, "invalid general.alignment (a power of two up to 1 MiB)");
        g->alignment = a;
    }
    struct Raw {
        const char *name;
        uint64_t name_len;
        uint32_t n_dims;
        uint64_t dims[kMaxDims];
        uint32_t type;
        uint64_t off;
    };
    std::vector<Raw> raw;
    raw.reserve((size_t)n_tensors);
    for (uint64_t k = 0; k < n_tensors; k++) {
        Raw r{};
        if (!c.str(&r.name, &r.name_len)) return fail(INFR_E_INVALID, "tensor name runs past the end of the file");
        r.n_dims = c.get<uint32_t>();
        if (!c.ok || r.n_dims > kMaxDims) return fail(INFR_E_INVALID, "tensor '" + std::string(r.name, r.name_len) + "' declares more than 8 dimensions");
        for (uint32_t d = 0; d < r.n_dims; d++) r.dims[d] = c.get<uint64_t>();
        r.type = c.get<uint32_t>();
        r.off = c.get<uint64_t>();
        if (!c.ok) return fail(INFR_E_INVALID, "tensor table runs past the end of the file");
        raw.push_back(r);
    }
    g->data_start = (c.pos + g->alignment - 1) / g->alignment * g->alignment;
    g->names.reserve(raw.size());
    for (const Raw &r : raw) {
        const std::string name(r.name, r.name_len);
        const BlockGeom bg = geom_of(r.type);
        if (!bg.elems) return fail(INFR_E_UNSUPPORTED, "ggml type " + std::to_string(r.type) + " (tensor '" + name + "')");
        uint64_t numel = 1;
        for (uint32_t d = 0; d < r.n_dims; d++) {
            if (r.dims[d] && numel > UINT64_MAX / r.dims[d]) return fail(INFR_E_INVALID, "tensor '" + name + "' shape overflows");
            numel *= r.dims[d];
        }
        if (numel % bg.elems)
            return fail(INFR_E_INVALID, "tensor '" + name + "' has " + std::to_string(numel) + " elements, not a whole number of " +
                                            std::to_string(bg.elems) + "-element blocks");
        const uint64_t blocks = numel / bg.elems;
        if (blocks > UINT64_MAX / bg.bytes) return fail(INFR_E_INVALID, "tensor '" + name + "' byte size overflows");
        const uint64_t nbytes = blocks * bg.bytes;
        if (r.off % g->alignment) return fail(INFR_E_INVALID, "tensor '" + name + "' is not aligned to general.alignment");
        if (g->data_start > g->len || r.off > g->len - g->data_start || nbytes > g->len - g->data_start - r.off)
            return fail(INFR_E_INVALID, "tensor '" + name + "' lies outside the file");
        infr_gguf_tensor t{};
        g->names.push_back(name);
        t.ggml_type = r.type;
        t.dtype = dtype_of(r.type);
        t.n_dims = r.n_dims;
        for (uint32_t d = 0; d < kMaxDims; d++) t.dims[d] = d < r.n_dims ? r.dims[d] : 1;
        t.numel = numel;
        t.nbytes = nbytes;
        t.file_offset = g->data_start + r.off;
        if (g->by_name.count(name)) return fail(INFR_E_INVALID, "tensor '" + name + "' appears twice");
        g->by_name[name] = g->tensors.size();
        g->tensors.push_back(t);
    }
    for (size_t i = 0; i < g->tensors.size(); i++) g->tensors[i].name = g->names[i].c_str();  // (the vector no longer grows)
    *out = g;
    return INFR_OK;
}

INFR_API void infr_gguf_close(infr_gguf *g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t *>(g->map), (size_t)g->len);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

INFR_API uint32_t infr_gguf_version(const infr_gguf *g) { return g ? g->version : 0; }
INFR_API uint64_t infr_gguf_alignment(const infr_gguf *g) { return g ? g->alignment : 0; }
INFR_API uint64_t infr_gguf_tensor_count(const infr_gguf *g) { return g ? g->tensors.size() : 0; }

INFR_API int32_t infr_gguf_tensor_at(const infr_gguf *g, uint64_t index, infr_gguf_tensor *out) {
    if (!g || !out || index >= g->tensors.size()) return INFR_E_INVALID;
    *out = g->tensors[(size_t)index];
    return INFR_OK;
}

INFR_API int32_t infr_gguf_find(const infr_gguf *g, const char *name, infr_gguf_tensor *out) {
    if (!g || !name || !out) return INFR_E_INVALID;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return INFR_E_INVALID;
    *out = g->tensors[it->second];
    return INFR_OK;
}

INFR_API const void *infr_gguf_tensor_data(const infr_gguf *g, const infr_gguf_tensor *t) {
    if (!g || !t || t->file_offset > g->len || t->nbytes > g->len - t->file_offset) return nullptr;
    return g->map + t->file_offset;
}

INFR_API uint64_t infr_gguf_meta_count(const infr_gguf *g) { return g ? g->keys.size() : 0; }
INFR_API const char *infr_gguf_meta_key(const infr_gguf *g, uint64_t index) {
    return g && index < g->keys.size() ? g->keys[(size_t)index].c_str() : nullptr;
}
INFR_API int32_t infr_gguf_meta_type(const infr_gguf *g, const char *key) {
    if (!g || !key) return -1;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? -1 : (int32_t)it->second.type;
}

// Any integer or bool value as u64 (negative values are INFR_E_INVALID).
INFR_API int32_t infr_gguf_meta_u64(const infr_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return INFR_E_INVALID;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return INFR_E_INVALID;
    const MetaValue &v = it->second;
    switch (v.type) {
        case kU8: case kU16: case kU32: case kU64: case kBool: *out = v.u; return INFR_OK;
        case kI8: case kI16: case kI32: case kI64:
            if (v.i < 0) return INFR_E_INVALID;
            *out = (uint64_t)v.i;
            return INFR_OK;
        default: return INFR_E_INVALID;
    }
}

// Any numeric value as f64.
INFR_API int32_t infr_gguf_meta_f64(const infr_gguf *g, const char *key, double *out) {
    if (!g || !key || !out) return INFR_E_INVALID;
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return INFR_E_INVALID;
    const MetaValue &v = it->second;
    switch (v.type) {
        case kF32: case kF64: *out = v.f; return INFR_OK;
        case kU8: case kU16: case kU32: case kU64: *out = (double)v.u; return INFR_OK;
        case kI8: case kI16: case kI32: case kI64: *out = (double)v.i; return INFR_OK;
        default: return INFR_E_INVALID;
    }
}

// A string value: pointer into the mapping (not NUL-terminated) and its length.
INFR_API int32_t infr_gguf_meta_str(const infr_gguf *g, const char *key, const char **s, uint64_t *len) {
    if (!g || !key || !s || !len) return INFR_E_INVALID;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != kStr) return INFR_E_INVALID;
    *s = it->second.str;
    *len = it->second.str_len;
    return INFR_OK;
}

// An array value: element type (GGUF value type code), count, and for fixed-size element types the packed elements.
INFR_API int32_t infr_gguf_meta_array(const infr_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count, const void **data) {
    if (!g || !key || !elem_type || !count) return INFR_E_INVALID;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != kArr) return INFR_E_INVALID;
    *elem_type = it->second.elem_type;
    *count = it->second.count;
    if (data) *data = scalar_size(it->second.elem_type) ? it->second.arr : nullptr;
    return INFR_OK;
}

}  // extern "C"
