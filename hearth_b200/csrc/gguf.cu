// GGUF reader: the loader side of the drop-in, so that a model file goes from disk to resident device weights
// without the caller parsing anything.  Mirrors hearth_gguf::GgufFile (hearth-gguf/src/gguf.rs:137-259): magic
// "GGUF", version 2 or 3, little-endian; metadata key/values of the thirteen GGUF value types; tensor infos (name,
// shape with the innermost dimension first, GGML type id, offset); the data section starts at the next multiple of
// general.alignment (default 32) in version 3 and right after the infos in version 2.  Host code only: the file is
// mapped read-only and tensors are uploaded straight from the mapping.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/hb200.h"
#include "common.cuh"

namespace {

struct MetaValue {
    uint32_t type = 0;          // GGUF value type id; 9 = array
    uint32_t elem_type = 0;     // for arrays
    uint64_t u = 0;             // integers and bool, zero- or sign-extended
    double f = 0.0;             // f32 / f64
    std::string s;              // string
    std::vector<MetaValue> items;
};

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> shape;
    uint32_t dtype_id = 0;
    uint64_t offset = 0;
};

}  // namespace

struct hb200_gguf {
    int fd = -1;
    const uint8_t* data = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0;
    std::map<std::string, MetaValue> meta;
    std::vector<TensorInfo> tensors;
};

namespace {

using hb200::set_error;

struct Reader {
    const uint8_t* d;
    size_t n, pos;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (pos + sizeof(T) > n) { ok = false; return v; }
        memcpy(&v, d + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok || len > n - pos) { ok = false; return std::string(); }
        std::string s(reinterpret_cast<const char*>(d + pos), (size_t)len);
        pos += (size_t)len;
        return s;
    }
};

// Type ids GgmlDType::from_id accepts (hearth-gguf/src/ggml.rs:58-103); anything else fails the open, as there.
bool known_dtype(uint32_t id) {
    return id <= 3 || (id >= 6 && id <= 39) || id == 41 || id == 42 || id == 43 || id == 142 || id == 143;
}

bool read_value(Reader& r, uint32_t type, MetaValue& v, int depth) {
    v.type = type;
    switch (type) {
        case 0: v.u = r.get<uint8_t>(); break;
        case 1: v.u = (uint64_t)(int64_t)r.get<int8_t>(); break;
        case 2: v.u = r.get<uint16_t>(); break;
        case 3: v.u = (uint64_t)(int64_t)r.get<int16_t>(); break;
        case 4: v.u = r.get<uint32_t>(); break;
        case 5: v.u = (uint64_t)(int64_t)r.get<int32_t>(); break;
        case 6: v.f = r.get<float>(); break;
        case 7: v.u = r.get<uint8_t>() != 0; break;
        case 8: v.s = r.str(); break;
        case 9: {
            if (depth > 4) return false;
            v.elem_type = r.get<uint32_t>();
            const uint64_t count = r.get<uint64_t>();
            if (!r.ok || count > r.n - r.pos) return false;  // every element takes at least one of the bytes that remain
            v.items.resize((size_t)count);
            for (auto& it : v.items)
                if (!read_value(r, v.elem_type, it, depth + 1)) return false;
            break;
        }
        case 10: v.u = r.get<uint64_t>(); break;
        case 11: v.u = (uint64_t)r.get<int64_t>(); break;
        case 12: v.f = r.get<double>(); break;
        default: v.type = 8; v.s = "<unknown_type_" + std::to_string(type) + ">"; break;  // gguf.rs:123
    }
    return r.ok;
}

size_t tensor_bytes(const TensorInfo& t) {
    uint64_t n = 1;
    for (uint64_t d : t.shape) {
        if (d != 0 && n > UINT64_MAX / d) return 0;
        n *= d;
    }
    if (t.dtype_id == 0) return (size_t)n * 4;                    // F32
    if (t.dtype_id == 1 || t.dtype_id == 30) return (size_t)n * 2;  // F16, BF16
    return hb200_byte_size((int)t.dtype_id, (size_t)n);           // formats of this path; 0 otherwise
}

const MetaValue* find_meta(hb200_gguf_t g, const char* key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" int hb200_gguf_close(hb200_gguf_t g) {
    if (!g) return HB200_OK;
    if (g->data) munmap(const_cast<uint8_t*>(g->data), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
    return HB200_OK;
}

extern "C" int hb200_gguf_open(const char* path, hb200_gguf_t* out) {
    hb200_gguf* g = nullptr;  // outside the try block: the catch path must close the file and the mapping too
    try {
        if (!path || !out) { set_error("null path or output handle"); return HB200_ERR_NULL; }
        g = new hb200_gguf();
        auto fail = [&](int code) { hb200_gguf_close(g); return code; };
        g->fd = open(path, O_RDONLY);
        if (g->fd < 0) { set_error("cannot open %s: %s", path, strerror(errno)); return fail(HB200_ERR_IO); }
        struct stat sb;
        if (fstat(g->fd, &sb) != 0) { set_error("cannot stat %s: %s", path, strerror(errno)); return fail(HB200_ERR_IO); }
        g->size = (size_t)sb.st_size;
        if (g->size < 4) { set_error("GGUF: file too small"); return fail(HB200_ERR_BAD_FORMAT); }
        void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
        if (m == MAP_FAILED) { set_error("cannot map %s: %s", path, strerror(errno)); return fail(HB200_ERR_IO); }
        g->data = static_cast<const uint8_t*>(m);
        if (memcmp(g->data, "GGUF", 4) != 0) { set_error("GGUF: invalid magic"); return fail(HB200_ERR_BAD_FORMAT); }
        Reader r{g->data, g->size, 4};
        g->version = r.get<uint32_t>();
        if (!r.ok || (g->version != 2 && g->version != 3)) { set_error("GGUF: unsupported version %u", g->version); return fail(HB200_ERR_BAD_FORMAT); }
        const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
        if (!r.ok || n_tensors > g->size || n_kv > g->size) { set_error("GGUF: unexpected end of file at offset %zu", r.pos); return fail(HB200_ERR_BAD_FORMAT); }
        for (uint64_t i = 0; i < n_kv; i++) {
            std::string key = r.str();
            const uint32_t type = r.get<uint32_t>();
            MetaValue v;
            if (!r.ok || !read_value(r, type, v, 0)) { set_error("GGUF: unexpected end of file at offset %zu", r.pos); return fail(HB200_ERR_BAD_FORMAT); }
            g->meta[key] = std::move(v);
        }
        if (const MetaValue* a = find_meta(g, "general.alignment"))
            if ((a->type == 4 || a->type == 5) && (uint32_t)a->u != 0) g->alignment = (uint32_t)a->u;
        g->tensors.reserve((size_t)n_tensors);
        for (uint64_t i = 0; i < n_tensors; i++) {
            TensorInfo t;
            t.name = r.str();
            const uint32_t n_dims = r.get<uint32_t>();
            if (!r.ok || n_dims > 8) { set_error("GGUF: bad tensor info at offset %zu", r.pos); return fail(HB200_ERR_BAD_FORMAT); }
            for (uint32_t k = 0; k < n_dims; k++) t.shape.push_back(r.get<uint64_t>());
            t.dtype_id = r.get<uint32_t>();
            t.offset = r.get<uint64_t>();
            if (!r.ok) { set_error("GGUF: unexpected end of file at offset %zu", r.pos); return fail(HB200_ERR_BAD_FORMAT); }
            if (!known_dtype(t.dtype_id)) { set_error("GGUF: unknown dtype id %u for tensor %s", t.dtype_id, t.name.c_str()); return fail(HB200_ERR_BAD_DTYPE); }
            g->tensors.push_back(std::move(t));
        }
        uint64_t pos = r.pos;
        if (g->version == 3) pos += (g->alignment - pos % g->alignment) % g->alignment;
        g->data_offset = pos;
        *out = g;
        return HB200_OK;
    } catch (...) {
        hb200_gguf_close(g);
        set_error("GGUF: out of memory or malformed file");
        return HB200_ERR_BAD_FORMAT;
    }
}

extern "C" size_t hb200_gguf_tensor_count(hb200_gguf_t g) { return g ? g->tensors.size() : 0; }
extern "C" uint32_t hb200_gguf_version(hb200_gguf_t g) { return g ? g->version : 0; }
extern "C" uint64_t hb200_gguf_data_offset(hb200_gguf_t g) { return g ? g->data_offset : 0; }

extern "C" int hb200_gguf_tensor_info(hb200_gguf_t g, size_t index, const char** name, int* dtype_id, size_t* n_dims,
                                      uint64_t shape[8], uint64_t* offset, size_t* bytes) {
    if (!g) { set_error("null GGUF handle"); return HB200_ERR_NULL; }
    if (index >= g->tensors.size()) { set_error("tensor index %zu of %zu", index, g->tensors.size()); return HB200_ERR_BAD_SHAPE; }
    const TensorInfo& t = g->tensors[index];
    if (name) *name = t.name.c_str();
    if (dtype_id) *dtype_id = (int)t.dtype_id;
    if (n_dims) *n_dims = t.shape.size();
    if (shape)
        for (size_t k = 0; k < 8; k++) shape[k] = k < t.shape.size() ? t.shape[k] : 0;
    if (offset) *offset = t.offset;
    if (bytes) *bytes = tensor_bytes(t);
    return HB200_OK;
}

extern "C" int hb200_gguf_find_tensor(hb200_gguf_t g, const char* name, size_t* index) {
    if (!g || !name || !index) { set_error("null argument"); return HB200_ERR_NULL; }
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) { *index = i; return HB200_OK; }
    set_error("no tensor named %s", name);
    return HB200_ERR_NOT_FOUND;
}

extern "C" int hb200_gguf_tensor_data(hb200_gguf_t g, size_t index, const uint8_t** data, size_t* bytes) {
    if (!g || !data || !bytes) { set_error("null argument"); return HB200_ERR_NULL; }
    if (index >= g->tensors.size()) { set_error("tensor index %zu of %zu", index, g->tensors.size()); return HB200_ERR_BAD_SHAPE; }
    const TensorInfo& t = g->tensors[index];
    const size_t nbytes = tensor_bytes(t);
    if (nbytes == 0) { set_error("tensor %s: type id %u has no size on this path", t.name.c_str(), t.dtype_id); return HB200_ERR_BAD_DTYPE; }
    const uint64_t start = g->data_offset + t.offset;
    if (start > g->size || nbytes > g->size - start) { set_error("tensor %s: data past the end of the file", t.name.c_str()); return HB200_ERR_BAD_FORMAT; }
    *data = g->data + start;
    *bytes = nbytes;
    return HB200_OK;
}

// TensorEntry::n_cols / n_rows (hearth-llm/src/model/tensor.rs:57-71): shape[0] columns, shape[1] rows (1 if absent).
extern "C" int hb200_gguf_upload_tensor(hb200_gguf_t g, size_t index, hb200_weight_t* out) {
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    int rc = hb200_gguf_tensor_data(g, index, &data, &bytes);
    if (rc) return rc;
    const TensorInfo& t = g->tensors[index];
    if (t.shape.empty() || t.shape.size() > 2) { set_error("tensor %s: %zu dimensions, a weight matrix has one or two", t.name.c_str(), t.shape.size()); return HB200_ERR_BAD_SHAPE; }
    const size_t n_cols = (size_t)t.shape[0], n_rows = t.shape.size() >= 2 ? (size_t)t.shape[1] : 1;
    return hb200_weight_upload((int)t.dtype_id, n_rows, n_cols, data, bytes, out);
}

extern "C" int hb200_gguf_meta_u64(hb200_gguf_t g, const char* key, uint64_t* out) {
    const MetaValue* v = find_meta(g, key);
    if (!v || !out) { set_error("no metadata key %s", key ? key : "(null)"); return HB200_ERR_NOT_FOUND; }
    switch (v->type) {
        case 0: case 1: case 2: case 3: case 4: case 5: case 7: case 10: case 11: *out = v->u; return HB200_OK;
        default: set_error("metadata %s is not an integer", key); return HB200_ERR_BAD_DTYPE;
    }
}

extern "C" int hb200_gguf_meta_f64(hb200_gguf_t g, const char* key, double* out) {
    const MetaValue* v = find_meta(g, key);
    if (!v || !out) { set_error("no metadata key %s", key ? key : "(null)"); return HB200_ERR_NOT_FOUND; }
    if (v->type != 6 && v->type != 12) { set_error("metadata %s is not a float", key); return HB200_ERR_BAD_DTYPE; }
    *out = v->f;
    return HB200_OK;
}

extern "C" int hb200_gguf_meta_str(hb200_gguf_t g, const char* key, const char** out, size_t* len) {
    const MetaValue* v = find_meta(g, key);
    if (!v || !out) { set_error("no metadata key %s", key ? key : "(null)"); return HB200_ERR_NOT_FOUND; }
    if (v->type != 8) { set_error("metadata %s is not a string", key); return HB200_ERR_BAD_DTYPE; }
    *out = v->s.c_str();
    if (len) *len = v->s.size();
    return HB200_OK;
}

// Numeric arrays as f32 (the per-width sign vectors of the Hadamard fold are stored this way,
// hearth-llm/src/model/qwen35.rs:544-600).  Call with out == null to get the count.
extern "C" int hb200_gguf_meta_array_f32(hb200_gguf_t g, const char* key, float* out, size_t capacity, size_t* count) {
    const MetaValue* v = find_meta(g, key);
    if (!v) { set_error("no metadata key %s", key ? key : "(null)"); return HB200_ERR_NOT_FOUND; }
    if (v->type != 9) { set_error("metadata %s is not an array", key); return HB200_ERR_BAD_DTYPE; }
    if (count) *count = v->items.size();
    if (!out) return HB200_OK;
    if (capacity < v->items.size()) { set_error("metadata %s has %zu elements, room for %zu", key, v->items.size(), capacity); return HB200_ERR_TOO_LARGE; }
    for (size_t i = 0; i < v->items.size(); i++) {
        const MetaValue& e = v->items[i];
        switch (e.type) {
            case 6: case 12: out[i] = (float)e.f; break;
            case 1: case 3: case 5: case 11: out[i] = (float)(int64_t)e.u; break;
            case 0: case 2: case 4: case 7: case 10: out[i] = (float)e.u; break;
            default: set_error("metadata %s: element %zu is not numeric", key, i); return HB200_ERR_BAD_DTYPE;
        }
    }
    return HB200_OK;
}
