// GGUF reader: header, metadata and tensor directory of a GGUF v2/v3 file, mapped read-only.
// The kernels multiply Q8_0 / Q4_K blocks exactly as they sit in the file, so loading a weight is
// "find the tensor, copy its bytes to the device": no repacked copy exists.
// Stands where the reference uses Candle's gguf_file::Content behind GgufLoader
// (crates/izwi-core/src/models/shared/weights/gguf.rs:36-143).
// Every length and offset read from the file is checked against the mapping before it is used.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/izwi_b200.h"

namespace {

enum GgufValueType : uint32_t {
    GV_U8 = 0, GV_I8 = 1, GV_U16 = 2, GV_I16 = 3, GV_U32 = 4, GV_I32 = 5, GV_F32 = 6, GV_BOOL = 7,
    GV_STRING = 8, GV_ARRAY = 9, GV_U64 = 10, GV_I64 = 11, GV_F64 = 12,
};

struct TypeTraits {
    int64_t block;  // values per block
    int64_t bytes;  // bytes per block
    int32_t wfmt;   // izb_wfmt the kernels accept for these bytes, or -1
};

// GGML tensor types by their on-disk id (the public ggml.h enumeration).
bool ggml_type_traits(uint32_t t, TypeTraits* out) {
    switch (t) {
        case 0: *out = {1, 4, -1}; return true;             // F32
        case 1: *out = {1, 2, -1}; return true;             // F16
        case 2: *out = {32, 18, -1}; return true;           // Q4_0
        case 3: *out = {32, 20, -1}; return true;           // Q4_1
        case 6: *out = {32, 22, -1}; return true;           // Q5_0
        case 7: *out = {32, 24, -1}; return true;           // Q5_1
        case 8: *out = {32, 34, IZB_W_Q8_0}; return true;   // Q8_0
        case 9: *out = {32, 36, -1}; return true;           // Q8_1
        case 10: *out = {256, 84, -1}; return true;         // Q2_K
        case 11: *out = {256, 110, -1}; return true;        // Q3_K
        case 12: *out = {256, 144, IZB_W_Q4_K}; return true;  // Q4_K
        case 13: *out = {256, 176, -1}; return true;        // Q5_K
        case 14: *out = {256, 210, IZB_W_Q6_K}; return true;  // Q6_K
        case 15: *out = {256, 292, -1}; return true;        // Q8_K
        case 24: *out = {1, 1, -1}; return true;            // I8
        case 25: *out = {1, 2, -1}; return true;            // I16
        case 26: *out = {1, 4, -1}; return true;            // I32
        case 27: *out = {1, 8, -1}; return true;            // I64
        case 28: *out = {1, 8, -1}; return true;            // F64
        case 30: *out = {1, 2, IZB_W_BF16}; return true;    // BF16
        default: return false;
    }
}

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0;      // integers and bool
    double f = 0.0;      // floats
    const char* s = nullptr;  // strings: pointer into the mapping (not NUL-terminated)
    uint64_t s_len = 0;
    uint32_t elem_type = 0;  // arrays
    uint64_t count = 0;
};

struct TensorEntry {
    std::string name;
    uint32_t ggml_type = 0;
    int32_t n_dims = 0;
    int64_t dims[4] = {1, 1, 1, 1};  // outermost first (row-major), as Candle reports shapes
    uint64_t offset = 0;             // from the start of the data section
    uint64_t bytes = 0;
    TypeTraits traits{};
};

class Cursor {
  public:
    Cursor(const uint8_t* base, uint64_t size) : base_(base), size_(size) {}
    bool read(void* dst, uint64_t n) {
        if (n > size_ - pos_) return false;
        std::memcpy(dst, base_ + pos_, n);
        pos_ += n;
        return true;
    }
    template <typename T>
    bool get(T* v) { return read(v, sizeof(T)); }
    bool skip(uint64_t n) {
        if (n > size_ - pos_) return false;
        pos_ += n;
        return true;
    }
    bool str(const char** p, uint64_t* len) {
        uint64_t n;
        if (!get(&n) || n > size_ - pos_) return false;
        *p = reinterpret_cast<const char*>(base_ + pos_);
        *len = n;
        pos_ += n;
        return true;
    }
    uint64_t pos() const { return pos_; }

  private:
    const uint8_t* base_;
    uint64_t size_, pos_ = 0;
};

uint64_t scalar_size(uint32_t t) {
    switch (t) {
        case GV_U8: case GV_I8: case GV_BOOL: return 1;
        case GV_U16: case GV_I16: return 2;
        case GV_U32: case GV_I32: case GV_F32: return 4;
        case GV_U64: case GV_I64: case GV_F64: return 8;
        default: return 0;
    }
}

bool read_scalar(Cursor& c, uint32_t t, MetaValue* v) {
    v->type = t;
    switch (t) {
        case GV_U8: { uint8_t x; if (!c.get(&x)) return false; v->u = x; v->f = x; return true; }
        case GV_I8: { int8_t x; if (!c.get(&x)) return false; v->u = static_cast<uint64_t>(static_cast<int64_t>(x)); v->f = x; return true; }
        case GV_U16: { uint16_t x; if (!c.get(&x)) return false; v->u = x; v->f = x; return true; }
        case GV_I16: { int16_t x; if (!c.get(&x)) return false; v->u = static_cast<uint64_t>(static_cast<int64_t>(x)); v->f = x; return true; }
        case GV_U32: { uint32_t x; if (!c.get(&x)) return false; v->u = x; v->f = x; return true; }
        case GV_I32: { int32_t x; if (!c.get(&x)) return false; v->u = static_cast<uint64_t>(static_cast<int64_t>(x)); v->f = x; return true; }
        case GV_U64: { uint64_t x; if (!c.get(&x)) return false; v->u = x; v->f = static_cast<double>(x); return true; }
        case GV_I64: { int64_t x; if (!c.get(&x)) return false; v->u = static_cast<uint64_t>(x); v->f = static_cast<double>(x); return true; }
        case GV_F32: { float x; if (!c.get(&x)) return false; v->f = x; v->u = static_cast<uint64_t>(x); return true; }
        case GV_F64: { double x; if (!c.get(&x)) return false; v->f = x; v->u = static_cast<uint64_t>(x); return true; }
        case GV_BOOL: { uint8_t x; if (!c.get(&x)) return false; v->u = x != 0; v->f = static_cast<double>(v->u); return true; }
        default: return false;
    }
}

bool read_value(Cursor& c, uint32_t t, MetaValue* v, int depth) {
    if (t == GV_STRING) {
        v->type = t;
        return c.str(&v->s, &v->s_len);
    }
    if (t == GV_ARRAY) {
        if (depth > 2) return false;
        v->type = t;
        if (!c.get(&v->elem_type) || !c.get(&v->count)) return false;
        const uint64_t es = scalar_size(v->elem_type);
        if (es) return v->count <= UINT64_MAX / es && c.skip(v->count * es);
        for (uint64_t i = 0; i < v->count; ++i) {  // strings or nested arrays: walk them
            MetaValue tmp;
            if (!read_value(c, v->elem_type, &tmp, depth + 1)) return false;
        }
        return true;
    }
    return read_scalar(c, t, v);
}

}  // namespace

struct izb_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    uint64_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32;
    uint64_t data_start = 0;
    std::vector<TensorEntry> tensors;
    std::unordered_map<std::string, size_t> by_name;
    std::unordered_map<std::string, MetaValue> meta;
    std::vector<std::string> meta_keys;
};

namespace {

int32_t parse(izb_gguf* g) {
    Cursor c(g->map, g->size);
    uint32_t magic;
    if (!c.get(&magic) || magic != 0x46554747u) return IZB_ERR_BAD_ARG;  // "GGUF"
    if (!c.get(&g->version) || g->version < 2 || g->version > 3) return IZB_ERR_UNSUPPORTED;
    uint64_t n_tensors, n_kv;
    if (!c.get(&n_tensors) || !c.get(&n_kv)) return IZB_ERR_BAD_ARG;
    if (n_tensors > g->size / 24 || n_kv > g->size / 12) return IZB_ERR_BAD_ARG;  // cannot fit in the file
    for (uint64_t i = 0; i < n_kv; ++i) {
        const char* k;
        uint64_t klen;
        uint32_t t;
        MetaValue v;
        if (!c.str(&k, &klen) || !c.get(&t) || !read_value(c, t, &v, 0)) return IZB_ERR_BAD_ARG;
        std::string key(k, klen);
        if (g->meta.emplace(key, v).second) g->meta_keys.push_back(key);
    }
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end() && al->second.type != GV_STRING && al->second.type != GV_ARRAY) {
        g->alignment = al->second.u;
        if (g->alignment == 0 || (g->alignment & (g->alignment - 1)) != 0 || g->alignment > (1u << 20)) return IZB_ERR_BAD_ARG;
    }
    g->tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        TensorEntry e;
        const char* nm;
        uint64_t nlen;
        uint32_t nd;
        if (!c.str(&nm, &nlen) || !c.get(&nd) || nd == 0 || nd > 4) return IZB_ERR_BAD_ARG;
        e.name.assign(nm, nlen);
        e.n_dims = static_cast<int32_t>(nd);
        uint64_t ne[4] = {1, 1, 1, 1};
        uint64_t elems = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            if (!c.get(&ne[d]) || ne[d] == 0 || ne[d] > static_cast<uint64_t>(INT64_MAX)) return IZB_ERR_BAD_ARG;
            if (elems > static_cast<uint64_t>(INT64_MAX) / ne[d]) return IZB_ERR_BAD_ARG;
            elems *= ne[d];
        }
        for (uint32_t d = 0; d < nd; ++d) e.dims[d] = static_cast<int64_t>(ne[nd - 1 - d]);  // file order is innermost first
        if (!c.get(&e.ggml_type) || !c.get(&e.offset)) return IZB_ERR_BAD_ARG;
        if (!ggml_type_traits(e.ggml_type, &e.traits)) return IZB_ERR_UNSUPPORTED;
        if (ne[0] % static_cast<uint64_t>(e.traits.block) != 0) return IZB_ERR_BAD_ARG;  // rows hold whole blocks
        e.bytes = elems / static_cast<uint64_t>(e.traits.block) * static_cast<uint64_t>(e.traits.bytes);
        if (e.offset % g->alignment != 0) return IZB_ERR_BAD_ARG;
        if (!g->by_name.emplace(e.name, g->tensors.size()).second) return IZB_ERR_BAD_ARG;  // duplicate name
        g->tensors.push_back(std::move(e));
    }
    g->data_start = (c.pos() + g->alignment - 1) / g->alignment * g->alignment;
    if (g->data_start > g->size && n_tensors > 0) return IZB_ERR_BAD_ARG;
    for (const TensorEntry& e : g->tensors) {
        const uint64_t room = g->size - g->data_start;
        if (e.offset > room || e.bytes > room - e.offset) return IZB_ERR_BAD_ARG;  // data past the end of the file
    }
    return IZB_OK;
}

void fill(const izb_gguf* g, const TensorEntry& e, izb_gguf_tensor* out) {
    out->name = e.name.c_str();
    out->ggml_type = static_cast<int32_t>(e.ggml_type);
    out->wfmt = e.traits.wfmt;
    out->n_dims = e.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = e.dims[d];
    out->cols = e.dims[e.n_dims - 1];
    int64_t rows = 1;
    for (int d = 0; d < e.n_dims - 1; ++d) rows *= e.dims[d];
    out->rows = rows;
    out->data = g->map + g->data_start + e.offset;
    out->bytes = static_cast<size_t>(e.bytes);
}

const MetaValue* find_meta(const izb_gguf* g, const char* key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

int32_t izb_gguf_open(const char* path, izb_gguf** out) {
    if (!path || !out) return IZB_ERR_BAD_ARG;
    *out = nullptr;
    izb_gguf* g = new (std::nothrow) izb_gguf();
    if (!g) return IZB_ERR_LAUNCH;
    g->fd = ::open(path, O_RDONLY | O_CLOEXEC);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        if (g->fd >= 0) ::close(g->fd);
        delete g;
        return IZB_ERR_BAD_ARG;
    }
    g->size = static_cast<uint64_t>(st.st_size);
    void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        ::close(g->fd);
        delete g;
        return IZB_ERR_LAUNCH;
    }
    g->map = static_cast<const uint8_t*>(m);
    const int32_t rc = parse(g);
    if (rc != IZB_OK) {
        izb_gguf_close(g);
        return rc;
    }
    *out = g;
    return IZB_OK;
}

int32_t izb_gguf_close(izb_gguf* g) {
    if (!g) return IZB_ERR_BAD_ARG;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) ::close(g->fd);
    delete g;
    return IZB_OK;
}

int32_t izb_gguf_version(const izb_gguf* g) { return g ? static_cast<int32_t>(g->version) : 0; }
int64_t izb_gguf_tensor_count(const izb_gguf* g) { return g ? static_cast<int64_t>(g->tensors.size()) : 0; }
int64_t izb_gguf_meta_count(const izb_gguf* g) { return g ? static_cast<int64_t>(g->meta_keys.size()) : 0; }

const char* izb_gguf_meta_key(const izb_gguf* g, int64_t index) {
    if (!g || index < 0 || index >= static_cast<int64_t>(g->meta_keys.size())) return nullptr;
    return g->meta_keys[static_cast<size_t>(index)].c_str();
}

int32_t izb_gguf_tensor_at(const izb_gguf* g, int64_t index, izb_gguf_tensor* out) {
    if (!g || !out || index < 0 || index >= static_cast<int64_t>(g->tensors.size())) return IZB_ERR_BAD_ARG;
    fill(g, g->tensors[static_cast<size_t>(index)], out);
    return IZB_OK;
}

int32_t izb_gguf_find(const izb_gguf* g, const char* name, izb_gguf_tensor* out) {
    if (!g || !name || !out) return IZB_ERR_BAD_ARG;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return IZB_ERR_UNSUPPORTED;
    fill(g, g->tensors[it->second], out);
    return IZB_OK;
}

int32_t izb_gguf_meta_u64(const izb_gguf* g, const char* key, uint64_t* out) {
    const MetaValue* v = find_meta(g, key);
    if (!out) return IZB_ERR_BAD_ARG;
    if (!v) return IZB_ERR_UNSUPPORTED;
    if (v->type == GV_STRING || v->type == GV_ARRAY || v->type == GV_F32 || v->type == GV_F64) return IZB_ERR_BAD_ARG;
    *out = v->u;
    return IZB_OK;
}

int32_t izb_gguf_meta_f64(const izb_gguf* g, const char* key, double* out) {
    const MetaValue* v = find_meta(g, key);
    if (!out) return IZB_ERR_BAD_ARG;
    if (!v) return IZB_ERR_UNSUPPORTED;
    if (v->type == GV_STRING || v->type == GV_ARRAY) return IZB_ERR_BAD_ARG;
    *out = v->f;
    return IZB_OK;
}

int32_t izb_gguf_meta_str(const izb_gguf* g, const char* key, const char** out, size_t* len) {
    const MetaValue* v = find_meta(g, key);
    if (!out || !len) return IZB_ERR_BAD_ARG;
    if (!v) return IZB_ERR_UNSUPPORTED;
    if (v->type != GV_STRING) return IZB_ERR_BAD_ARG;
    *out = v->s;
    *len = static_cast<size_t>(v->s_len);
    return IZB_OK;
}

int32_t izb_gguf_upload(const izb_gguf* g, const izb_gguf_tensor* t, void* dev_dst, size_t dst_bytes, izb_stream stream) {
    if (!g || !t || !t->data) return IZB_ERR_BAD_ARG;
    const uint8_t* p = static_cast<const uint8_t*>(t->data);
    if (p < g->map + g->data_start || t->bytes > g->size || p + t->bytes > g->map + g->size) return IZB_ERR_BAD_ARG;
    if (t->bytes == 0) return IZB_OK;
    if (!dev_dst || dst_bytes < t->bytes) return IZB_ERR_BAD_ARG;
    // pageable source: the runtime stages it; the call returns once the source has been read
    if (cudaMemcpyAsync(dev_dst, p, t->bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        return IZB_ERR_LAUNCH;
    }
    return IZB_OK;
}

}  // extern "C"
