// See gguf.hpp.  Parser, and the C ABI around it (mg_gguf_*): open a file (memory-mapped, read-only),
// look up metadata and tensor infos, get a pointer to a tensor's bytes.
#include "gguf.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

#include "modgrad_cuda.h"

namespace mggguf {

void block_size(uint32_t dtype, size_t* bb, size_t* be) {
    size_t b = 0, e = 1;
    switch (dtype) {
        case kF32: b = 4; e = 1; break;
        case kF16: b = 2; e = 1; break;
        case kBF16: b = 2; e = 1; break;
        case kQ4_0: b = 18; e = 32; break;
        case kQ4_1: b = 20; e = 32; break;
        case kQ5_0: b = 22; e = 32; break;
        case kQ5_1: b = 24; e = 32; break;
        case kQ8_0: b = 34; e = 32; break;
        case kQ8_1: b = 36; e = 32; break;
        case kQ2_K: b = 84; e = 256; break;
        case kQ3_K: b = 110; e = 256; break;
        case kQ4_K: b = 144; e = 256; break;
        case kQ5_K: b = 176; e = 256; break;
        case kQ6_K: b = 210; e = 256; break;
        case kQ8_K: b = 292; e = 256; break;
        default: break;
    }
    *bb = b;
    *be = e;
}

size_t data_size(uint32_t dtype, size_t n_elements) {
    size_t bb, be;
    block_size(dtype, &bb, &be);
    return (n_elements + be - 1) / be * bb;
}

bool MetaValue::as_u32(uint32_t* out) const {
    switch (kind) {
        case U32: *out = (uint32_t)u; return true;
        case I32: *out = (uint32_t)i; return true;
        case U64: *out = (uint32_t)u; return true;
        default: return false;
    }
}
bool MetaValue::as_f32(float* out) const {
    if (kind == F32 || kind == F64) {
        *out = (float)f;
        return true;
    }
    return false;
}
const std::string* MetaValue::as_str() const { return kind == Str ? &s : nullptr; }

size_t TensorInfo::n_elements() const {
    size_t n = 1;
    for (size_t d : dims) n *= d;
    return n > 0 ? n : 1;
}
size_t TensorInfo::data_bytes() const { return data_size(dtype, n_elements()); }

namespace {

struct Cursor {
    const uint8_t* p;
    size_t n, pos = 0;
    std::string* err;
    bool take(void* dst, size_t k) {
        if (k > n - pos) {
            *err = "failed to fill whole buffer";  // what read_exact reports at end of file
            return false;
        }
        memcpy(dst, p + pos, k);
        pos += k;
        return true;
    }
    template <class T>
    bool get(T* v) { return take(v, sizeof(T)); }  // the host is little-endian, like the format
};

bool read_string(Cursor& c, std::string* out) {
    uint64_t len = 0;
    if (!c.get(&len)) return false;
    if (len > 1000000) {
        *c.err = "string too long";
        return false;
    }
    out->resize((size_t)len);
    return len == 0 || c.take(&(*out)[0], (size_t)len);
}

bool read_typed(Cursor& c, uint32_t vtype, MetaValue* out, int depth) {
    switch (vtype) {
        case 0: { uint8_t v; if (!c.get(&v)) return false; out->kind = MetaValue::U8; out->u = v; return true; }
        case 1: { int8_t v; if (!c.get(&v)) return false; out->kind = MetaValue::I8; out->i = v; return true; }
        case 2: { uint16_t v; if (!c.get(&v)) return false; out->kind = MetaValue::U16; out->u = v; return true; }
        case 3: { int16_t v; if (!c.get(&v)) return false; out->kind = MetaValue::I16; out->i = v; return true; }
        case 4: { uint32_t v; if (!c.get(&v)) return false; out->kind = MetaValue::U32; out->u = v; return true; }
        case 5: { int32_t v; if (!c.get(&v)) return false; out->kind = MetaValue::I32; out->i = v; return true; }
        case 6: { float v; if (!c.get(&v)) return false; out->kind = MetaValue::F32; out->f = v; return true; }
        case 7: { uint8_t v; if (!c.get(&v)) return false; out->kind = MetaValue::Bool; out->u = v != 0; return true; }
        case 8: out->kind = MetaValue::Str; return read_string(c, &out->s);
        case 9: {
            uint32_t atype = 0;
            uint64_t alen = 0;
            if (!c.get(&atype) || !c.get(&alen)) return false;
            if (depth > 8) {
                *c.err = "array nesting too deep";
                return false;
            }
            out->kind = MetaValue::Array;
            out->arr.reserve((size_t)(alen < 1024 ? alen : 1024));
            for (uint64_t k = 0; k < alen; ++k) {
                MetaValue v;
                if (!read_typed(c, atype, &v, depth + 1)) return false;
                out->arr.push_back(std::move(v));
            }
            return true;
        }
        case 10: { uint64_t v; if (!c.get(&v)) return false; out->kind = MetaValue::U64; out->u = v; return true; }
        case 11: { int64_t v; if (!c.get(&v)) return false; out->kind = MetaValue::I64; out->i = v; return true; }
        case 12: { double v; if (!c.get(&v)) return false; out->kind = MetaValue::F64; out->f = v; return true; }
        default:
            *c.err = "unknown GGUF value type " + std::to_string(vtype);
            return false;
    }
}

}  // namespace

bool File::parse(const uint8_t* data, size_t bytes, File* out, std::string* err) {
    Cursor c{data, bytes, 0, err};
    char magic[4];
    if (!c.take(magic, 4)) return false;
    if (memcmp(magic, "GGUF", 4) != 0) {
        *err = "not a GGUF file";
        return false;
    }
    uint32_t version = 0;
    if (!c.get(&version)) return false;
    if (version < 2 || version > 3) {
        *err = "unsupported GGUF version " + std::to_string(version);
        return false;
    }
    uint64_t n_tensors = 0, n_kv = 0;
    if (!c.get(&n_tensors) || !c.get(&n_kv)) return false;
    File f;
    f.version = version;
    for (uint64_t k = 0; k < n_kv; ++k) {
        std::string key;
        uint32_t vtype = 0;
        MetaValue v;
        if (!read_string(c, &key) || !c.get(&vtype) || !read_typed(c, vtype, &v, 0)) return false;
        f.metadata[key] = std::move(v);
    }
    for (uint64_t k = 0; k < n_tensors; ++k) {
        TensorInfo t;
        uint32_t n_dims = 0;
        if (!read_string(c, &t.name) || !c.get(&n_dims)) return false;
        if (n_dims > 8) {
            *err = "tensor " + t.name + ": too many dimensions";
            return false;
        }
        for (uint32_t d = 0; d < n_dims; ++d) {
            uint64_t v = 0;
            if (!c.get(&v)) return false;
            t.dims.push_back((size_t)v);
        }
        uint64_t off = 0;
        if (!c.get(&t.dtype) || !c.get(&off)) return false;
        t.offset = (size_t)off;
        f.tensor_list.push_back(t.name);
        f.tensors[t.name] = std::move(t);
    }
    f.data_offset = (c.pos + 31) & ~(size_t)31;  // the data section starts 32-byte aligned
    *out = std::move(f);
    return true;
}

const MetaValue* File::meta(const std::string& key) const {
    auto it = metadata.find(key);
    return it == metadata.end() ? nullptr : &it->second;
}
const std::string* File::architecture() const {
    const MetaValue* v = meta("general.architecture");
    return v ? v->as_str() : nullptr;
}
bool File::meta_u32(const std::string& key, uint32_t* out) const {
    const MetaValue* v = meta(key);
    return v && v->as_u32(out);
}
bool File::meta_f32(const std::string& key, float* out) const {
    const MetaValue* v = meta(key);
    return v && v->as_f32(out);
}
const TensorInfo* File::tensor(const std::string& name) const {
    auto it = tensors.find(name);
    return it == tensors.end() ? nullptr : &it->second;
}

}  // namespace mggguf

// ---- C ABI ----------------------------------------------------------------------------------------
struct mg_gguf {
    mggguf::File file;
    const uint8_t* data = nullptr;  // the whole file
    size_t bytes = 0;
    bool mapped = false;
};

namespace {
thread_local std::string g_gguf_error;
}

extern "C" {

const char* mg_gguf_last_error(void) { return g_gguf_error.c_str(); }

// Parses a GGUF image already in memory (the caller keeps it alive); 0, or -4 (Runtime) with
// mg_gguf_last_error().
int mg_gguf_parse_memory(const void* data, size_t bytes, mg_gguf** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!data) {
        g_gguf_error = "null buffer";
        return -4;
    }
    mg_gguf* g = new mg_gguf();
    if (!mggguf::File::parse(static_cast<const uint8_t*>(data), bytes, &g->file, &g_gguf_error)) {
        delete g;
        return -4;
    }
    g->data = static_cast<const uint8_t*>(data);
    g->bytes = bytes;
    *out = g;
    return 0;
}

// Opens and memory-maps `path` read-only (tensor bytes cost no resident memory until touched,
// as in the reference) and parses its header.
int mg_gguf_open(const char* path, mg_gguf** out) {
    if (!out) return -4;
    *out = nullptr;
    if (!path) {
        g_gguf_error = "null path";
        return -4;
    }
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        g_gguf_error = std::string("cannot open ") + path + ": " + strerror(errno);
        return -4;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        g_gguf_error = std::string("cannot stat ") + path;
        close(fd);
        return -4;
    }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) {
        g_gguf_error = std::string("cannot map ") + path + ": " + strerror(errno);
        return -4;
    }
    const int rc = mg_gguf_parse_memory(p, (size_t)st.st_size, out);
    if (rc) {
        munmap(p, (size_t)st.st_size);
        return rc;
    }
    (*out)->mapped = true;
    return 0;
}

void mg_gguf_close(mg_gguf* g) {
    if (!g) return;
    if (g->mapped) munmap(const_cast<uint8_t*>(g->data), g->bytes);
    delete g;
}

int mg_gguf_version(const mg_gguf* g) { return g ? (int)g->file.version : 0; }
size_t mg_gguf_data_offset(const mg_gguf* g) { return g ? g->file.data_offset : 0; }
int mg_gguf_n_tensors(const mg_gguf* g) { return g ? (int)g->file.tensor_list.size() : 0; }
int mg_gguf_n_meta(const mg_gguf* g) { return g ? (int)g->file.metadata.size() : 0; }

// Index of tensor `name` in file order, or -1.
int mg_gguf_find_tensor(const mg_gguf* g, const char* name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->file.tensor_list.size(); ++i)
        if (g->file.tensor_list[i] == name) return (int)i;
    return -1;
}

// Tensor `index` in file order: name, dims (up to 4 returned, n_dims the real count), dtype id,
// absolute file offset of its data and its size in bytes.  0, or -4 for a bad index.
int mg_gguf_tensor(const mg_gguf* g, int index, const char** name, int* n_dims, uint64_t* dims4, uint32_t* dtype,
                   uint64_t* file_offset, uint64_t* data_bytes) {
    if (!g || index < 0 || index >= (int)g->file.tensor_list.size()) return -4;
    const mggguf::TensorInfo& t = g->file.tensors.at(g->file.tensor_list[index]);
    if (name) *name = t.name.c_str();
    if (n_dims) *n_dims = (int)t.dims.size();
    if (dims4)
        for (int d = 0; d < 4; ++d) dims4[d] = d < (int)t.dims.size() ? t.dims[d] : 1;
    if (dtype) *dtype = t.dtype;
    if (file_offset) *file_offset = g->file.data_offset + t.offset;
    if (data_bytes) *data_bytes = t.data_bytes();
    return 0;
}

// Pointer to the tensor's bytes inside the mapped file, NULL when the tensor runs past the end.
const void* mg_gguf_tensor_data(const mg_gguf* g, int index) {
    if (!g || index < 0 || index >= (int)g->file.tensor_list.size()) return nullptr;
    const mggguf::TensorInfo& t = g->file.tensors.at(g->file.tensor_list[index]);
    const size_t start = g->file.data_offset + t.offset, n = t.data_bytes();
    if (start > g->bytes || n > g->bytes - start) return nullptr;
    return g->data + start;
}

// Metadata lookups with the reference's conversions (gguf.rs:116-146): 0 found, -1 absent or of
// another kind.
int mg_gguf_meta_u32(const mg_gguf* g, const char* key, uint32_t* out) {
    return g && key && out && g->file.meta_u32(key, out) ? 0 : -1;
}
int mg_gguf_meta_f32(const mg_gguf* g, const char* key, float* out) {
    return g && key && out && g->file.meta_f32(key, out) ? 0 : -1;
}
const char* mg_gguf_meta_str(const mg_gguf* g, const char* key) {
    if (!g || !key) return nullptr;
    const mggguf::MetaValue* v = g->file.meta(key);
    const std::string* s = v ? v->as_str() : nullptr;
    return s ? s->c_str() : nullptr;
}
// Length of an array-valued key (-1 when absent or not an array).
long long mg_gguf_meta_array_len(const mg_gguf* g, const char* key) {
    if (!g || !key) return -1;
    const mggguf::MetaValue* v = g->file.meta(key);
    return v && v->kind == mggguf::MetaValue::Array ? (long long)v->arr.size() : -1;
}
// Bytes / elements per block of a ggml type id (0 bytes for a type the reference does not size).
void mg_gguf_block_size(uint32_t dtype, size_t* block_bytes, size_t* block_elems) {
    size_t b, e;
    mggguf::block_size(dtype, &b, &e);
    if (block_bytes) *block_bytes = b;
    if (block_elems) *block_elems = e;
}

}  // extern "C"

// For the decoder loader (decoder_gguf.cpp).
const mggguf::File& mg_gguf_file(const mg_gguf* g) { return g->file; }
const uint8_t* mg_gguf_bytes(const mg_gguf* g, size_t* n) {
    *n = g->bytes;
    return g->data;
}
