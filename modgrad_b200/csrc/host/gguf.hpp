// GGUF v2 / v3 header parser: the host-side counterpart of the reference's
//   GgufFile::parse, GgmlType::block_size, TensorInfo, MetaValue
//   (crates/modgrad-device/src/kfd/gguf.rs:11-234, :665-694).
// Only the header is decoded (metadata key/values and tensor infos); tensor data stays in the
// memory-mapped file and is addressed by offset, as in the reference.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace mggguf {

// ggml tensor types by their numeric id (gguf.rs:13-31).
enum : uint32_t {
    kF32 = 0, kF16 = 1, kQ4_0 = 2, kQ4_1 = 3, kQ5_0 = 6, kQ5_1 = 7, kQ8_0 = 8, kQ8_1 = 9, kQ2_K = 10, kQ3_K = 11,
    kQ4_K = 12, kQ5_K = 13, kQ6_K = 14, kQ8_K = 15, kIQ2_XXS = 16, kBF16 = 30
};

// (bytes per block, elements per block); (0, 1) for a type the reference does not size (gguf.rs:48-67).
void block_size(uint32_t dtype, size_t* block_bytes, size_t* block_elems);
// Bytes of n_elements of `dtype` (gguf.rs:70-74).
size_t data_size(uint32_t dtype, size_t n_elements);

struct MetaValue {
    enum Kind { U8, I8, U16, I16, U32, I32, F32, Bool, Str, Array, U64, I64, F64 } kind = U8;
    uint64_t u = 0;   // unsigned kinds and Bool
    int64_t i = 0;    // signed kinds
    double f = 0.0;   // F32 / F64
    std::string s;
    std::vector<MetaValue> arr;
    // the reference's accessors (gguf.rs:116-146)
    bool as_u32(uint32_t* out) const;  // U32, I32 (cast), U64 (truncated)
    bool as_f32(float* out) const;     // F32, F64
    const std::string* as_str() const;
};

struct TensorInfo {
    std::string name;
    std::vector<size_t> dims;  // dims[0] = in_dim (fastest), dims[1] = out_dim for a matrix
    uint32_t dtype = 0;
    size_t offset = 0;  // from the start of the data section
    size_t n_elements() const;
    size_t data_bytes() const;
};

struct File {
    uint32_t version = 0;
    std::map<std::string, MetaValue> metadata;
    std::map<std::string, TensorInfo> tensors;
    std::vector<std::string> tensor_list;  // file order
    size_t data_offset = 0;                // absolute offset of the data section (32-byte aligned)

    // Parses the header found in [data, data + bytes).  false + message on malformed input; every read
    // is bounds-checked.
    static bool parse(const uint8_t* data, size_t bytes, File* out, std::string* err);
    const MetaValue* meta(const std::string& key) const;
    const std::string* architecture() const;  // "general.architecture"
    bool meta_u32(const std::string& key, uint32_t* out) const;
    bool meta_f32(const std::string& key, float* out) const;
    const TensorInfo* tensor(const std::string& name) const;
};

}  // namespace mggguf
