// GGUF container reader (host only): header, metadata, tensor directory over a read-only memory map.
// Follows the file walk of the reference's loader (src/load_gguf.jl:54-133, 317-336): magic "GGUF", version,
// tensor count, metadata key/values, tensor infos, then tensor data from the next multiple of general.alignment.
// Unlike the reference (which reads six metadata value types, src/load_gguf.jl:59-77) every value type of the
// format is walked, so files with 64-bit or float64 metadata load too.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace l2b {

struct GgufValue {
    uint32_t type = 0;       // GGUF_METADATA_VALUE_TYPE (src/load_gguf.jl:1-24)
    double num = 0.0;        // scalars (integers, floats, bool)
    int64_t inum = 0;        // the same as an integer, for integer types
    std::string str;         // type 8
    uint32_t elem_type = 0;  // arrays: element type and count; the elements stay in the file map
    uint64_t count = 0;
    const uint8_t* elems = nullptr;  // arrays: first byte of the elements inside the map (bounds already checked)
    uint64_t elems_bytes = 0;        // arrays: bytes the elements occupy
};

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> dims;  // dims[0] is the contiguous (input) dimension
    uint32_t type = 0;           // GGML_TYPE (src/load_gguf.jl:26-42)
    const uint8_t* data = nullptr;
    uint64_t nbytes = 0;         // 0 when the type is not one the decode path supports
    uint64_t rows() const {      // product of the dimensions after the first
        uint64_t r = 1;
        for (size_t i = 1; i < dims.size(); ++i) r *= dims[i];
        return r;
    }
};

class GgufFile {
public:
    GgufFile() = default;
    ~GgufFile();
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;
    // Returns false and sets error() on anything that is not a well-formed GGUF file.
    bool open(const char* path);
    const std::string& error() const { return err_; }
    const GgufValue* find(const std::string& key) const;
    const GgufTensor* tensor(const std::string& name) const;
    const std::vector<GgufTensor>& tensors() const { return tensors_; }
    uint32_t version() const { return version_; }

private:
    int fd_ = -1;
    const uint8_t* base_ = nullptr;
    size_t size_ = 0;
    uint32_t version_ = 0;
    std::map<std::string, GgufValue> kv_;
    std::vector<GgufTensor> tensors_;
    std::map<std::string, size_t> index_;
    std::string err_;
};

}  // namespace l2b
