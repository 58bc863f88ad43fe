#include "gguf_reader.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

namespace l2b {

namespace {

// Bounds-checked cursor over the mapped file.
struct Cursor {
    const uint8_t* base;
    size_t size, pos;
    bool ok = true;
    template <typename T>
    T take() {
        T v{};
        if (!ok || size - pos < sizeof(T) || pos > size) {
            ok = false;
            return v;
        }
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    bool skip(uint64_t n) {
        if (!ok || n > size - pos) {
            ok = false;
            return false;
        }
        pos += (size_t)n;
        return true;
    }
    std::string string() {  // gguf_string_t: u64 length + bytes (src/load_gguf.jl:54-57)
        const uint64_t n = take<uint64_t>();
        if (!ok || n > size - pos) {
            ok = false;
            return std::string();
        }
        std::string s(reinterpret_cast<const char*>(base + pos), (size_t)n);
        pos += (size_t)n;
        return s;
    }
};

int scalar_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;   // u8, i8, bool
        case 2: case 3: return 2;           // u16, i16
        case 4: case 5: case 6: return 4;   // u32, i32, f32
        case 10: case 11: case 12: return 8;  // u64, i64, f64
        default: return 0;
    }
}

bool read_value(Cursor& c, uint32_t type, GgufValue& v, int depth) {
    v.type = type;
    switch (type) {
        case 0: v.inum = c.take<uint8_t>(); v.num = (double)v.inum; break;
        case 1: v.inum = c.take<int8_t>(); v.num = (double)v.inum; break;
        case 2: v.inum = c.take<uint16_t>(); v.num = (double)v.inum; break;
        case 3: v.inum = c.take<int16_t>(); v.num = (double)v.inum; break;
        case 4: v.inum = c.take<uint32_t>(); v.num = (double)v.inum; break;
        case 5: v.inum = c.take<int32_t>(); v.num = (double)v.inum; break;
        case 6: v.num = c.take<float>(); v.inum = (int64_t)v.num; break;
        case 7: v.inum = c.take<uint8_t>() != 0; v.num = (double)v.inum; break;
        case 8: v.str = c.string(); break;
        case 10: v.inum = (int64_t)c.take<uint64_t>(); v.num = (double)v.inum; break;
        case 11: v.inum = c.take<int64_t>(); v.num = (double)v.inum; break;
        case 12: v.num = c.take<double>(); v.inum = (int64_t)v.num; break;
        case 9: {  // array: element type, count, elements (walked and bounds-checked; they stay in the map)
            v.elem_type = c.take<uint32_t>();
            v.count = c.take<uint64_t>();
            if (!c.ok) return false;
            const size_t elems_at = c.pos;
            const int es = scalar_size(v.elem_type);
            if (es > 0) {
                if (v.count > (c.size - c.pos) / (uint64_t)es) return c.ok = false;
                c.skip(v.count * (uint64_t)es);
            } else if (v.elem_type == 8) {
                for (uint64_t i = 0; i < v.count && c.ok; ++i) {
                    const uint64_t n = c.take<uint64_t>();
                    c.skip(n);
                }
            } else if (v.elem_type == 9 && depth < 4) {
                for (uint64_t i = 0; i < v.count && c.ok; ++i) {
                    GgufValue inner;
                    if (!read_value(c, 9, inner, depth + 1)) return false;
                }
            } else {
                return c.ok = false;
            }
            if (c.ok) {
                v.elems = c.base + elems_at;
                v.elems_bytes = c.pos - elems_at;
            }
            break;
        }
        default: return c.ok = false;
    }
    return c.ok;
}

// Bytes of a tensor of the types the decode path supports (src/load_gguf.jl:135-155); 0 otherwise.
uint64_t tensor_bytes(uint32_t type, const std::vector<uint64_t>& dims) {
    if (dims.empty()) return 0;
    uint64_t rows = 1;
    for (size_t i = 1; i < dims.size(); ++i) rows *= dims[i];
    switch (type) {
        case 0: return dims[0] * rows * 4;                                  // F32
        case 12: return dims[0] % 256 ? 0 : dims[0] / 256 * rows * 144;     // Q4_K
        case 13: return dims[0] % 256 ? 0 : dims[0] / 256 * rows * 176;     // Q5_K
        case 14: return dims[0] % 256 ? 0 : dims[0] / 256 * rows * 210;     // Q6_K
        default: return 0;
    }
}

}  // namespace

GgufFile::~GgufFile() {
    if (base_) munmap(const_cast<uint8_t*>(base_), size_);
    if (fd_ >= 0) close(fd_);
}

bool GgufFile::open(const char* path) {
    fd_ = ::open(path, O_RDONLY);
    if (fd_ < 0) {
        err_ = std::string("cannot open ") + path;
        return false;
    }
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 24) {
        err_ = "Not a GGUF file";
        return false;
    }
    size_ = (size_t)st.st_size;
    void* m = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (m == MAP_FAILED) {
        err_ = "mmap failed";
        return false;
    }
    base_ = static_cast<const uint8_t*>(m);
    Cursor c{base_, size_, 0};
    if (memcmp(base_, "GGUF", 4) != 0) {  // src/load_gguf.jl:86-90
        err_ = "Not a GGUF file";
        return false;
    }
    c.pos = 4;
    version_ = c.take<uint32_t>();
    const uint64_t n_tensors = c.take<uint64_t>();
    const uint64_t n_kv = c.take<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
        err_ = "GGUF header is truncated or implausible";
        return false;
    }
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.string();
        const uint32_t type = c.take<uint32_t>();
        GgufValue v;
        if (!c.ok || !read_value(c, type, v, 0)) {
            err_ = "GGUF metadata is truncated or has a value type that cannot be read (key " + key + ")";
            return false;
        }
        kv_[key] = std::move(v);
    }
    std::vector<uint64_t> offsets;
    for (uint64_t i = 0; i < n_tensors; ++i) {  // src/load_gguf.jl:121-129
        GgufTensor t;
        t.name = c.string();
        const uint32_t nd = c.take<uint32_t>();
        if (!c.ok || nd > 8) {
            err_ = "GGUF tensor directory is truncated";
            return false;
        }
        for (uint32_t d = 0; d < nd; ++d) t.dims.push_back(c.take<uint64_t>());
        t.type = c.take<uint32_t>();
        offsets.push_back(c.take<uint64_t>());
        if (!c.ok) {
            err_ = "GGUF tensor directory is truncated";
            return false;
        }
        t.nbytes = tensor_bytes(t.type, t.dims);
        tensors_.push_back(std::move(t));
    }
    uint64_t alignment = 32;  // src/load_gguf.jl:329
    if (const GgufValue* a = find("general.alignment"))
        if (a->inum > 0) alignment = (uint64_t)a->inum;
    const uint64_t data_start = c.pos + (alignment - (c.pos % alignment)) % alignment;  // align_offset, :131-133
    for (size_t i = 0; i < tensors_.size(); ++i) {
        GgufTensor& t = tensors_[i];
        const uint64_t begin = data_start + offsets[i];
        if (t.nbytes > 0) {
            if (begin > size_ || t.nbytes > size_ - begin) {
                err_ = "tensor " + t.name + " reaches beyond the end of the file";
                return false;
            }
            t.data = base_ + begin;
        }
        index_[t.name] = i;
    }
    return true;
}

const GgufValue* GgufFile::find(const std::string& key) const {
    auto it = kv_.find(key);
    return it == kv_.end() ? nullptr : &it->second;
}

const GgufTensor* GgufFile::tensor(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &tensors_[it->second];
}

}  // namespace l2b
