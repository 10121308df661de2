// Reader for GGUF model files (versions 2 and 3), host side of the decoder: memory-maps the file, parses the header,
// the metadata key/value pairs and the tensor directory, and hands out bounds-checked views of tensor payloads.
//
// Plays the part of rust/crates/quintrit-format/src/gguf.rs (GgufFile::open :190-313, get_tensor_data :316-339,
// get_tensor_scale :343-358, byte_len :161-176) for the tensor types the decoder needs. Written from the published GGUF
// layout: magic "GGUF", u32 version, u64 tensor count, u64 metadata count; strings are u64 length + bytes; metadata
// values are typed (u8 0, i8 1, u16 2, i16 3, u32 4, i32 5, f32 6, bool 7, string 8, array 9, u64 10, i64 11, f64 12);
// a tensor entry is name, u32 rank, u64 dimensions (innermost first), u32 type, u64 offset into the data section, which
// starts at the next multiple of general.alignment (default 32) after the directory.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace qtb {

enum GgmlType : uint32_t { kGgmlF32 = 0, kGgmlF16 = 1, kGgmlQ8_0 = 8, kGgmlBF16 = 30, kGgmlTq1 = 34, kGgmlTq2 = 35, kGgmlI2S = 36, kGgmlQ2 = 42,
                           // not a GGML type: a projection already transcoded to planar velurex rows (ceil(cols / 160) blocks of 32 bytes per row) with its
                           // f32 scale behind the payload, as the pre-transcoded container of this library stores it (quintrit_b200/container.py)
                           kGgmlVelurex = 0x5156 };

struct GgufValue {
    uint32_t type = 0;      // the GGUF value type; arrays keep only their element type and count
    uint64_t u = 0;         // integers and bool
    double f = 0.0;         // floats
    std::string s;          // strings
    uint32_t elem_type = 0; // arrays
    uint64_t count = 0;
    uint64_t max_u = 0;     // arrays of integers: the largest element (per-layer head counts, config.rs:502-512)
    std::vector<std::string> strs;  // arrays of strings (tokenizer.ggml.tokens, tokenizer.ggml.merges)
    std::vector<int64_t> ints;      // arrays of integers (tokenizer.ggml.token_type)
    bool is_int() const { return type <= 5 || type == 7 || type == 10 || type == 11; }
};

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> shape;  // innermost dimension first
    uint32_t type = 0;
    uint64_t offset = 0;
    uint64_t elements() const {
        uint64_t n = 1;
        for (uint64_t d : shape) {
            if (d != 0 && n > UINT64_MAX / d) return UINT64_MAX;
            n *= d;
        }
        return n;
    }
    // bytes of the payload, 0 for a type or shape this reader does not know (gguf.rs:161-176; Q2_0 blocks of 64)
    uint64_t byte_len() const {
        const uint64_t n = elements();
        if (n == UINT64_MAX) return 0;
        switch (type) {
            case kGgmlF32: return n * 4;
            case kGgmlF16:
            case kGgmlBF16: return n * 2;
            case kGgmlQ8_0: return n % 32 == 0 ? n / 32 * 34 : 0;
            case kGgmlI2S: return (n + 3) / 4;
            case kGgmlVelurex: return shape.size() == 2 ? shape[1] * ((shape[0] + 159) / 160) * 32 : 0;  // rows x planar row bytes
            case kGgmlTq1: return n % 256 == 0 ? n / 256 * 54 : 0;
            case kGgmlTq2: return n % 256 == 0 ? n / 256 * 66 : 0;
            case kGgmlQ2: return n % 64 == 0 ? n / 64 * 18 : 0;
            default: return 0;
        }
    }
};

class GgufFile {
  public:
    GgufFile() = default;
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;
    ~GgufFile() { close(); }

    // 0 = fine, 1 = cannot be read (not a regular file, open/mmap failed), 2 = malformed; `error` says why.
    int open(const char* path, std::string& error) {
        close();
        struct stat st;
        if (::stat(path, &st) != 0 || !S_ISREG(st.st_mode)) {
            error = std::string("'") + path + "' is not a regular file";
            return 1;
        }
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) {
            error = std::string("cannot open '") + path + "'";
            return 1;
        }
        size_ = static_cast<size_t>(st.st_size);
        if (size_ < 24) {
            ::close(fd);
            error = "the file is too short for a GGUF header";
            return 2;
        }
        void* p = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) {
            error = "cannot map the file into memory";
            size_ = 0;
            return 1;
        }
        base_ = static_cast<const uint8_t*>(p);
        return parse(error) ? 0 : 2;
    }

    void close() {
        if (base_ != nullptr) ::munmap(const_cast<uint8_t*>(base_), size_);
        base_ = nullptr;
        size_ = 0;
        metadata.clear();
        tensors.clear();
        order.clear();
    }

    const GgufValue* find(const std::string& key) const {
        auto it = metadata.find(key);
        return it == metadata.end() ? nullptr : &it->second;
    }
    const GgufTensor* tensor(const std::string& name) const {
        auto it = tensors.find(name);
        return it == tensors.end() ? nullptr : &it->second;
    }
    // Payload of a tensor, nullptr if it is unknown, of an unknown layout, or does not lie inside the file.
    const uint8_t* data(const GgufTensor& t, uint64_t* len = nullptr) const {
        const uint64_t n = t.byte_len();
        if (n == 0 || t.offset > size_ - data_start_ || n > size_ - data_start_ - t.offset) return nullptr;
        if (len != nullptr) *len = n;
        return base_ + data_start_ + t.offset;
    }
    // The f32 that follows an I2_S payload (gguf.rs:343-358); false if it is not inside the file.
    bool trailing_scale(const GgufTensor& t, float* out) const {
        uint64_t n = 0;
        const uint8_t* p = data(t, &n);
        if (p == nullptr || static_cast<uint64_t>(p - base_) + n + 4 > size_) return false;
        std::memcpy(out, p + n, 4);
        return true;
    }

    uint64_t data_start() const { return data_start_; }

    uint32_t version = 0;
    std::map<std::string, GgufValue> metadata;
    std::map<std::string, GgufTensor> tensors;
    std::vector<std::string> order;  // tensor names in file order

  private:
    const uint8_t* base_ = nullptr;
    size_t size_ = 0, pos_ = 0, data_start_ = 0;

    template <typename T>
    bool read(T* out) {
        if (size_ - pos_ < sizeof(T)) return false;
        std::memcpy(out, base_ + pos_, sizeof(T));
        pos_ += sizeof(T);
        return true;
    }
    bool read_string(std::string* out) {
        uint64_t n = 0;
        if (!read(&n) || n > size_ - pos_) return false;
        out->assign(reinterpret_cast<const char*>(base_ + pos_), static_cast<size_t>(n));
        pos_ += static_cast<size_t>(n);
        return true;
    }
    static size_t scalar_size(uint32_t type) {
        switch (type) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
            default: return 0;
        }
    }
    bool read_scalar(uint32_t type, GgufValue* v) {
        const size_t n = scalar_size(type);
        if (n == 0 || size_ - pos_ < n) return false;
        uint64_t raw = 0;
        std::memcpy(&raw, base_ + pos_, n);  // little-endian host
        pos_ += n;
        switch (type) {
            case 1: v->u = static_cast<uint64_t>(static_cast<int64_t>(static_cast<int8_t>(raw))); break;
            case 3: v->u = static_cast<uint64_t>(static_cast<int64_t>(static_cast<int16_t>(raw))); break;
            case 5: v->u = static_cast<uint64_t>(static_cast<int64_t>(static_cast<int32_t>(raw))); break;
            case 6: {
                float f;
                const uint32_t bits = static_cast<uint32_t>(raw);
                std::memcpy(&f, &bits, 4);
                v->f = f;
                break;
            }
            case 12: std::memcpy(&v->f, &raw, 8); break;
            default: v->u = raw; break;
        }
        return true;
    }
    bool read_value(GgufValue* v, int depth) {
        if (!read(&v->type)) return false;
        if (v->type == 8) return read_string(&v->s);
        if (v->type == 9) {
            if (depth > 0 || !read(&v->elem_type) || !read(&v->count)) return false;  // nested arrays are not used by model files
            if (v->elem_type == 8) {
                if (v->count > (size_ - pos_) / 8) return false;  // every string has an 8-byte length
                v->strs.resize(static_cast<size_t>(v->count));
                for (uint64_t i = 0; i < v->count; ++i)
                    if (!read_string(&v->strs[static_cast<size_t>(i)])) return false;
                return true;
            }
            const size_t n = scalar_size(v->elem_type);
            if (n == 0 || v->count > (size_ - pos_) / n) return false;
            GgufValue e;
            e.type = v->elem_type;
            for (uint64_t i = 0; i < v->count; ++i) {
                if (!read_scalar(v->elem_type, &e)) return false;
                if (e.is_int() && e.u > v->max_u) v->max_u = e.u;
                if (e.is_int()) v->ints.push_back(static_cast<int64_t>(e.u));
            }
            return true;
        }
        return read_scalar(v->type, v);
    }
    bool parse(std::string& error) {
        pos_ = 0;
        uint32_t magic = 0;
        uint64_t n_tensors = 0, n_kv = 0;
        if (!read(&magic) || magic != 0x46554747u) {  // "GGUF"
            error = "the file does not start with the GGUF magic";
            return false;
        }
        if (!read(&version) || (version != 2 && version != 3)) {
            error = "GGUF version " + std::to_string(version) + " is not supported (2 or 3)";
            return false;
        }
        if (!read(&n_tensors) || !read(&n_kv) || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
            error = "implausible tensor or metadata count";
            return false;
        }
        for (uint64_t i = 0; i < n_kv; ++i) {
            std::string key;
            GgufValue v;
            if (!read_string(&key) || !read_value(&v, 0)) {
                error = "metadata entry " + std::to_string(i) + " is truncated or of an unknown type";
                return false;
            }
            metadata[key] = std::move(v);
        }
        for (uint64_t i = 0; i < n_tensors; ++i) {
            GgufTensor t;
            uint32_t rank = 0;
            if (!read_string(&t.name) || !read(&rank) || rank > 8) {
                error = "tensor entry " + std::to_string(i) + " is truncated";
                return false;
            }
            t.shape.resize(rank);
            for (uint32_t d = 0; d < rank; ++d)
                if (!read(&t.shape[d])) {
                    error = "tensor entry " + std::to_string(i) + " is truncated";
                    return false;
                }
            if (!read(&t.type) || !read(&t.offset)) {
                error = "tensor entry " + std::to_string(i) + " is truncated";
                return false;
            }
            order.push_back(t.name);
            tensors[t.name] = std::move(t);
        }
        uint64_t align = 32;
        if (const GgufValue* a = find("general.alignment"))
            if (a->is_int() && a->u >= 1 && a->u <= (1u << 20)) align = a->u;
        data_start_ = (pos_ + align - 1) / align * align;
        if (data_start_ > size_) {
            error = "the data section starts beyond the end of the file";
            return false;
        }
        return true;
    }
};

}  // namespace qtb
