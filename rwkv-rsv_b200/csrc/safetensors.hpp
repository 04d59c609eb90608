// Minimal read-only safetensors container parser (header-only, no dependencies).
//
// File format: u64 little-endian header length N, N bytes of JSON
// {"name": {"dtype": "F16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {...}},
// then the raw tensor bytes; offsets are relative to the first byte after the header.
// The reference reads the same container through the `safetensors` crate
// (src/model.rs:276-279, src/gpu_model.rs:401-405); nothing else of that crate is used.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace rsv {

struct StTensor {
    std::string dtype;           // "F16", "F32", "U8", "U32", ...
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;
    size_t nbytes = 0;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

class SafeTensorsFile {
public:
    explicit SafeTensorsFile(const std::string& path) {
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw std::runtime_error("safetensors: cannot open " + path);
        struct stat st;
        if (fstat(fd_, &st) != 0 || st.st_size < 8) {
            ::close(fd_);
            throw std::runtime_error("safetensors: file too small: " + path);
        }
        size_ = (size_t)st.st_size;
        base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (base_ == MAP_FAILED) {
            ::close(fd_);
            throw std::runtime_error("safetensors: mmap failed: " + path);
        }
        try {
            uint64_t hlen;
            memcpy(&hlen, base_, 8);
            if (hlen > size_ - 8) throw std::runtime_error("safetensors: header length exceeds file size");
            parse_header((const char*)base_ + 8, (size_t)hlen, base_ + 8 + hlen, size_ - 8 - (size_t)hlen);
        } catch (...) {
            munmap((void*)base_, size_);
            ::close(fd_);
            throw;
        }
    }
    ~SafeTensorsFile() {
        if (base_ && base_ != MAP_FAILED) munmap((void*)base_, size_);
        if (fd_ >= 0) ::close(fd_);
    }
    SafeTensorsFile(const SafeTensorsFile&) = delete;
    SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;

    bool has(const std::string& name) const { return tensors_.count(name) != 0; }
    const StTensor& get(const std::string& name) const {
        auto it = tensors_.find(name);
        if (it == tensors_.end()) throw std::runtime_error("safetensors: missing tensor " + name);
        return it->second;
    }
    const std::map<std::string, StTensor>& tensors() const { return tensors_; }
    const std::map<std::string, std::string>& metadata() const { return meta_; }

private:
    int fd_ = -1;
    size_t size_ = 0;
    const uint8_t* base_ = nullptr;
    std::map<std::string, StTensor> tensors_;
    std::map<std::string, std::string> meta_;

    // --- tiny JSON subset parser: objects, arrays of integers, strings, integers ---
    struct Cur {
        const char* p;
        const char* e;
    };
    static void ws(Cur& c) {
        while (c.p < c.e && (*c.p == ' ' || *c.p == '\n' || *c.p == '\t' || *c.p == '\r')) ++c.p;
    }
    static void expect(Cur& c, char ch) {
        ws(c);
        if (c.p >= c.e || *c.p != ch) throw std::runtime_error(std::string("safetensors: header parse error, expected '") + ch + "'");
        ++c.p;
    }
    static bool peek(Cur& c, char ch) {
        ws(c);
        return c.p < c.e && *c.p == ch;
    }
    static std::string str(Cur& c) {
        expect(c, '"');
        std::string s;
        while (c.p < c.e && *c.p != '"') {
            if (*c.p == '\\' && c.p + 1 < c.e) {
                ++c.p;
                switch (*c.p) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'u':  // keep \uXXXX escapes verbatim; tensor names are ASCII
                        s += "\\u";
                        break;
                    default: s += *c.p;
                }
                ++c.p;
            } else {
                s += *c.p++;
            }
        }
        expect(c, '"');
        return s;
    }
    static int64_t integer(Cur& c) {
        ws(c);
        bool neg = false;
        if (c.p < c.e && *c.p == '-') {
            neg = true;
            ++c.p;
        }
        if (c.p >= c.e || *c.p < '0' || *c.p > '9') throw std::runtime_error("safetensors: header parse error, expected integer");
        int64_t v = 0;
        while (c.p < c.e && *c.p >= '0' && *c.p <= '9') v = v * 10 + (*c.p++ - '0');
        return neg ? -v : v;
    }
    static std::vector<int64_t> int_array(Cur& c) {
        std::vector<int64_t> out;
        expect(c, '[');
        if (peek(c, ']')) {
            ++c.p;
            return out;
        }
        for (;;) {
            out.push_back(integer(c));
            if (peek(c, ',')) {
                ++c.p;
                continue;
            }
            expect(c, ']');
            return out;
        }
    }
    static void skip_value(Cur& c) {
        ws(c);
        if (c.p >= c.e) throw std::runtime_error("safetensors: truncated header");
        if (*c.p == '"') {
            (void)str(c);
        } else if (*c.p == '{') {
            ++c.p;
            if (peek(c, '}')) {
                ++c.p;
                return;
            }
            for (;;) {
                (void)str(c);
                expect(c, ':');
                skip_value(c);
                if (peek(c, ',')) {
                    ++c.p;
                    continue;
                }
                expect(c, '}');
                return;
            }
        } else if (*c.p == '[') {
            ++c.p;
            if (peek(c, ']')) {
                ++c.p;
                return;
            }
            for (;;) {
                skip_value(c);
                if (peek(c, ',')) {
                    ++c.p;
                    continue;
                }
                expect(c, ']');
                return;
            }
        } else {
            while (c.p < c.e && *c.p != ',' && *c.p != '}' && *c.p != ']') ++c.p;
        }
    }

    void parse_header(const char* h, size_t n, const uint8_t* data, size_t data_len) {
        Cur c{h, h + n};
        expect(c, '{');
        if (peek(c, '}')) return;
        for (;;) {
            std::string name = str(c);
            expect(c, ':');
            if (name == "__metadata__") {
                expect(c, '{');
                if (!peek(c, '}')) {
                    for (;;) {
                        std::string k = str(c);
                        expect(c, ':');
                        ws(c);
                        if (c.p < c.e && *c.p == '"')
                            meta_[k] = str(c);
                        else
                            skip_value(c);
                        if (peek(c, ',')) {
                            ++c.p;
                            continue;
                        }
                        break;
                    }
                }
                expect(c, '}');
            } else {
                StTensor t;
                int64_t b = -1, e = -1;
                expect(c, '{');
                for (;;) {
                    std::string k = str(c);
                    expect(c, ':');
                    if (k == "dtype")
                        t.dtype = str(c);
                    else if (k == "shape")
                        t.shape = int_array(c);
                    else if (k == "data_offsets") {
                        auto v = int_array(c);
                        if (v.size() != 2) throw std::runtime_error("safetensors: bad data_offsets for " + name);
                        b = v[0];
                        e = v[1];
                    } else
                        skip_value(c);
                    if (peek(c, ',')) {
                        ++c.p;
                        continue;
                    }
                    break;
                }
                expect(c, '}');
                if (b < 0 || e < b || (size_t)e > data_len) throw std::runtime_error("safetensors: data_offsets out of range for " + name);
                t.data = data + b;
                t.nbytes = (size_t)(e - b);
                // the byte range must be exactly shape x element size (the reference's safetensors crate rejects such files too):
                // readers copy numel() elements without looking at nbytes again
                {
                    size_t es = 0;
                    if (t.dtype == "F64" || t.dtype == "I64" || t.dtype == "U64") es = 8;
                    else if (t.dtype == "F32" || t.dtype == "I32" || t.dtype == "U32") es = 4;
                    else if (t.dtype == "F16" || t.dtype == "BF16" || t.dtype == "I16" || t.dtype == "U16") es = 2;
                    else if (t.dtype == "U8" || t.dtype == "I8" || t.dtype == "BOOL" || t.dtype == "F8_E4M3" || t.dtype == "F8_E5M2") es = 1;
                    if (es) {
                        size_t n = 1;
                        for (int64_t d : t.shape) {
                            if (d < 0) throw std::runtime_error("safetensors: negative dimension in " + name);
                            if (d != 0 && n > (size_t)-1 / (size_t)d) throw std::runtime_error("safetensors: shape overflows in " + name);
                            n *= (size_t)d;
                        }
                        if (n > (size_t)-1 / es || n * es != t.nbytes)
                            throw std::runtime_error("safetensors: " + name + " holds " + std::to_string(t.nbytes) + " bytes but its shape and dtype need " +
                                                     std::to_string(n * es));
                    }
                }
                tensors_[name] = std::move(t);
            }
            if (peek(c, ',')) {
                ++c.p;
                continue;
            }
            break;
        }
        expect(c, '}');
    }
};

// IEEE binary16 -> binary32 widening (exact), as `half::f16::to_f32` does for the reference
// (src/model.rs:208-217).
static inline float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do {
                ++e;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// binary32 -> binary16, round to nearest even (matches `half::f16::from_f32`, numpy astype(float16),
// and CUDA __float2half_rn).
static inline uint16_t float_to_half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
    }
    if (ax >= 0x477FF000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax < 0x33000001u) {  // < 2^-25 (or exactly 2^-25, ties to even 0)
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    if (e < -14) {  // subnormal half
        int shift = 13 + (-14 - e);
        uint32_t r = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (r & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;  // carry may bump the exponent: correct
    return (uint16_t)(sign | r);
}

}  // namespace rsv
