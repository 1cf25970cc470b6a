// Minimal reader of the safetensors container (host code): 8-byte little-endian header length, a JSON
// object {name: {"dtype": ..., "shape": [...], "data_offsets": [begin, end]}, ...}, then the tensor bytes.
// The file is mapped read-only; tensors are handed out as pointers into the mapping.
//
// Replaces, for the MoE block, FFAI's loader path: Loader/SafeTensors.swift:377-396 (container),
// Layers.swift:340-363 (bit width derived from the packed and the scale shapes) and the stacked expert
// triplets `…switch_mlp.{gate,up,down}_proj.{weight,scales,biases}` (Qwen3xText.swift:605-624) /
// `…experts.switch_glu.*` (Gemma4Text.swift:540-554).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <climits>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace ffai {
namespace st {

struct Tensor {
    std::string dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;
};

struct File {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    const uint8_t* data = nullptr;     // first byte after the header
    std::map<std::string, Tensor> tensors;
    std::string error;
};

// ── a JSON walker for exactly this shape of document ──
struct Cursor {
    const char* p;
    const char* end;
    bool ok = true;
    int depth = 0;                     // nesting of skipped values (bounded: the walker recurses)
    static constexpr int MAX_DEPTH = 32;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
    bool peek(char c) { ws(); return p < end && *p == c; }
    std::string str() {
        ws();
        std::string out;
        if (p >= end || *p != '"') { ok = false; return out; }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'u':                              // names of interest are ASCII
                        if (end - p < 5) { ok = false; return out; }
                        p += 4; out += '?'; break;
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) { ok = false; return out; }
        ++p;
        return out;
    }
    int64_t integer() {   // decimal digits with an optional sign; never reads at or past `end`
        ws();
        bool neg = false;
        if (p < end && (*p == '-' || *p == '+')) { neg = *p == '-'; ++p; }
        if (p >= end || *p < '0' || *p > '9') { ok = false; return 0; }
        uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (uint64_t)INT64_MAX / 10) { ok = false; return 0; }
            v = v * 10 + (uint64_t)(*p - '0');
            if (v > (uint64_t)INT64_MAX) { ok = false; return 0; }
            ++p;
        }
        return neg ? -(int64_t)v : (int64_t)v;
    }
    void skip_value() {   // any JSON value
        ws();
        if (p >= end) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            if (++depth > MAX_DEPTH) { ok = false; return; }
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (eat(close)) { --depth; return; }
            do {
                if (open == '{') { str(); if (!ok || !eat(':')) { ok = false; return; } }
                skip_value();
                if (!ok) return;
            } while (eat(','));
            if (!eat(close)) ok = false;
            --depth;
            return;
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;   // number, true, false, null
    }
};

inline bool parse_header(File& f, const char* json, size_t n) {
    Cursor c{json, json + n};
    if (!c.eat('{')) { f.error = "header is not a JSON object"; return false; }
    if (c.eat('}')) return true;
    do {
        const std::string name = c.str();
        if (!c.ok || !c.eat(':')) { f.error = "malformed header near a tensor name"; return false; }
        if (name == "__metadata__") { c.skip_value(); continue; }
        Tensor t;
        if (!c.eat('{')) { f.error = "tensor entry is not an object: " + name; return false; }
        if (!c.peek('}')) {
            do {
                const std::string key = c.str();
                if (!c.eat(':')) { c.ok = false; break; }
                if (key == "dtype") t.dtype = c.str();
                else if (key == "shape") {
                    if (!c.eat('[')) { c.ok = false; break; }
                    if (!c.peek(']')) { do t.shape.push_back(c.integer()); while (c.eat(',')); }
                    if (!c.eat(']')) c.ok = false;
                } else if (key == "data_offsets") {
                    if (!c.eat('[')) { c.ok = false; break; }
                    t.begin = (uint64_t)c.integer();
                    if (!c.eat(',')) c.ok = false;
                    t.end = (uint64_t)c.integer();
                    if (!c.eat(']')) c.ok = false;
                } else c.skip_value();
            } while (c.ok && c.eat(','));
        }
        if (!c.ok || !c.eat('}')) { f.error = "malformed entry for tensor " + name; return false; }
        f.tensors[name] = t;
    } while (c.eat(','));
    if (!c.eat('}')) { f.error = "header does not end with '}'"; return false; }
    return true;
}

// Bytes per element of the dtypes the container defines; 0 for a name this reader does not know.
inline int dtype_bytes(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}

// The byte range of a tensor must be exactly what its shape and dtype say (a header that declares a large
// shape over a short range would otherwise send readers past the mapping).  False on a negative dimension,
// an overflowing element count, or a size mismatch for a known dtype.
inline bool shape_matches_range(const Tensor& t) {
    uint64_t n = 1;
    for (int64_t d : t.shape) {
        if (d < 0) return false;
        if (d != 0 && n > UINT64_MAX / (uint64_t)d) return false;
        n *= (uint64_t)d;
    }
    const int eb = dtype_bytes(t.dtype);
    if (eb == 0) return true;
    if (n > UINT64_MAX / (uint64_t)eb) return false;
    return n * (uint64_t)eb == t.end - t.begin;
}

inline File* open_file(const char* path, std::string* err) {
    File* f = new File();
    f->fd = ::open(path, O_RDONLY);
    struct stat sb;
    if (f->fd < 0 || fstat(f->fd, &sb) != 0 || sb.st_size < 8) {
        *err = std::string("cannot open ") + path;
        if (f->fd >= 0) ::close(f->fd);
        delete f;
        return nullptr;
    }
    f->size = (size_t)sb.st_size;
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { *err = "mmap failed"; ::close(f->fd); delete f; return nullptr; }
    f->map = static_cast<const uint8_t*>(m);
    uint64_t hlen = 0;
    memcpy(&hlen, f->map, 8);
    if (hlen > f->size - 8) { *err = "header length exceeds the file"; munmap(m, f->size); ::close(f->fd); delete f; return nullptr; }
    f->data = f->map + 8 + hlen;
    if (!parse_header(*f, reinterpret_cast<const char*>(f->map + 8), (size_t)hlen)) {
        *err = f->error;
        munmap(m, f->size); ::close(f->fd); delete f;
        return nullptr;
    }
    const uint64_t payload = f->size - 8 - hlen;
    for (const auto& kv : f->tensors)
        if (kv.second.end < kv.second.begin || kv.second.end > payload || !shape_matches_range(kv.second)) {
            *err = "tensor " + kv.first + (kv.second.end > payload || kv.second.end < kv.second.begin
                                               ? " lies outside the file" : ": shape and dtype do not match its byte range");
            munmap(m, f->size); ::close(f->fd); delete f;
            return nullptr;
        }
    return f;
}

inline void close_file(File* f) {
    if (!f) return;
    if (f->map) munmap(const_cast<uint8_t*>(f->map), f->size);
    if (f->fd >= 0) ::close(f->fd);
    delete f;
}

inline const Tensor* find(const File* f, const std::string& name) {
    auto it = f->tensors.find(name);
    return it == f->tensors.end() ? nullptr : &it->second;
}

}  // namespace st
}  // namespace ffai
