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
                    case 'u': p += 4; out += '?'; break;   // names of interest are ASCII
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
    int64_t integer() {
        ws();
        char* e = nullptr;
        const long long v = strtoll(p, &e, 10);
        if (e == p) ok = false;
        p = e;
        return v;
    }
    void skip_value() {   // any JSON value
        ws();
        if (p >= end) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (eat(close)) return;
            do {
                if (open == '{') { str(); if (!eat(':')) { ok = false; return; } }
                skip_value();
                if (!ok) return;
            } while (eat(','));
            if (!eat(close)) ok = false;
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
        if (kv.second.end < kv.second.begin || kv.second.end > payload) {
            *err = "tensor " + kv.first + " lies outside the file";
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
