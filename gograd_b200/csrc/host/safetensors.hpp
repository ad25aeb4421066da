// safetensors v1 container as gograd writes and reads it (autograd/safetensors.go:30-98,
// autograd/safetensors_stream.go:28-96): 8-byte little-endian header length, JSON header
// padded with spaces to a multiple of 8, entries sorted by name, dtype F32 only,
// contiguous data_offsets, header at most 16 MiB; written to a temporary file in the
// target directory, fsync'ed and renamed over the target.
#ifndef GG_SAFETENSORS_HPP
#define GG_SAFETENSORS_HPP

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <climits>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "json_min.hpp"

namespace autograd {

struct SafeTensorEntry {
    std::vector<float> Values;
    std::vector<int> Shape;
};

using EntryMap = std::map<std::string, SafeTensorEntry>;   // std::map iterates in sorted-name order
using Metadata = std::map<std::string, std::string>;

constexpr size_t kSafeTensorHeaderLimit = 16u << 20;

// safeNumel (autograd/safetensors.go:100-124): product of the dimensions, 0 when any
// dimension is 0, an error for negative or oversized shapes.
inline bool safe_numel(const std::vector<int>& shape, long long limit, long long* count) {
    bool zero = false;
    for (int d : shape) {
        if (d < 0) return false;
        zero = zero || d == 0;
    }
    if (zero) {
        *count = 0;
        return true;
    }
    long long c = 1;
    for (int d : shape) {
        if (d > limit || c > limit / d) return false;
        c *= d;
    }
    if (c > limit) return false;
    *count = c;
    return true;
}

inline std::string write_safetensors(const std::string& path, const EntryMap& entries, const Metadata* metadata) {
    // Go marshals map[string]any with sorted keys; "__metadata__" sorts before any
    // name starting with a letter but not before every possible name, so merge by key.
    std::map<std::string, std::string> header;  // name -> JSON text
    long long offset = 0;
    for (const auto& kv : entries) {
        const std::string& name = kv.first;
        const SafeTensorEntry& e = kv.second;
        long long count = 0;
        if (!safe_numel(e.Shape, (long long)e.Values.size(), &count) || count != (long long)e.Values.size() ||
            name == "__metadata__")
            return "autograd: incompatible tensor " + name;
        long long end = offset + count * 4;
        std::string j = "{\"dtype\":\"F32\",\"shape\":[";
        for (size_t i = 0; i < e.Shape.size(); i++) j += (i ? "," : "") + std::to_string(e.Shape[i]);
        j += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(end) + "]}";
        header[name] = j;
        offset = end;
    }
    if (metadata) {
        std::string j = "{";
        bool first = true;
        for (const auto& kv : *metadata) {
            j += (first ? "" : ",") + ggjson::quote(kv.first) + ":" + ggjson::quote(kv.second);
            first = false;
        }
        header["__metadata__"] = j + "}";
    }
    std::string h = "{";
    bool first = true;
    for (const auto& kv : header) {
        h += (first ? "" : ",") + ggjson::quote(kv.first) + ":" + kv.second;
        first = false;
    }
    h += "}";
    while (h.size() % 8 != 0) h += ' ';
    if (h.size() > kSafeTensorHeaderLimit) return "autograd: invalid safetensors header length";

    std::string dir = ".";
    size_t slash = path.rfind('/');
    if (slash != std::string::npos) dir = slash == 0 ? "/" : path.substr(0, slash);
    std::string tmpl = dir + "/.gograd-checkpoint-XXXXXX";
    std::vector<char> name(tmpl.begin(), tmpl.end());
    name.push_back(0);
    int fd = mkstemp(name.data());
    if (fd < 0) return "autograd: cannot create a temporary file in " + dir;
    auto write_all = [&](const void* data, size_t n) {
        const char* p = (const char*)data;
        while (n > 0) {
            ssize_t w = ::write(fd, p, n);
            if (w <= 0) return false;
            p += w;
            n -= (size_t)w;
        }
        return true;
    };
    unsigned char prefix[8];
    uint64_t hl = h.size();
    for (int i = 0; i < 8; i++) prefix[i] = (unsigned char)(hl >> (8 * i));
    bool ok = write_all(prefix, 8) && write_all(h.data(), h.size());
    for (const auto& kv : entries) {  // host is little-endian: floats are written as they are
        if (!ok) break;
        if (!kv.second.Values.empty()) ok = write_all(kv.second.Values.data(), kv.second.Values.size() * 4);
    }
    ok = ok && fsync(fd) == 0;
    ok = (close(fd) == 0) && ok;
    if (!ok || rename(name.data(), path.c_str()) != 0) {
        unlink(name.data());
        return "autograd: writing " + path + " failed";
    }
    return "";
}

inline std::string read_safetensors(const std::string& path, EntryMap* entries, Metadata* metadata) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return "open " + path + ": no such file or it cannot be read";
    struct Closer {
        FILE* f;
        ~Closer() { fclose(f); }
    } closer{f};
    struct stat st;
    if (fstat(fileno(f), &st) != 0) return "autograd: cannot stat " + path;
    if (st.st_size < 8) return "autograd: short safetensors file";
    unsigned char prefix[8];
    if (fread(prefix, 1, 8, f) != 8) return "autograd: short safetensors file";
    uint64_t hlen = 0;
    for (int i = 0; i < 8; i++) hlen |= (uint64_t)prefix[i] << (8 * i);
    if (hlen > kSafeTensorHeaderLimit || hlen > (uint64_t)(st.st_size - 8)) return "autograd: invalid safetensors header length";
    std::string text(hlen, 0);
    if (hlen && fread(&text[0], 1, hlen, f) != hlen) return "autograd: short safetensors header";
    ggjson::Value root;
    std::string err;
    if (!ggjson::Parser(text).parse(&root, &err) || !root.is(ggjson::Value::Obj)) return "autograd: invalid safetensors header: " + err;
    metadata->clear();
    entries->clear();
    long long data_size = (long long)st.st_size - 8 - (long long)hlen;
    long long limit = data_size / 4;
    struct Range {
        long long a, b;
        std::string name;
        std::vector<int> shape;
    };
    std::vector<Range> ranges;
    for (const auto& kv : *root.obj) {
        if (kv.first == "__metadata__") {
            if (!kv.second.is(ggjson::Value::Obj)) return "autograd: invalid safetensors metadata";
            for (const auto& m : *kv.second.obj) {
                if (!m.second.is(ggjson::Value::String)) return "autograd: invalid safetensors metadata";
                (*metadata)[m.first] = m.second.raw;
            }
            continue;
        }
        const ggjson::Value& h = kv.second;
        const ggjson::Value *dt = h.get("dtype"), *sh = h.get("shape"), *of = h.get("data_offsets");
        if (!dt || !sh || !of || !dt->is(ggjson::Value::String) || !sh->is(ggjson::Value::Arr) ||
            !of->is(ggjson::Value::Arr) || of->arr->size() != 2)
            return "autograd: " + kv.first + ": invalid header entry";
        if (dt->raw != "F32") return "autograd: incompatible dtype " + dt->raw + " for " + kv.first;
        Range r;
        r.name = kv.first;
        for (const auto& d : *sh->arr) {
            if (!d.is(ggjson::Value::Number) || d.num != std::floor(d.num) || std::fabs(d.num) > INT_MAX)
                return "autograd: invalid shape " + kv.first;
            r.shape.push_back((int)d.num);
        }
        long long count = 0;
        if (!safe_numel(r.shape, limit, &count)) return "autograd: invalid shape " + kv.first;
        r.a = (long long)(*of->arr)[0].num;
        r.b = (long long)(*of->arr)[1].num;
        if (r.a < 0 || r.b < r.a || r.b > data_size || r.b - r.a != count * 4) return "autograd: invalid offsets " + kv.first;
        ranges.push_back(r);
    }
    std::vector<Range> sorted = ranges;
    std::sort(sorted.begin(), sorted.end(), [](const Range& x, const Range& y) { return x.a < y.a; });
    long long prev_end = -1;
    for (const Range& r : sorted) {
        if (r.b == r.a) continue;
        if (prev_end > r.a) return "autograd: overlapping tensor ranges";
        prev_end = r.b;
    }
    for (const Range& r : ranges) {
        SafeTensorEntry e;
        e.Shape = r.shape;
        e.Values.resize((size_t)(r.b - r.a) / 4);
        if (!e.Values.empty()) {
            if (fseeko(f, (off_t)(8 + hlen + r.a), SEEK_SET) != 0 ||
                fread(e.Values.data(), 4, e.Values.size(), f) != e.Values.size())
                return "autograd: short read of " + r.name;
        }
        (*entries)[r.name] = std::move(e);
    }
    return "";
}

}  // namespace autograd
#endif
