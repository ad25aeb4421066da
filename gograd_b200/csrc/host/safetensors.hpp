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

// The JSON header of a container holding F32 entries of the given shapes in sorted-name order
// with contiguous offsets, padded with spaces to a multiple of 8 (autograd/safetensors.go:30-98).
// Go marshals map[string]any with sorted keys; "__metadata__" sorts before any name starting
// with a letter but not before every possible name, so it is merged by key.
inline std::string safetensors_header(const std::map<std::string, std::vector<int>>& shapes, const Metadata* metadata,
                                      std::string* out) {
    std::map<std::string, std::string> header;  // name -> JSON text
    long long offset = 0;
    for (const auto& kv : shapes) {
        const std::string& name = kv.first;
        long long count = 0;
        if (!safe_numel(kv.second, (long long)1 << 40, &count) || name == "__metadata__")
            return "autograd: incompatible tensor " + name;
        long long end = offset + count * 4;
        std::string j = "{\"dtype\":\"F32\",\"shape\":[";
        for (size_t i = 0; i < kv.second.size(); i++) j += (i ? "," : "") + std::to_string(kv.second[i]);
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
    *out = std::move(h);
    return "";
}

// A container written front to back without holding its data: the shapes are known first, the
// values arrive entry by entry in sorted-name order (an entry may arrive in consecutive pieces).
// Temporary file in the target directory, fsync, rename: the same discipline and the same bytes
// as write_safetensors.
class SafeTensorStream {
   public:
    SafeTensorStream() = default;
    SafeTensorStream(const SafeTensorStream&) = delete;
    SafeTensorStream& operator=(const SafeTensorStream&) = delete;
    ~SafeTensorStream() { Abort(); }

    std::string Begin(const std::string& path, const std::map<std::string, std::vector<int>>& shapes,
                      const Metadata* metadata) {
        if (fd_ >= 0) return "autograd: the stream is already open";
        std::string h;
        std::string e = safetensors_header(shapes, metadata, &h);
        if (!e.empty()) return e;
        order_.clear();
        for (const auto& kv : shapes) {
            long long count = 0;
            safe_numel(kv.second, (long long)1 << 40, &count);
            order_.push_back({kv.first, count});
        }
        next_ = 0;
        done_in_entry_ = 0;
        skip_empty();
        path_ = path;
        std::string dir = ".";
        size_t slash = path.rfind('/');
        if (slash != std::string::npos) dir = slash == 0 ? "/" : path.substr(0, slash);
        std::string tmpl = dir + "/.gograd-checkpoint-XXXXXX";
        std::vector<char> name(tmpl.begin(), tmpl.end());
        name.push_back(0);
        fd_ = mkstemp(name.data());
        if (fd_ < 0) return "autograd: cannot create a temporary file in " + dir;
        tmp_ = name.data();
        unsigned char prefix[8];
        uint64_t hl = h.size();
        for (int i = 0; i < 8; i++) prefix[i] = (unsigned char)(hl >> (8 * i));
        if (!write_all(prefix, 8) || !write_all(h.data(), h.size())) {
            Abort();
            return "autograd: writing " + path + " failed";
        }
        return "";
    }

    // The entry the file wants next and how many of its values are still missing; false at the end.
    bool Next(std::string* name, long long* remaining) const {
        if (next_ >= order_.size()) return false;
        *name = order_[next_].first;
        *remaining = order_[next_].second - done_in_entry_;
        return true;
    }

    std::string Append(const std::string& name, const float* values, long long count) {
        if (fd_ < 0) return "autograd: the stream is not open";
        if (next_ >= order_.size() || order_[next_].first != name)
            return "autograd: entry " + name + " is out of order" +
                   (next_ < order_.size() ? " (the file wants " + order_[next_].first + ")" : " (the file is complete)");
        if (count < 0 || count > order_[next_].second - done_in_entry_) return "autograd: too many values for " + name;
        if (count > 0 && !write_all(values, (size_t)count * 4)) {  // host is little-endian: floats are written as they are
            Abort();
            return "autograd: writing " + path_ + " failed";
        }
        done_in_entry_ += count;
        if (done_in_entry_ == order_[next_].second) {
            next_++;
            done_in_entry_ = 0;
            skip_empty();
        }
        return "";
    }

    std::string Finish() {
        if (fd_ < 0) return "autograd: the stream is not open";
        if (next_ < order_.size()) {
            std::string missing = order_[next_].first;
            Abort();
            return "autograd: entry " + missing + " was not written";
        }
        bool ok = fsync(fd_) == 0;
        ok = (close(fd_) == 0) && ok;
        fd_ = -1;
        if (!ok || rename(tmp_.c_str(), path_.c_str()) != 0) {
            unlink(tmp_.c_str());
            return "autograd: writing " + path_ + " failed";
        }
        return "";
    }

    void Abort() {
        if (fd_ >= 0) {
            close(fd_);
            unlink(tmp_.c_str());
            fd_ = -1;
        }
    }

   private:
    int fd_ = -1;
    std::string path_, tmp_;
    std::vector<std::pair<std::string, long long>> order_;
    size_t next_ = 0;
    long long done_in_entry_ = 0;

    void skip_empty() {
        while (next_ < order_.size() && order_[next_].second == 0) next_++;
    }
    bool write_all(const void* data, size_t n) {
        const char* p = (const char*)data;
        while (n > 0) {
            ssize_t w = ::write(fd_, p, n);
            if (w <= 0) return false;
            p += w;
            n -= (size_t)w;
        }
        return true;
    }
};

inline std::string write_safetensors(const std::string& path, const EntryMap& entries, const Metadata* metadata) {
    std::map<std::string, std::vector<int>> shapes;
    for (const auto& kv : entries) {
        long long count = 0;
        if (!safe_numel(kv.second.Shape, (long long)kv.second.Values.size(), &count) ||
            count != (long long)kv.second.Values.size() || kv.first == "__metadata__")
            return "autograd: incompatible tensor " + kv.first;
        shapes[kv.first] = kv.second.Shape;
    }
    SafeTensorStream stream;
    std::string e = stream.Begin(path, shapes, metadata);
    if (!e.empty()) return e;
    for (const auto& kv : entries) {
        if (kv.second.Values.empty()) continue;
        e = stream.Append(kv.first, kv.second.Values.data(), (long long)kv.second.Values.size());
        if (!e.empty()) return e;
    }
    return stream.Finish();
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
