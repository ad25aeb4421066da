// A small JSON value, parser and writer: enough for safetensors headers and the
// optimizer configuration stored in checkpoint metadata. Objects keep their keys
// sorted, which is also what Go's encoding/json produces for maps; struct-ordered
// objects are written by hand where the reference's field order matters.
#ifndef GG_JSON_MIN_HPP
#define GG_JSON_MIN_HPP

#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace ggjson {

struct Value;
using Object = std::map<std::string, Value>;
using Array = std::vector<Value>;

struct Value {
    enum Kind { Null, Bool, Number, String, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    std::string raw;  // number text as written (keeps integers exact) or string payload
    std::shared_ptr<Array> arr;
    std::shared_ptr<Object> obj;

    bool is(Kind k) const { return kind == k; }
    const Value* get(const std::string& key) const {
        if (kind != Obj) return nullptr;
        auto it = obj->find(key);
        return it == obj->end() ? nullptr : &it->second;
    }
};

// Go's encoding/json escapes <, >, & and U+2028/2029 besides the mandatory ones.
inline std::string quote(const std::string& s) {
    std::string o = "\"";
    for (size_t i = 0; i < s.size(); i++) {
        unsigned char c = (unsigned char)s[i];
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            case '<': o += "\\u003c"; break;
            case '>': o += "\\u003e"; break;
            case '&': o += "\\u0026"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof buf, "\\u%04x", c);
                    o += buf;
                } else if (c == 0xE2 && i + 2 < s.size() && (unsigned char)s[i + 1] == 0x80 &&
                           ((unsigned char)s[i + 2] == 0xA8 || (unsigned char)s[i + 2] == 0xA9)) {
                    o += (unsigned char)s[i + 2] == 0xA8 ? "\\u2028" : "\\u2029";
                    i += 2;
                } else {
                    o += (char)c;
                }
        }
    }
    return o + "\"";
}

// Shortest decimal text that parses back to the same binary32 / binary64 value, in the
// layout Go's encoding/json uses ('e' form below 1e-6 and from 1e21 on, exponent
// without padding zeros).
inline std::string number_text(double v, bool single) {
    if (v == 0) return std::signbit(v) ? "-0" : "0";
    char buf[64];
    double a = std::fabs(v);
    bool exp_form = a < 1e-6 || a >= 1e21;
    for (int prec = 1; prec <= 17; prec++) {
        snprintf(buf, sizeof buf, "%.*e", prec - 1, v);
        bool same = single ? (float)strtod(buf, nullptr) == (float)v : strtod(buf, nullptr) == v;
        if (!same) continue;
        if (!exp_form) {
            // re-render the same digits in positional form
            int e10 = atoi(strchr(buf, 'e') + 1);
            int decimals = prec - 1 - e10;
            if (decimals < 0) decimals = 0;
            snprintf(buf, sizeof buf, "%.*f", decimals, v);
            return buf;
        }
        std::string s(buf);
        size_t e = s.find('e');
        std::string mant = s.substr(0, e), ex = s.substr(e + 1);
        char sign = ex[0];
        size_t k = 1;
        while (k + 1 < ex.size() && ex[k] == '0') k++;
        std::string digits = ex.substr(k);
        return mant + "e" + (sign == '-' ? "-" : "+") + (digits.size() < 2 ? "0" + digits : digits);
    }
    snprintf(buf, sizeof buf, "%.17g", v);
    return buf;
}

class Parser {
   public:
    explicit Parser(const std::string& text) : s_(text) {}
    bool parse(Value* out, std::string* err) {
        skip();
        if (!value(out)) {
            if (err) *err = err_.empty() ? "invalid JSON" : err_;
            return false;
        }
        skip();
        if (p_ != s_.size()) {
            if (err) *err = "trailing characters after JSON value";
            return false;
        }
        return true;
    }

   private:
    const std::string& s_;
    size_t p_ = 0;
    std::string err_;
    int depth_ = 0;

    void skip() {
        while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) p_++;
    }
    bool lit(const char* w) {
        size_t n = strlen(w);
        if (s_.compare(p_, n, w) == 0) {
            p_ += n;
            return true;
        }
        return false;
    }
    bool value(Value* v) {
        if (++depth_ > 64) {
            err_ = "JSON nested too deeply";
            return false;
        }
        bool ok = value_inner(v);
        depth_--;
        return ok;
    }
    bool value_inner(Value* v) {
        if (p_ >= s_.size()) return false;
        char c = s_[p_];
        if (c == '{') return object(v);
        if (c == '[') return array(v);
        if (c == '"') {
            v->kind = Value::String;
            return string(&v->raw);
        }
        if (lit("true")) {
            v->kind = Value::Bool;
            v->b = true;
            return true;
        }
        if (lit("false")) {
            v->kind = Value::Bool;
            v->b = false;
            return true;
        }
        if (lit("null")) {
            v->kind = Value::Null;
            return true;
        }
        size_t start = p_;
        if (p_ < s_.size() && s_[p_] == '-') p_++;
        while (p_ < s_.size() && (isdigit((unsigned char)s_[p_]) || s_[p_] == '.' || s_[p_] == 'e' || s_[p_] == 'E' ||
                                  s_[p_] == '+' || s_[p_] == '-'))
            p_++;
        if (p_ == start) return false;
        v->kind = Value::Number;
        v->raw = s_.substr(start, p_ - start);
        char* end = nullptr;
        v->num = strtod(v->raw.c_str(), &end);
        return end && *end == 0;
    }
    bool string(std::string* out) {
        p_++;  // opening quote
        out->clear();
        while (p_ < s_.size()) {
            char c = s_[p_++];
            if (c == '"') return true;
            if (c != '\\') {
                *out += c;
                continue;
            }
            if (p_ >= s_.size()) return false;
            char e = s_[p_++];
            switch (e) {
                case 'n': *out += '\n'; break;
                case 't': *out += '\t'; break;
                case 'r': *out += '\r'; break;
                case 'b': *out += '\b'; break;
                case 'f': *out += '\f'; break;
                case 'u': {
                    if (p_ + 4 > s_.size()) return false;
                    unsigned cp = (unsigned)strtoul(s_.substr(p_, 4).c_str(), nullptr, 16);
                    p_ += 4;
                    if (cp < 0x80) {
                        *out += (char)cp;
                    } else if (cp < 0x800) {
                        *out += (char)(0xC0 | (cp >> 6));
                        *out += (char)(0x80 | (cp & 0x3F));
                    } else {
                        *out += (char)(0xE0 | (cp >> 12));
                        *out += (char)(0x80 | ((cp >> 6) & 0x3F));
                        *out += (char)(0x80 | (cp & 0x3F));
                    }
                    break;
                }
                default: *out += e;
            }
        }
        return false;
    }
    bool array(Value* v) {
        v->kind = Value::Arr;
        v->arr = std::make_shared<Array>();
        p_++;
        skip();
        if (p_ < s_.size() && s_[p_] == ']') {
            p_++;
            return true;
        }
        for (;;) {
            Value item;
            skip();
            if (!value(&item)) return false;
            v->arr->push_back(item);
            skip();
            if (p_ < s_.size() && s_[p_] == ',') {
                p_++;
                continue;
            }
            if (p_ < s_.size() && s_[p_] == ']') {
                p_++;
                return true;
            }
            return false;
        }
    }
    bool object(Value* v) {
        v->kind = Value::Obj;
        v->obj = std::make_shared<Object>();
        p_++;
        skip();
        if (p_ < s_.size() && s_[p_] == '}') {
            p_++;
            return true;
        }
        for (;;) {
            skip();
            if (p_ >= s_.size() || s_[p_] != '"') return false;
            std::string key;
            if (!string(&key)) return false;
            skip();
            if (p_ >= s_.size() || s_[p_] != ':') return false;
            p_++;
            skip();
            Value item;
            if (!value(&item)) return false;
            if (v->obj->count(key)) {
                err_ = "duplicate key " + key;
                return false;
            }
            (*v->obj)[key] = item;
            skip();
            if (p_ < s_.size() && s_[p_] == ',') {
                p_++;
                continue;
            }
            if (p_ < s_.size() && s_[p_] == '}') {
                p_++;
                return true;
            }
            return false;
        }
    }
};

}  // namespace ggjson
#endif
