// json_min.h - a small strict JSON reader for safetensors headers and shard
// indexes: objects, arrays, strings (with escapes), numbers, true/false/null.
// Nesting is capped; any syntax error makes parse() return false.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace pdkjson {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool is_uint = false;
    uint64_t u = 0;
    std::string str;
    std::vector<Value> arr;
    std::vector<std::pair<std::string, Value>> obj;  // insertion order kept

    const Value* get(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

class Parser {
  public:
    Parser(const char* p, size_t n) : p_(p), end_(p + n) {}
    bool parse(Value& out) {
        if (!value(out, 0)) return false;
        ws();
        return p_ == end_;
    }

  private:
    static constexpr int kMaxDepth = 32;
    const char* p_;
    const char* end_;

    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
    }
    bool lit(const char* s) {
        const char* q = p_;
        while (*s) {
            if (q >= end_ || *q != *s) return false;
            ++q; ++s;
        }
        p_ = q;
        return true;
    }
    static void put_utf8(std::string& s, uint32_t c) {
        if (c < 0x80) s.push_back((char)c);
        else if (c < 0x800) { s.push_back((char)(0xC0 | (c >> 6))); s.push_back((char)(0x80 | (c & 0x3F))); }
        else if (c < 0x10000) {
            s.push_back((char)(0xE0 | (c >> 12))); s.push_back((char)(0x80 | ((c >> 6) & 0x3F)));
            s.push_back((char)(0x80 | (c & 0x3F)));
        } else {
            s.push_back((char)(0xF0 | (c >> 18))); s.push_back((char)(0x80 | ((c >> 12) & 0x3F)));
            s.push_back((char)(0x80 | ((c >> 6) & 0x3F))); s.push_back((char)(0x80 | (c & 0x3F)));
        }
    }
    bool hex4(uint32_t& v) {
        if (end_ - p_ < 4) return false;
        v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else return false;
        }
        return true;
    }
    bool string(std::string& s) {
        if (p_ >= end_ || *p_ != '"') return false;
        ++p_;
        while (p_ < end_) {
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return true;
            if (c < 0x20) return false;
            if (c != '\\') { s.push_back((char)c); continue; }
            if (p_ >= end_) return false;
            const char e = *p_++;
            switch (e) {
                case '"': s.push_back('"'); break;
                case '\\': s.push_back('\\'); break;
                case '/': s.push_back('/'); break;
                case 'b': s.push_back('\b'); break;
                case 'f': s.push_back('\f'); break;
                case 'n': s.push_back('\n'); break;
                case 'r': s.push_back('\r'); break;
                case 't': s.push_back('\t'); break;
                case 'u': {
                    uint32_t v;
                    if (!hex4(v)) return false;
                    if (v >= 0xD800 && v < 0xDC00) {  // surrogate pair
                        uint32_t lo;
                        if (end_ - p_ < 6 || p_[0] != '\\' || p_[1] != 'u') return false;
                        p_ += 2;
                        if (!hex4(lo) || lo < 0xDC00 || lo > 0xDFFF) return false;
                        v = 0x10000 + ((v - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (v >= 0xDC00 && v <= 0xDFFF) {
                        return false;
                    }
                    put_utf8(s, v);
                    break;
                }
                default: return false;
            }
        }
        return false;
    }
    bool number(Value& out) {
        const char* s = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') return false;
        bool integral = true;
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return false;
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return false;
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        const std::string tok(s, p_);
        out.kind = Value::Number;
        out.num = std::strtod(tok.c_str(), nullptr);
        if (integral && tok[0] != '-' && tok.size() <= 20) {
            uint64_t v = 0;
            bool ok = true;
            for (char c : tok) {
                const uint64_t d = (uint64_t)(c - '0');
                if (v > (UINT64_MAX - d) / 10) { ok = false; break; }
                v = v * 10 + d;
            }
            out.is_uint = ok;
            out.u = v;
        }
        return true;
    }
    bool value(Value& out, int depth) {
        if (depth > kMaxDepth) return false;
        ws();
        if (p_ >= end_) return false;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            out.kind = Value::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!string(key)) return false;
                ws();
                if (p_ >= end_ || *p_++ != ':') return false;
                Value v;
                if (!value(v, depth + 1)) return false;
                out.obj.emplace_back(std::move(key), std::move(v));
                ws();
                if (p_ >= end_) return false;
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == '}') { ++p_; return true; }
                return false;
            }
        }
        if (c == '[') {
            ++p_;
            out.kind = Value::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return true; }
            for (;;) {
                Value v;
                if (!value(v, depth + 1)) return false;
                out.arr.push_back(std::move(v));
                ws();
                if (p_ >= end_) return false;
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; return true; }
                return false;
            }
        }
        if (c == '"') { out.kind = Value::String; return string(out.str); }
        if (c == 't') { out.kind = Value::Bool; out.b = true; return lit("true"); }
        if (c == 'f') { out.kind = Value::Bool; out.b = false; return lit("false"); }
        if (c == 'n') { out.kind = Value::Null; return lit("null"); }
        return number(out);
    }
};

}  // namespace pdkjson
