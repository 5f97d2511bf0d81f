// Minimal JSON reader for the three host-side formats on either side of the token
// loop: the safetensors header and the ModelMetadata sidecar
// (src/serialization/safetensors_format.rs:89-138, src/serialization/mod.rs:28-37),
// the legacy weights JSON [{shape, data}] (src/wasm_api.rs:166-199,
// src/serialization/mod.rs:52-74) and the tokenizer files
// (src/tokenization/bpe_tokenizer.rs:207-247).
//
// Arrays that start with a number are read on a fast path into a float vector (the
// `data` arrays of the legacy format hold every weight of the model as text); the first
// 64 numbers are also kept as doubles so that shapes and byte offsets stay exact.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

struct rg_json {
    enum kind { NUL, BOOL, NUM, STR, ARR, OBJ, NUMS } t = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<rg_json> arr;
    std::vector<std::pair<std::string, rg_json>> obj;
    std::vector<float> nums;
    std::vector<double> head;  // first 64 entries of nums, exact

    const rg_json* get(const char* key) const {
        if (t != OBJ) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_number_array() const { return t == NUMS || (t == ARR && arr.empty()); }
    size_t count() const { return t == NUMS ? nums.size() : arr.size(); }
    // element i of a numeric array as an exact integer (only the first 64 are exact)
    bool index_at(size_t i, uint64_t* out) const {
        if (t != NUMS || i >= head.size()) return false;
        const double d = head[i];
        if (d < 0 || d != (double)(uint64_t)d) return false;
        *out = (uint64_t)d;
        return true;
    }
    bool as_index(uint64_t* out) const {
        if (t != NUM || num < 0 || num != (double)(uint64_t)num) return false;
        *out = (uint64_t)num;
        return true;
    }
};

class rg_json_parser {
   public:
    rg_json_parser(const char* p, size_t n) : p_(p), begin_(p), end_(p + n) {}
    // false on malformed input; err() then says where
    bool parse(rg_json* out) {
        if (!value(out, 0)) return false;
        ws();
        if (p_ != end_) return fail("trailing characters");
        return true;
    }
    const std::string& err() const { return err_; }

   private:
    const char* p_;
    const char* begin_;
    const char* end_;
    std::string err_;

    bool fail(const char* what) {
        if (err_.empty()) err_ = std::string(what) + " at byte " + std::to_string((size_t)(p_ - begin_));
        return false;
    }

    void ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) p_++;
    }
    bool lit(const char* s) {
        const size_t n = strlen(s);
        if ((size_t)(end_ - p_) < n || memcmp(p_, s, n) != 0) return fail("bad literal");
        p_ += n;
        return true;
    }
    static void utf8(std::string& s, uint32_t c) {
        if (c < 0x80) {
            s += (char)c;
        } else if (c < 0x800) {
            s += (char)(0xC0 | (c >> 6)), s += (char)(0x80 | (c & 0x3F));
        } else if (c < 0x10000) {
            s += (char)(0xE0 | (c >> 12)), s += (char)(0x80 | ((c >> 6) & 0x3F)), s += (char)(0x80 | (c & 0x3F));
        } else {
            s += (char)(0xF0 | (c >> 18)), s += (char)(0x80 | ((c >> 12) & 0x3F)), s += (char)(0x80 | ((c >> 6) & 0x3F)),
                s += (char)(0x80 | (c & 0x3F));
        }
    }
    bool hex4(uint32_t* out) {
        if (end_ - p_ < 4) return fail("short \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; i++) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else return fail("bad \\u escape");
        }
        *out = v;
        return true;
    }
    bool string(std::string* s) {
        if (p_ >= end_ || *p_ != '"') return fail("expected string");
        p_++;
        s->clear();
        while (p_ < end_) {
            const char c = *p_++;
            if (c == '"') return true;
            if (c != '\\') {
                *s += c;
                continue;
            }
            if (p_ >= end_) break;
            const char e = *p_++;
            switch (e) {
                case '"': *s += '"'; break;
                case '\\': *s += '\\'; break;
                case '/': *s += '/'; break;
                case 'b': *s += '\b'; break;
                case 'f': *s += '\f'; break;
                case 'n': *s += '\n'; break;
                case 'r': *s += '\r'; break;
                case 't': *s += '\t'; break;
                case 'u': {
                    uint32_t c1;
                    if (!hex4(&c1)) return false;
                    if (c1 >= 0xD800 && c1 < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        uint32_t c2;
                        if (!hex4(&c2)) return false;
                        c1 = 0x10000 + ((c1 - 0xD800) << 10) + (c2 - 0xDC00);
                    }
                    utf8(*s, c1);
                    break;
                }
                default: return fail("bad escape");
            }
        }
        return fail("unterminated string");
    }
    bool number(double* out) {
        // strtod needs a terminated buffer: numbers are short, copy the candidate span
        char buf[64];
        size_t n = 0;
        while (p_ + n < end_ && n < sizeof(buf) - 1) {
            const char c = p_[n];
            if ((c >= '0' && c <= '9') || c == '-' || c == '+' || c == '.' || c == 'e' || c == 'E') n++;
            else break;
        }
        if (n == 0) return fail("expected number");
        memcpy(buf, p_, n);
        buf[n] = 0;
        char* stop = nullptr;
        *out = strtod(buf, &stop);
        if (stop != buf + n) return fail("bad number");
        p_ += n;
        return true;
    }
    bool value(rg_json* v, int depth) {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (p_ >= end_) return fail("unexpected end");
        const char c = *p_;
        if (c == '{') {
            p_++;
            v->t = rg_json::OBJ;
            ws();
            if (p_ < end_ && *p_ == '}') return p_++, true;
            for (;;) {
                ws();
                std::string key;
                if (!string(&key)) return false;
                ws();
                if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
                p_++;
                v->obj.emplace_back(std::move(key), rg_json());
                if (!value(&v->obj.back().second, depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') {
                    p_++;
                    continue;
                }
                if (p_ < end_ && *p_ == '}') return p_++, true;
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            p_++;
            ws();
            if (p_ < end_ && *p_ == ']') return v->t = rg_json::ARR, p_++, true;
            if (p_ < end_ && (*p_ == '-' || (*p_ >= '0' && *p_ <= '9'))) {
                v->t = rg_json::NUMS;
                for (;;) {
                    ws();
                    double d;
                    if (!number(&d)) return false;
                    v->nums.push_back((float)d);
                    if (v->head.size() < 64) v->head.push_back(d);
                    ws();
                    if (p_ < end_ && *p_ == ',') {
                        p_++;
                        continue;
                    }
                    if (p_ < end_ && *p_ == ']') return p_++, true;
                    return fail("expected ',' or ']' in a number array");
                }
            }
            v->t = rg_json::ARR;
            for (;;) {
                v->arr.emplace_back();
                if (!value(&v->arr.back(), depth + 1)) return false;
                ws();
                if (p_ < end_ && *p_ == ',') {
                    p_++;
                    continue;
                }
                if (p_ < end_ && *p_ == ']') return p_++, true;
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') return v->t = rg_json::STR, string(&v->str);
        if (c == 't') return v->t = rg_json::BOOL, v->b = true, lit("true");
        if (c == 'f') return v->t = rg_json::BOOL, v->b = false, lit("false");
        if (c == 'n') return v->t = rg_json::NUL, lit("null");
        v->t = rg_json::NUM;
        return number(&v->num);
    }
};
