// Tokenizer front-end of the token loop (text -> ids -> text).  Host code only.
//
//   * CharTokenizer: sorted unique characters of a text, or an explicit vocabulary
//     (src/tokenization/char_tokenizer.rs:34-84); encode drops unknown characters,
//     decode drops unknown ids (:95-107).
//   * BPETokenizer as loaded from its JSON file (src/tokenization/bpe_tokenizer.rs:224-247):
//     encode splits on Unicode white space, starts every word as single characters and
//     applies the merge rules in file order, each rule scanned left to right over the
//     word (:186-205, :250-267); a loaded tokenizer has no [UNK] id, so pieces missing
//     from the vocabulary are dropped.  decode joins the tokens with single spaces (:269-275).
#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "rg_internal.cuh"
#include "rg_json.h"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

struct rg_tokenizer {
    bool bpe = false;
    // char tokenizer
    std::unordered_map<uint32_t, uint32_t> char_to_id;
    std::unordered_map<uint32_t, uint32_t> id_to_char;
    // BPE
    std::unordered_map<std::string, uint32_t> token_to_id;
    std::unordered_map<uint32_t, std::string> id_to_token;
    std::vector<std::pair<std::string, std::string>> merges;
    size_t vocab = 0;
};

namespace {

// Decodes one UTF-8 scalar value; returns its byte length or 0 when the bytes are not valid UTF-8.
int utf8_next(const unsigned char* p, size_t n, uint32_t* cp) {
    if (n == 0) return 0;
    const unsigned c = p[0];
    if (c < 0x80) return *cp = c, 1;
    int len = 0;
    uint32_t v = 0, lo = 0;
    if ((c & 0xE0) == 0xC0) len = 2, v = c & 0x1F, lo = 0x80;
    else if ((c & 0xF0) == 0xE0) len = 3, v = c & 0x0F, lo = 0x800;
    else if ((c & 0xF8) == 0xF0) len = 4, v = c & 0x07, lo = 0x10000;
    else return 0;
    if ((size_t)len > n) return 0;
    for (int i = 1; i < len; i++) {
        if ((p[i] & 0xC0) != 0x80) return 0;
        v = (v << 6) | (p[i] & 0x3F);
    }
    if (v < lo || v > 0x10FFFF || (v >= 0xD800 && v < 0xE000)) return 0;
    *cp = v;
    return len;
}

void utf8_put(std::string& s, uint32_t c) {
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

// char::is_whitespace: the Unicode White_Space property, which str::split_whitespace splits on
bool is_space(uint32_t c) {
    return (c >= 0x09 && c <= 0x0D) || c == 0x20 || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
           c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}

rg_status decode_text(const char* text, size_t len, std::vector<uint32_t>* cps, std::vector<uint32_t>* offs) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(text);
    size_t i = 0;
    while (i < len) {
        uint32_t cp = 0;
        const int k = utf8_next(p + i, len - i, &cp);
        if (k == 0) return rg_fail(RG_ERR_INVALID_INPUT, "text is not valid UTF-8 at byte %zu", i);
        cps->push_back(cp);
        if (offs) offs->push_back((uint32_t)i);
        i += (size_t)k;
    }
    if (offs) offs->push_back((uint32_t)len);
    return RG_OK;
}

void bpe_word(const rg_tokenizer* t, const char* text, const std::vector<uint32_t>& offs, size_t a, size_t b, std::vector<uint32_t>* ids) {
    std::vector<std::string> tok;
    tok.reserve(b - a);
    for (size_t i = a; i < b; i++) tok.emplace_back(text + offs[i], offs[i + 1] - offs[i]);
    for (const auto& mr : t->merges) {
        if (tok.size() < 2) break;
        size_t i = 0;
        while (i + 1 < tok.size()) {
            if (tok[i] == mr.first && tok[i + 1] == mr.second) {
                tok[i] += mr.second;  // stays at i: the merged piece is compared with its new neighbour next
                tok.erase(tok.begin() + (long)i + 1);
            } else {
                i++;
            }
        }
    }
    for (const std::string& s : tok) {
        auto it = t->token_to_id.find(s);
        if (it != t->token_to_id.end()) ids->push_back(it->second);
    }
}

}  // namespace

extern "C" rg_status rg_tokenizer_char_from_text(const char* text, size_t len, rg_tokenizer** out) {
    if (!out || (!text && len)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    std::vector<uint32_t> cps;
    RG_TRY(decode_text(text, len, &cps, nullptr));
    std::sort(cps.begin(), cps.end());
    cps.erase(std::unique(cps.begin(), cps.end()), cps.end());
    rg_tokenizer* t = new rg_tokenizer();
    for (size_t i = 0; i < cps.size(); i++) t->char_to_id[cps[i]] = (uint32_t)i, t->id_to_char[(uint32_t)i] = cps[i];
    t->vocab = cps.size();
    *out = t;
    return RG_OK;
}

extern "C" rg_status rg_tokenizer_char_from_vocab(const uint32_t* codepoints, size_t n, rg_tokenizer** out) {
    if (!out || (!codepoints && n)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    rg_tokenizer* t = new rg_tokenizer();
    for (size_t i = 0; i < n; i++) {  // collect() into a HashMap: a repeated character keeps its last id
        t->char_to_id[codepoints[i]] = (uint32_t)i;
        t->id_to_char[(uint32_t)i] = codepoints[i];
    }
    t->vocab = n;
    *out = t;
    return RG_OK;
}

extern "C" rg_status rg_tokenizer_bpe_load(const char* path, rg_tokenizer** out) {
    if (!out || !path) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    std::string buf;
    {
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) return rg_fail(RG_ERR_IO, "cannot open %s: %s", path, strerror(errno));
        char tmp[1 << 16];
        ssize_t k;
        while ((k = ::read(fd, tmp, sizeof(tmp))) > 0) buf.append(tmp, (size_t)k);
        ::close(fd);
        if (k < 0) return rg_fail(RG_ERR_IO, "cannot read %s: %s", path, strerror(errno));
    }
    rg_json j;
    rg_json_parser ps(buf.data(), buf.size());
    if (!ps.parse(&j) || j.t != rg_json::OBJ) return rg_fail(RG_ERR_SERIALIZATION, "%s: %s", path, ps.err().empty() ? "not a JSON object" : ps.err().c_str());
    const rg_json* t2i = j.get("token_to_id");
    const rg_json* i2t = j.get("id_to_token");
    const rg_json* mg = j.get("merges");
    const rg_json* vs = j.get("vocab_size");
    uint64_t vocab = 0;
    if (!t2i || t2i->t != rg_json::OBJ || !i2t || i2t->t != rg_json::OBJ || !mg || (mg->t != rg_json::ARR) || !vs || !vs->as_index(&vocab))
        return rg_fail(RG_ERR_SERIALIZATION, "%s: expected token_to_id, id_to_token, merges, vocab_size", path);
    std::unique_ptr<rg_tokenizer> t(new rg_tokenizer());
    t->bpe = true;
    t->vocab = (size_t)vocab;
    for (const auto& kv : t2i->obj) {
        uint64_t id = 0;
        if (!kv.second.as_index(&id) || id > 0xffffffffull) return rg_fail(RG_ERR_SERIALIZATION, "%s: bad id of token `%s`", path, kv.first.c_str());
        t->token_to_id[kv.first] = (uint32_t)id;
    }
    for (const auto& kv : i2t->obj) {
        char* stop = nullptr;
        const unsigned long long id = strtoull(kv.first.c_str(), &stop, 10);
        if (kv.first.empty() || *stop != 0 || id > 0xffffffffull || kv.second.t != rg_json::STR)
            return rg_fail(RG_ERR_SERIALIZATION, "%s: bad id_to_token entry `%s`", path, kv.first.c_str());
        t->id_to_token[(uint32_t)id] = kv.second.str;
    }
    for (const rg_json& m : mg->arr) {
        if (m.t != rg_json::ARR || m.arr.size() != 2 || m.arr[0].t != rg_json::STR || m.arr[1].t != rg_json::STR)
            return rg_fail(RG_ERR_SERIALIZATION, "%s: a merge rule is not a pair of strings", path);
        t->merges.emplace_back(m.arr[0].str, m.arr[1].str);
    }
    *out = t.release();
    return RG_OK;
}

extern "C" rg_status rg_tokenizer_vocab_size(const rg_tokenizer* t, size_t* out) {
    if (!t || !out) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    *out = t->vocab;
    return RG_OK;
}

extern "C" rg_status rg_tokenizer_encode(const rg_tokenizer* t, const char* text, size_t len, uint32_t* ids_out, size_t cap,
                                         size_t* n_out) {
    if (!t || !n_out || (!text && len)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    std::vector<uint32_t> cps, offs, ids;
    RG_TRY(decode_text(text, len, &cps, &offs));
    if (!t->bpe) {
        for (uint32_t c : cps) {
            auto it = t->char_to_id.find(c);
            if (it != t->char_to_id.end()) ids.push_back(it->second);
        }
    } else {
        size_t i = 0;
        while (i < cps.size()) {
            while (i < cps.size() && is_space(cps[i])) i++;
            size_t e = i;
            while (e < cps.size() && !is_space(cps[e])) e++;
            if (e > i) bpe_word(t, text, offs, i, e, &ids);
            i = e;
        }
    }
    *n_out = ids.size();
    if (!ids_out) return RG_OK;  // size query
    if (cap < ids.size()) return rg_fail(RG_ERR_INVALID_INPUT, "ids_out holds %zu ids, %zu needed", cap, ids.size());
    if (!ids.empty()) memcpy(ids_out, ids.data(), ids.size() * sizeof(uint32_t));
    return RG_OK;
}

extern "C" rg_status rg_tokenizer_decode(const rg_tokenizer* t, const uint32_t* ids, size_t n, char* out, size_t cap, size_t* len_out) {
    if (!t || !len_out || (!ids && n)) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
    std::string s;
    if (!t->bpe) {
        for (size_t i = 0; i < n; i++) {
            auto it = t->id_to_char.find(ids[i]);
            if (it != t->id_to_char.end()) utf8_put(s, it->second);
        }
    } else {
        bool first = true;
        for (size_t i = 0; i < n; i++) {
            auto it = t->id_to_token.find(ids[i]);
            if (it == t->id_to_token.end()) continue;
            if (!first) s += ' ';
            s += it->second;
            first = false;
        }
    }
    *len_out = s.size();
    if (!out) return RG_OK;  // size query
    if (cap < s.size()) return rg_fail(RG_ERR_INVALID_INPUT, "out holds %zu bytes, %zu needed", cap, s.size());
    if (!s.empty()) memcpy(out, s.data(), s.size());
    return RG_OK;
}

extern "C" void rg_tokenizer_free(rg_tokenizer* t) { delete t; }
