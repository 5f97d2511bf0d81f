// Weight ingest from disk: the step before the token loop.  Host code only; the
// tensors end up on the device through the same upload path as rg_gpt_load_params.
//
//   * safetensors, F32 only like the reference's reader
//     (src/serialization/safetensors_format.rs:89-138), with the ModelMetadata
//     sidecar `<file>.json` it writes next to the weights (:76-81,
//     src/serialization/mod.rs:28-37).  The file is memory-mapped; tensors that need
//     no re-arrangement are uploaded straight from the mapping.
//   * the legacy JSON of WasmGptTrainer::loadWeightsFromJson: an array of
//     {shape, data} in parameters() order (src/wasm_api.rs:166-199), or a
//     JsonCheckpoint object holding it under "weights" (src/serialization/mod.rs:52-74).
//   * tensor names: the descriptive names of the crate's examples
//     (examples/serialization_demo.rs:24-101, examples/train_gpt_e2e.rs:146-160) or
//     the Hugging Face GPT-2 names of the crate's loader
//     (src/models/hf_loader.rs:256-276), whose fused c_attn [D, 3D] is split into
//     q | k | v and whose tied LM head is the transposed token table
//     (the reference stops at the name map: :290-296 "Weight copying not yet implemented").
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <list>
#include <map>
#include <memory>

#include "rg_gpt.h"

#include <exception>
#include "rg_json.h"

namespace {

struct mapped_file {
    const unsigned char* p = nullptr;
    size_t n = 0;
    ~mapped_file() {
        if (p && n) munmap(const_cast<unsigned char*>(p), n);
    }
    rg_status open(const char* path) {
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) return rg_fail(RG_ERR_IO, "cannot open %s: %s", path, strerror(errno));
        struct stat st;
        if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
            ::close(fd);
            return rg_fail(RG_ERR_IO, "%s is not a regular file", path);
        }
        n = (size_t)st.st_size;
        if (n > 0) {
            void* q = mmap(nullptr, n, PROT_READ, MAP_PRIVATE, fd, 0);
            if (q == MAP_FAILED) {
                ::close(fd);
                n = 0;
                return rg_fail(RG_ERR_IO, "cannot map %s: %s", path, strerror(errno));
            }
            p = static_cast<const unsigned char*>(q);
        }
        ::close(fd);
        return RG_OK;
    }
};

struct host_tensor {
    const float* data = nullptr;
    std::vector<size_t> shape;
    size_t count() const {
        size_t c = 1;
        for (size_t d : shape) c *= d;
        return c;
    }
};

rg_status parse_json_file(const mapped_file& f, const char* path, rg_json* out) {
    rg_json_parser ps(reinterpret_cast<const char*>(f.p), f.n);
    if (!ps.parse(out)) return rg_fail(RG_ERR_SERIALIZATION, "%s: %s", path, ps.err().c_str());
    return RG_OK;
}

rg_status metadata_from_json(const rg_json& j, const char* path, rg_gpt_config* cfg) {
    struct field {
        const char* key;
        size_t* dst;
    } fields[] = {{"vocab_size", &cfg->vocab_size},
                  {"embedding_dim", &cfg->embedding_dim},
                  {"num_layers", &cfg->num_layers},
                  {"num_heads", &cfg->num_heads},
                  {"block_size", &cfg->block_size}};
    for (const field& f : fields) {
        const rg_json* v = j.get(f.key);
        uint64_t x = 0;
        if (!v || !v->as_index(&x) || x == 0 || x > 0x7fffffffull)
            return rg_fail(RG_ERR_SERIALIZATION, "%s: missing or invalid field `%s`", path, f.key);
        *f.dst = (size_t)x;
    }
    return RG_OK;
}

// ---- safetensors --------------------------------------------------------------------------------------------
struct st_file {
    mapped_file map;
    std::map<std::string, host_tensor> tensors;
    std::list<std::vector<float>> copies;

    rg_status open(const char* path) {
        RG_TRY(map.open(path));
        if (map.n < 8) return rg_fail(RG_ERR_SERIALIZATION, "%s: shorter than a safetensors header", path);
        uint64_t hlen = 0;
        for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | map.p[i];
        if (hlen > map.n - 8) return rg_fail(RG_ERR_SERIALIZATION, "%s: header length %llu exceeds the file", path, (unsigned long long)hlen);
        rg_json hdr;
        rg_json_parser ps(reinterpret_cast<const char*>(map.p + 8), (size_t)hlen);
        if (!ps.parse(&hdr) || hdr.t != rg_json::OBJ)
            return rg_fail(RG_ERR_SERIALIZATION, "%s: header is not a JSON object (%s)", path, ps.err().c_str());
        const unsigned char* base = map.p + 8 + hlen;
        const size_t avail = map.n - 8 - (size_t)hlen;
        for (const auto& kv : hdr.obj) {
            if (kv.first == "__metadata__") continue;
            const rg_json& e = kv.second;
            const rg_json* dt = e.get("dtype");
            const rg_json* sh = e.get("shape");
            const rg_json* off = e.get("data_offsets");
            if (!dt || dt->t != rg_json::STR || !sh || !sh->is_number_array() || !off || off->t != rg_json::NUMS || off->count() != 2)
                return rg_fail(RG_ERR_SERIALIZATION, "%s: malformed entry `%s`", path, kv.first.c_str());
            if (dt->str != "F32")  // the reference reader accepts nothing else (safetensors_format.rs:111-116)
                return rg_fail(RG_ERR_SERIALIZATION, "%s: tensor `%s`: Expected F32 dtype, got %s", path, kv.first.c_str(), dt->str.c_str());
            host_tensor t;
            uint64_t elems = 1;  // checked product: a crafted shape must not wrap around to a small byte count
            for (size_t i = 0; i < sh->count(); i++) {
                uint64_t d = 0;
                if (!sh->index_at(i, &d)) return rg_fail(RG_ERR_SERIALIZATION, "%s: bad shape of `%s`", path, kv.first.c_str());
                if (d != 0 && elems > (uint64_t)avail / d)
                    return rg_fail(RG_ERR_SERIALIZATION, "%s: shape of `%s` describes more data than the file holds", path, kv.first.c_str());
                elems *= d;
                t.shape.push_back((size_t)d);
            }
            uint64_t b = 0, en = 0;
            if (elems > (uint64_t)avail / 4 || !off->index_at(0, &b) || !off->index_at(1, &en) || en < b || en > avail || en - b != elems * 4)
                return rg_fail(RG_ERR_SERIALIZATION, "%s: data_offsets of `%s` do not match its shape or the file", path, kv.first.c_str());
            if (((uintptr_t)(base + b)) & 3) {  // header length not a multiple of 4: floats cannot be read in place
                copies.emplace_back(t.count());
                memcpy(copies.back().data(), base + b, t.count() * 4);
                t.data = copies.back().data();
            } else {
                t.data = reinterpret_cast<const float*>(base + b);
            }
            tensors.emplace(kv.first, std::move(t));
        }
        return RG_OK;
    }
    const host_tensor* find(const std::string& name) const {
        auto it = tensors.find(name);
        return it == tensors.end() ? nullptr : &it->second;
    }
};

// One parameters() slot being assembled: either a view into the mapping or an owned re-arranged copy.
struct slot {
    const float* data = nullptr;
    size_t shape[2] = {0, 0};
    std::unique_ptr<std::vector<float>> owned;
};

class assembler {
   public:
    assembler(const rg_gpt* m, const st_file& f, const char* path) : m_(m), f_(f), path_(path) {}

    // a [r, c] matrix stored under `name`; vectors may be stored as [c] or [1, c]
    rg_status view(slot& s, const std::string& name, size_t r, size_t c, bool allow_more_rows = false) {
        const host_tensor* t = f_.find(name);
        if (!t) return rg_fail(RG_ERR_IO, "%s: Missing required weight: %s", path_, name.c_str());
        RG_TRY(check(*t, name, r, c, allow_more_rows));
        s.data = t->data, s.shape[0] = r, s.shape[1] = c;
        return RG_OK;
    }
    // like view(); a missing tensor becomes a constant (biases the example models never had, the identity final LayerNorm)
    rg_status view_or(slot& s, const std::string& name, size_t r, size_t c, float fill) {
        if (f_.find(name)) return view(s, name, r, c);
        s.owned.reset(new std::vector<float>(r * c, fill));
        s.data = s.owned->data(), s.shape[0] = r, s.shape[1] = c;
        return RG_OK;
    }
    // columns [c0, c0 + c) of a [r, ctot] matrix (a third of a fused qkv projection)
    rg_status columns(slot& s, const std::string& name, size_t r, size_t ctot, size_t c0, size_t c, bool optional = false) {
        const host_tensor* t = f_.find(name);
        if (!t) {
            if (!optional) return rg_fail(RG_ERR_IO, "%s: Missing required weight: %s", path_, name.c_str());
            s.owned.reset(new std::vector<float>(r * c, 0.f));
        } else {
            RG_TRY(check(*t, name, r, ctot, false));
            s.owned.reset(new std::vector<float>(r * c));
            for (size_t i = 0; i < r; i++) memcpy(s.owned->data() + i * c, t->data + i * ctot + c0, c * sizeof(float));
        }
        s.data = s.owned->data(), s.shape[0] = r, s.shape[1] = c;
        return RG_OK;
    }
    // the transpose of a [c, r] matrix (tied LM head: token table [V, D] -> [D, V])
    rg_status transposed(slot& s, const std::string& name, size_t r, size_t c) {
        const host_tensor* t = f_.find(name);
        if (!t) return rg_fail(RG_ERR_IO, "%s: Missing required weight: %s", path_, name.c_str());
        RG_TRY(check(*t, name, c, r, false));
        s.owned.reset(new std::vector<float>(r * c));
        float* o = s.owned->data();
        constexpr size_t TB = 32;  // blocked so that both sides stay in cache
        for (size_t i0 = 0; i0 < c; i0 += TB)
            for (size_t j0 = 0; j0 < r; j0 += TB)
                for (size_t i = i0; i < std::min(c, i0 + TB); i++)
                    for (size_t j = j0; j < std::min(r, j0 + TB); j++) o[j * c + i] = t->data[i * r + j];
        s.data = o, s.shape[0] = r, s.shape[1] = c;
        return RG_OK;
    }
    bool has(const std::string& name) const { return f_.find(name) != nullptr; }

   private:
    const rg_gpt* m_;
    const st_file& f_;
    const char* path_;

    rg_status check(const host_tensor& t, const std::string& name, size_t r, size_t c, bool allow_more_rows) {
        bool ok = false;
        if (t.shape.size() == 2) ok = t.shape[1] == c && (t.shape[0] == r || (allow_more_rows && t.shape[0] >= r));
        if (t.shape.size() == 1 && r == 1) ok = t.shape[0] == c;
        if (!ok) {
            std::string got = "[";
            for (size_t i = 0; i < t.shape.size(); i++) got += (i ? ", " : "") + std::to_string(t.shape[i]);
            got += "]";
            return rg_fail(RG_ERR_SHAPE, "%s: Mismatch in tensor shape during loading: `%s` is %s, expected [%zu, %zu]", path_,
                           name.c_str(), got.c_str(), r, c);
        }
        return RG_OK;
    }
};

rg_status assemble_rusty(const rg_gpt* m, assembler& a, std::vector<slot>& s) {
    const size_t D = m->D, F = m->F, V = m->V, C = m->C;
    RG_TRY(a.view(s[0], "token_embedding.weight", V, D));
    RG_TRY(a.view(s[1], "position_embedding.weight", C, D, true));
    for (int l = 0; l < m->L; l++) {
        slot* p = s.data() + 2 + 16 * l;
        const std::string pre = "layer_" + std::to_string(l) + ".";
        static const char* qkv[3] = {"q", "k", "v"};
        const bool fused = !a.has(pre + "attn.q.weight");  // train_gpt_e2e.rs keeps one [D, 3D] projection
        for (int j = 0; j < 3; j++) {
            if (fused) {
                RG_TRY(a.columns(p[2 * j], pre + "attn.qkv.weight", D, 3 * D, j * D, D));
                RG_TRY(a.columns(p[2 * j + 1], pre + "attn.qkv.bias", 1, 3 * D, j * D, D, true));
            } else {
                RG_TRY(a.view(p[2 * j], pre + "attn." + qkv[j] + ".weight", D, D));
                RG_TRY(a.view_or(p[2 * j + 1], pre + "attn." + qkv[j] + ".bias", 1, D, 0.f));
            }
        }
        const std::string o = a.has(pre + "attn.out_proj.weight") ? "attn.out_proj" : "attn.proj";
        RG_TRY(a.view(p[6], pre + o + ".weight", D, D));
        RG_TRY(a.view_or(p[7], pre + o + ".bias", 1, D, 0.f));
        RG_TRY(a.view_or(p[8], pre + "ln1.gamma", 1, D, 1.f));
        RG_TRY(a.view_or(p[9], pre + "ln1.beta", 1, D, 0.f));
        RG_TRY(a.view(p[10], pre + "ffn.fc1.weight", D, F));
        RG_TRY(a.view_or(p[11], pre + "ffn.fc1.bias", 1, F, 0.f));
        RG_TRY(a.view(p[12], pre + "ffn.fc2.weight", F, D));
        RG_TRY(a.view_or(p[13], pre + "ffn.fc2.bias", 1, D, 0.f));
        RG_TRY(a.view_or(p[14], pre + "ln2.gamma", 1, D, 1.f));
        RG_TRY(a.view_or(p[15], pre + "ln2.beta", 1, D, 0.f));
    }
    const size_t n = s.size();
    RG_TRY(a.view_or(s[n - 4], "ln_f.gamma", 1, D, 1.f));
    RG_TRY(a.view_or(s[n - 3], "ln_f.beta", 1, D, 0.f));
    RG_TRY(a.view(s[n - 2], "output_projection.weight", D, V));
    RG_TRY(a.view_or(s[n - 1], "output_projection.bias", 1, V, 0.f));
    return RG_OK;
}

rg_status assemble_hf(const rg_gpt* m, assembler& a, std::vector<slot>& s) {
    const size_t D = m->D, F = m->F, V = m->V, C = m->C;
    const std::string r = a.has("transformer.wte.weight") ? "transformer." : "";
    RG_TRY(a.view(s[0], r + "wte.weight", V, D));
    RG_TRY(a.view(s[1], r + "wpe.weight", C, D, true));
    for (int l = 0; l < m->L; l++) {
        slot* p = s.data() + 2 + 16 * l;
        const std::string pre = r + "h." + std::to_string(l) + ".";
        for (int j = 0; j < 3; j++) {  // c_attn: [D, 3D] = q | k | v, bias [3D]
            RG_TRY(a.columns(p[2 * j], pre + "attn.c_attn.weight", D, 3 * D, j * D, D));
            RG_TRY(a.columns(p[2 * j + 1], pre + "attn.c_attn.bias", 1, 3 * D, j * D, D));
        }
        RG_TRY(a.view(p[6], pre + "attn.c_proj.weight", D, D));
        RG_TRY(a.view(p[7], pre + "attn.c_proj.bias", 1, D));
        RG_TRY(a.view(p[8], pre + "ln_1.weight", 1, D));
        RG_TRY(a.view(p[9], pre + "ln_1.bias", 1, D));
        RG_TRY(a.view(p[10], pre + "mlp.c_fc.weight", D, F));
        RG_TRY(a.view(p[11], pre + "mlp.c_fc.bias", 1, F));
        RG_TRY(a.view(p[12], pre + "mlp.c_proj.weight", F, D));
        RG_TRY(a.view(p[13], pre + "mlp.c_proj.bias", 1, D));
        RG_TRY(a.view(p[14], pre + "ln_2.weight", 1, D));
        RG_TRY(a.view(p[15], pre + "ln_2.bias", 1, D));
    }
    const size_t n = s.size();
    RG_TRY(a.view(s[n - 4], r + "ln_f.weight", 1, D));
    RG_TRY(a.view(s[n - 3], r + "ln_f.bias", 1, D));
    // GPT-2 ties the LM head to the token table: logits = x . wte^T, no bias
    RG_TRY(a.transposed(s[n - 2], a.has("lm_head.weight") ? std::string("lm_head.weight") : r + "wte.weight", D, V));
    s[n - 1].owned.reset(new std::vector<float>(V, 0.f));
    s[n - 1].data = s[n - 1].owned->data(), s[n - 1].shape[0] = 1, s[n - 1].shape[1] = V;
    return RG_OK;
}

rg_status load_slots(rg_gpt* m, const std::vector<slot>& s) {
    std::vector<const float*> data(s.size());
    std::vector<const size_t*> shapes(s.size());
    std::vector<int> ndims(s.size(), 2);
    for (size_t i = 0; i < s.size(); i++) data[i] = s[i].data, shapes[i] = s[i].shape;
    return rg_gpt_load_params(m, data.data(), shapes.data(), ndims.data(), (int)s.size());
}

}  // namespace

extern "C" rg_status rg_model_metadata_read(const char* path, rg_gpt_config* cfg) {
    try {
        if (!path || !cfg) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
        mapped_file f;
        RG_TRY(f.open(path));
        rg_json j;
        RG_TRY(parse_json_file(f, path, &j));
        const rg_json* meta = j.get("metadata");  // a JsonCheckpoint carries it one level down
        return metadata_from_json(meta ? *meta : j, path, cfg);
    } catch (const std::exception& e) {
        return rg_fail(RG_ERR_SERIALIZATION, "%s: %s", path ? path : "(null)", e.what());
    }
}

extern "C" rg_status rg_gpt_load_safetensors(rg_gpt* m, const char* path, int names) {
    try {
        if (!m || !path) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
        if (names != RG_NAMES_AUTO && names != RG_NAMES_RUSTY && names != RG_NAMES_HF_GPT2)
            return rg_fail(RG_ERR_INVALID_INPUT, "unknown naming scheme %d", names);
        st_file f;
        RG_TRY(f.open(path));
        if (names == RG_NAMES_AUTO)
            names = (f.find("wte.weight") || f.find("transformer.wte.weight")) ? RG_NAMES_HF_GPT2 : RG_NAMES_RUSTY;
        std::vector<slot> s((size_t)rg_gpt_num_params(m));
        assembler a(m, f, path);
        RG_TRY(names == RG_NAMES_HF_GPT2 ? assemble_hf(m, a, s) : assemble_rusty(m, a, s));
        return load_slots(m, s);
    } catch (const std::exception& e) {
        return rg_fail(RG_ERR_SERIALIZATION, "%s: %s", path ? path : "(null)", e.what());
    }
}

extern "C" rg_status rg_gpt_load_json(rg_gpt* m, const char* path) {
    try {
        if (!m || !path) return rg_fail(RG_ERR_INVALID_INPUT, "NULL argument");
        mapped_file f;
        RG_TRY(f.open(path));
        rg_json j;
        RG_TRY(parse_json_file(f, path, &j));
        const rg_json* w = j.t == rg_json::OBJ ? j.get("weights") : &j;
        if (!w || w->t != rg_json::ARR) return rg_fail(RG_ERR_SERIALIZATION, "%s: expected an array of {shape, data}", path);
        const int want = rg_gpt_num_params(m);
        if ((int)w->arr.size() != want)
            return rg_fail(RG_ERR_SHAPE, "Mismatch in number of parameter tensors during loading: got %zu, model has %d", w->arr.size(), want);
        std::vector<slot> s((size_t)want);
        for (int i = 0; i < want; i++) {
            const rg_json* sh = w->arr[i].get("shape");
            const rg_json* da = w->arr[i].get("data");
            if (!sh || !sh->is_number_array() || !da || !da->is_number_array())
                return rg_fail(RG_ERR_SERIALIZATION, "%s: tensor %d lacks `shape` or `data`", path, i);
            size_t want_shape[2];
            rg_gpt_param_shape(m, i, want_shape);
            uint64_t d0 = 0, d1 = 0;
            if (sh->count() != 2 || !sh->index_at(0, &d0) || !sh->index_at(1, &d1) || d0 != want_shape[0] || d1 != want_shape[1])
                return rg_fail(RG_ERR_SHAPE, "Mismatch in tensor shape during loading: parameter %d expected [%zu, %zu]", i, want_shape[0],
                               want_shape[1]);
            if (da->count() != d0 * d1)  // Array::from_shape_vec fails there (src/wasm_api.rs:193-194)
                return rg_fail(RG_ERR_SHAPE, "%s: tensor %d holds %zu values for shape [%llu, %llu]", path, i, da->count(),
                               (unsigned long long)d0, (unsigned long long)d1);
            s[i].data = da->nums.data(), s[i].shape[0] = (size_t)d0, s[i].shape[1] = (size_t)d1;
        }
        return load_slots(m, s);
    } catch (const std::exception& e) {
        return rg_fail(RG_ERR_SERIALIZATION, "%s: %s", path ? path : "(null)", e.what());
    }
}
