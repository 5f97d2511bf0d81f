// rg_b200.hpp - C++ host-side mirror of the reference's interface for the GPT token
// loop, over the C ABI of rg_b200.h.  Same names, argument meaning and error variants
// as the crate (rusty-gradients 0.2.0):
//
//   rg::Error / ShapeError / DimensionError / InvalidInput / BackendError ...   src/error.rs:13-50
//   rg::B200Backend  - `trait Backend` as implemented by CudaBackend            src/backend/mod.rs:130-227, src/backend/cuda.rs:77-135
//   rg::Storage      - CudaStorage {data, shape, device}, an immutable value     src/backend/cuda.rs:29-74
//   rg::GptConfig, rg::GPTModel {forward, parameters order}                      src/models/gpt.rs:8-93
//   rg::GPTModel::generate(prompt_ids, max_new_tokens, temperature, top_k)       src/wasm_api.rs:97-163
//
// Header-only; link with -lrg_b200.  Errors are exceptions (Rust's Result::Err).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "rg_b200.h"

namespace rg {

struct Error : std::runtime_error {
    rg_status status;
    Error(rg_status s, const std::string& m) : std::runtime_error(m), status(s) {}
};
struct ShapeError : Error { using Error::Error; };
struct DimensionError : Error { using Error::Error; };
struct InvalidInput : Error { using Error::Error; };
struct BackendError : Error { using Error::Error; };
struct Unsupported : Error { using Error::Error; };
struct ContextFull : Error { using Error::Error; };
struct DeviceTimeout : Error { using Error::Error; };
struct SerializationError : Error { using Error::Error; };
struct IoError : Error { using Error::Error; };

inline void check(rg_status s) {
    if (s == RG_OK) return;
    const std::string msg = rg_last_error();
    switch (s) {
        case RG_ERR_SHAPE: throw ShapeError(s, msg);
        case RG_ERR_DIMENSION: throw DimensionError(s, msg);
        case RG_ERR_INVALID_INPUT: throw InvalidInput(s, msg);
        case RG_ERR_BACKEND: throw BackendError(s, msg);
        case RG_ERR_UNSUPPORTED: throw Unsupported(s, msg);
        case RG_ERR_CONTEXT_FULL: throw ContextFull(s, msg);
        case RG_ERR_TIMEOUT: throw DeviceTimeout(s, msg);
        case RG_ERR_SERIALIZATION: throw SerializationError(s, msg);
        case RG_ERR_IO: throw IoError(s, msg);
        default: throw Error(s, msg);
    }
}

// CudaStorage: owned, immutable; freed when the last copy goes away.
class Storage {
  public:
    Storage() = default;
    explicit Storage(rg_storage* h) : h_(h, [](rg_storage* p) { rg_storage_free(p); }) {}
    rg_storage* get() const { return h_.get(); }
    std::vector<size_t> shape() const {
        size_t buf[8];
        int nd = 0;
        check(rg_shape(h_.get(), buf, 8, &nd));
        return std::vector<size_t>(buf, buf + nd);
    }
    size_t len() const { return rg_storage_len(h_.get()); }

  private:
    std::shared_ptr<rg_storage> h_;
};

// `impl Backend for CudaBackend`: every method returns a new Storage and never modifies its inputs.
class B200Backend {
  public:
    explicit B200Backend(int device_index = 0) : index_(device_index) {
        rg_ctx* c = nullptr;
        check(rg_ctx_create(device_index, &c));
        ctx_.reset(c, [](rg_ctx* p) { rg_ctx_destroy(p); });
    }
    static int device_count() { return rg_device_count(); }
    static bool is_available() { return device_count() > 0; }
    int device_index() const { return index_; }
    rg_ctx* ctx() const { return ctx_.get(); }
    void synchronize() const { check(rg_synchronize(ctx_.get())); }

    Storage zeros(const std::vector<size_t>& shape) const { return make([&](rg_storage** o) { return rg_zeros(ctx_.get(), shape.data(), (int)shape.size(), o); }); }
    Storage ones(const std::vector<size_t>& shape) const { return make([&](rg_storage** o) { return rg_ones(ctx_.get(), shape.data(), (int)shape.size(), o); }); }
    Storage from_slice(const std::vector<float>& data, const std::vector<size_t>& shape) const {
        return make([&](rg_storage** o) { return rg_from_slice(ctx_.get(), data.data(), data.size(), shape.data(), (int)shape.size(), o); });
    }
    std::vector<float> to_vec(const Storage& s) const {
        std::vector<float> out(s.len());
        check(rg_to_vec(ctx_.get(), s.get(), out.data(), out.size()));
        return out;
    }
    std::vector<size_t> shape(const Storage& s) const { return s.shape(); }

    Storage add(const Storage& a, const Storage& b) const { return bin(rg_add, a, b); }
    Storage sub(const Storage& a, const Storage& b) const { return bin(rg_sub, a, b); }
    Storage mul(const Storage& a, const Storage& b) const { return bin(rg_mul, a, b); }
    Storage matmul(const Storage& a, const Storage& b) const { return bin(rg_matmul, a, b); }
    Storage embedding(const Storage& indices, const Storage& weights) const { return bin(rg_embedding, indices, weights); }
    Storage sparse_cross_entropy(const Storage& logits, const Storage& targets) const { return bin(rg_sparse_cross_entropy, logits, targets); }
    Storage relu(const Storage& a) const { return un(rg_relu, a); }
    Storage sigmoid(const Storage& a) const { return un(rg_sigmoid, a); }
    Storage exp(const Storage& a) const { return un(rg_exp, a); }
    Storage log(const Storage& a) const { return un(rg_log, a); }
    Storage gelu(const Storage& a) const { return un(rg_gelu, a); }
    Storage softmax(const Storage& a) const { return un(rg_softmax, a); }
    Storage sum(const Storage& a) const { return un(rg_sum, a); }
    Storage powf(const Storage& a, float p) const { return make([&](rg_storage** o) { return rg_powf(ctx_.get(), a.get(), p, o); }); }
    Storage sum_axis(const Storage& a, size_t axis) const { return make([&](rg_storage** o) { return rg_sum_axis(ctx_.get(), a.get(), axis, o); }); }
    Storage reshape(const Storage& a, const std::vector<size_t>& s) const { return make([&](rg_storage** o) { return rg_reshape(ctx_.get(), a.get(), s.data(), (int)s.size(), o); }); }
    Storage transpose(const Storage& a, size_t ax1, size_t ax2) const { return make([&](rg_storage** o) { return rg_transpose(ctx_.get(), a.get(), ax1, ax2, o); }); }
    Storage layer_norm(const Storage& x, const Storage& gamma, const Storage& beta, float eps) const {
        return make([&](rg_storage** o) { return rg_layer_norm(ctx_.get(), x.get(), gamma.get(), beta.get(), eps, o); });
    }

  private:
    template <typename F>
    Storage make(F f) const {
        rg_storage* h = nullptr;
        check(f(&h));
        return Storage(h);
    }
    using bin_fn = rg_status (*)(rg_ctx*, const rg_storage*, const rg_storage*, rg_storage**);
    using un_fn = rg_status (*)(rg_ctx*, const rg_storage*, rg_storage**);
    Storage bin(bin_fn f, const Storage& a, const Storage& b) const { return make([&](rg_storage** o) { return f(ctx_.get(), a.get(), b.get(), o); }); }
    Storage un(un_fn f, const Storage& a) const { return make([&](rg_storage** o) { return f(ctx_.get(), a.get(), o); }); }
    std::shared_ptr<rg_ctx> ctx_;
    int index_;
};

// GptConfig (src/models/gpt.rs:8-14) plus the engine's switches.
struct GptConfig {
    size_t block_size = 0, vocab_size = 0, num_layers = 0, num_heads = 0, embedding_dim = 0;
    bool causal = true;            // false: the reference's unmasked attention (no KV cache possible)
    bool gelu = true;              // false: ReLU, the reference's FeedForward
    bool bf16_weights = false;
    size_t max_batch = 1;
    int tp_rank = 0, tp_size = 1;
};

class GPTModel {
  public:
    GPTModel(const B200Backend& be, const GptConfig& c) : be_(be), cfg_(c) {
        rg_gpt_config k{c.block_size, c.vocab_size, c.num_layers, c.num_heads, c.embedding_dim, c.causal ? 1 : 0,
                        c.gelu ? RG_ACT_GELU_TANH : RG_ACT_RELU, c.bf16_weights ? RG_DTYPE_BF16 : RG_DTYPE_F32, c.max_batch,
                        c.tp_rank, c.tp_size};
        rg_gpt* m = nullptr;
        check(rg_gpt_create(be.ctx(), &k, &m));
        m_.reset(m, [](rg_gpt* p) { rg_gpt_destroy(p); });
    }
    // Module::parameters() order (gpt.rs:85-93): shapes of the 2 + 16 L + 4 tensors
    std::vector<std::pair<size_t, size_t>> parameter_shapes() const {
        std::vector<std::pair<size_t, size_t>> out;
        for (int i = 0; i < rg_gpt_num_params(m_.get()); i++) {
            size_t s[2];
            check(rg_gpt_param_shape(m_.get(), i, s));
            out.emplace_back(s[0], s[1]);
        }
        return out;
    }
    // loadWeightsFromJson's contract (wasm_api.rs:182-199): same count, same shapes, in order
    void load_parameters(const std::vector<std::vector<float>>& tensors) {
        const auto shp = parameter_shapes();
        std::vector<const float*> data;
        std::vector<std::vector<size_t>> shapes;
        std::vector<const size_t*> sp;
        std::vector<int> nd;
        for (size_t i = 0; i < tensors.size(); i++) {
            data.push_back(tensors[i].data());
            if (i < shp.size()) shapes.push_back({shp[i].first, shp[i].second});
            else shapes.push_back({tensors[i].size(), 1});
            if (shapes.back()[0] * shapes.back()[1] != tensors[i].size())
                throw ShapeError(RG_ERR_SHAPE, "Mismatch in tensor shape during loading: parameter " + std::to_string(i));
            nd.push_back(2);
        }
        for (auto& s : shapes) sp.push_back(s.data());
        check(rg_gpt_load_params(m_.get(), data.data(), sp.data(), nd.data(), (int)tensors.size()));
    }
    // load_model (src/serialization/safetensors_format.rs:89-138) + the copy into the model
    void load_safetensors(const std::string& path, rg_names names = RG_NAMES_AUTO) {
        check(rg_gpt_load_safetensors(m_.get(), path.c_str(), (int)names));
    }
    // loadWeightsFromJson (src/wasm_api.rs:179-199) from a file, or a JsonCheckpoint (src/serialization/mod.rs:52-74)
    void load_json(const std::string& path) { check(rg_gpt_load_json(m_.get(), path.c_str())); }
    // Module::forward: idx [B,T] carried as f32 -> logits [B,T,V]
    std::vector<float> forward(const std::vector<float>& idx, size_t B, size_t T) {
        std::vector<float> out(B * T * cfg_.vocab_size);
        check(rg_gpt_forward(m_.get(), idx.data(), B, T, out.data()));
        return out;
    }
    // WasmGptTrainer::generate for one prompt
    std::vector<uint32_t> generate(const std::vector<uint32_t>& prompt_ids, size_t max_new_tokens, float temperature = 1.f,
                                   size_t top_k = 1, uint64_t seed = 0) {
        std::vector<uint32_t> out(max_new_tokens);
        check(rg_gpt_generate(m_.get(), prompt_ids.data(), 1, prompt_ids.size(), max_new_tokens, temperature, top_k, seed, out.data()));
        return out;
    }
    rg_gpt* get() const { return m_.get(); }

  private:
    B200Backend be_;
    GptConfig cfg_;
    std::shared_ptr<rg_gpt> m_;
};

// DType and TensorV2 (src/tensor_v2.rs:16-23, 64-83, 85-305): a tensor that knows its device, dtype and whether it
// requires a gradient.  Like the reference's, every operation forwards to the Backend method of the same name and the
// result requires a gradient when an operand does; this library computes the forward path only, so no gradient is kept.
// The data lives on the backend's GPU (the reference's non-CPU arms are `unimplemented!`; here they are the only ones).
enum class DType { F32, F16, BF16, I32, U32 };

class TensorV2 {
  public:
    TensorV2(const B200Backend& be, Storage data, bool requires_grad) : be_(be), data_(std::move(data)), requires_grad_(requires_grad) {}
    // TensorV2::from_slice / zeros / ones
    static TensorV2 from_slice(const B200Backend& be, const std::vector<float>& data, const std::vector<size_t>& shape, bool requires_grad) {
        return TensorV2(be, be.from_slice(data, shape), requires_grad);
    }
    static TensorV2 zeros(const B200Backend& be, const std::vector<size_t>& shape, bool requires_grad) { return TensorV2(be, be.zeros(shape), requires_grad); }
    static TensorV2 ones(const B200Backend& be, const std::vector<size_t>& shape, bool requires_grad) { return TensorV2(be, be.ones(shape), requires_grad); }

    std::vector<size_t> shape() const { return data_.shape(); }
    DType dtype() const { return DType::F32; }
    bool requires_grad() const { return requires_grad_; }
    int device_index() const { return be_.device_index(); }
    std::vector<float> to_cpu_data() const { return be_.to_vec(data_); }
    const Storage& storage() const { return data_; }

    TensorV2 add(const TensorV2& o) const { return TensorV2(be_, be_.add(data_, o.data_), requires_grad_ || o.requires_grad_); }
    TensorV2 sub(const TensorV2& o) const { return TensorV2(be_, be_.sub(data_, o.data_), requires_grad_ || o.requires_grad_); }
    TensorV2 mul(const TensorV2& o) const { return TensorV2(be_, be_.mul(data_, o.data_), requires_grad_ || o.requires_grad_); }
    TensorV2 matmul(const TensorV2& o) const { return TensorV2(be_, be_.matmul(data_, o.data_), requires_grad_ || o.requires_grad_); }
    TensorV2 relu() const { return TensorV2(be_, be_.relu(data_), requires_grad_); }
    TensorV2 softmax() const { return TensorV2(be_, be_.softmax(data_), requires_grad_); }
    TensorV2 reshape(const std::vector<size_t>& s) const { return TensorV2(be_, be_.reshape(data_, s), requires_grad_); }
    TensorV2 transpose(size_t a, size_t b) const { return TensorV2(be_, be_.transpose(data_, a, b), requires_grad_); }

  private:
    B200Backend be_;
    Storage data_;
    bool requires_grad_;
};

// ops_v2 (src/ops_v2/basic.rs:15, 56, 94; src/ops_v2/matmul.rs:15)
inline TensorV2 add_op(const TensorV2& a, const TensorV2& b) { return a.add(b); }
inline TensorV2 mul_op(const TensorV2& a, const TensorV2& b) { return a.mul(b); }
inline TensorV2 sub_op(const TensorV2& a, const TensorV2& b) { return a.sub(b); }
inline TensorV2 matmul_op(const TensorV2& a, const TensorV2& b) { return a.matmul(b); }

// trait Tokenizer (src/tokenization/mod.rs): encode / decode / vocab_size
class Tokenizer {
  public:
    // CharTokenizer::new(text)
    static Tokenizer chars_of(const std::string& text) {
        rg_tokenizer* t = nullptr;
        check(rg_tokenizer_char_from_text(text.data(), text.size(), &t));
        return Tokenizer(t);
    }
    // CharTokenizer::from_vocab(&[char])
    static Tokenizer char_vocab(const std::vector<uint32_t>& codepoints) {
        rg_tokenizer* t = nullptr;
        check(rg_tokenizer_char_from_vocab(codepoints.data(), codepoints.size(), &t));
        return Tokenizer(t);
    }
    // BPETokenizer::load(path)
    static Tokenizer bpe_load(const std::string& path) {
        rg_tokenizer* t = nullptr;
        check(rg_tokenizer_bpe_load(path.c_str(), &t));
        return Tokenizer(t);
    }
    std::vector<uint32_t> encode(const std::string& text) const {
        size_t n = 0;
        check(rg_tokenizer_encode(t_.get(), text.data(), text.size(), nullptr, 0, &n));
        std::vector<uint32_t> ids(n);
        check(rg_tokenizer_encode(t_.get(), text.data(), text.size(), ids.data(), ids.size(), &n));
        return ids;
    }
    std::string decode(const std::vector<uint32_t>& ids) const {
        size_t n = 0;
        check(rg_tokenizer_decode(t_.get(), ids.data(), ids.size(), nullptr, 0, &n));
        std::string s(n, '\0');
        check(rg_tokenizer_decode(t_.get(), ids.data(), ids.size(), &s[0], s.size(), &n));
        return s;
    }
    size_t vocab_size() const {
        size_t n = 0;
        check(rg_tokenizer_vocab_size(t_.get(), &n));
        return n;
    }

  private:
    explicit Tokenizer(rg_tokenizer* t) : t_(t, [](rg_tokenizer* p) { rg_tokenizer_free(p); }) {}
    std::shared_ptr<rg_tokenizer> t_;
};

}  // namespace rg
