// Exercises the C++ host mirror (include/rg_b200.hpp) end to end on cuda:0.
// The cases are the reference's own: the 2x2 matmul of src/backend/cuda.rs:545-571,
// ReLU of src/backend/simd.rs:167-171, the LayerNorm row of src/backend/fused.rs:228-247,
// the error behaviour of src/ops/embedding.rs:51-56, and a GPT forward / generate
// round trip with the model shapes of tests/nn_test.rs.  Prints "OK" and returns 0.
#include <cmath>
#include <cstdio>
#include <random>

#include "rg_b200.hpp"

#define EXPECT(c)                                                     \
    do {                                                              \
        if (!(c)) {                                                   \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); \
            return 1;                                                 \
        }                                                             \
    } while (0)

int main() {
    EXPECT(rg::B200Backend::is_available());
    rg::B200Backend be(0);
    auto c = be.to_vec(be.matmul(be.from_slice({1, 2, 3, 4}, {2, 2}), be.from_slice({5, 6, 7, 8}, {2, 2})));
    EXPECT(c.size() == 4 && std::fabs(c[0] - 19) < 1e-5 && std::fabs(c[1] - 22) < 1e-5 && std::fabs(c[2] - 43) < 1e-5 &&
           std::fabs(c[3] - 50) < 1e-5);
    auto r = be.to_vec(be.relu(be.from_slice({-2, -1, 1, 2}, {4})));
    EXPECT(r[0] == 0 && r[1] == 0 && r[2] == 1 && r[3] == 2);
    auto ln = be.to_vec(be.layer_norm(be.from_slice({1, 2, 3, 4}, {1, 4}), be.ones({1, 4}), be.zeros({1, 4}), 1e-5f));
    float mean = 0, var = 0;
    for (float v : ln) mean += v / 4;
    for (float v : ln) var += (v - mean) * (v - mean) / 4;
    EXPECT(std::fabs(mean) < 1e-3 && std::fabs(var - 1) < 0.1);
    bool threw = false;
    try {
        be.embedding(be.from_slice({7}, {1, 1}), be.zeros({5, 4}));
    } catch (const rg::InvalidInput&) {
        threw = true;
    }
    EXPECT(threw);
    threw = false;
    try {
        be.add(be.zeros({2, 3}), be.zeros({3, 2}));
    } catch (const rg::ShapeError&) {
        threw = true;
    }
    EXPECT(threw);

    rg::GptConfig cfg;
    cfg.block_size = 16, cfg.vocab_size = 30, cfg.num_layers = 1, cfg.num_heads = 2, cfg.embedding_dim = 64;
    rg::GPTModel model(be, cfg);
    std::mt19937 gen(1);
    std::normal_distribution<float> nd(0.f, 0.02f);
    std::vector<std::vector<float>> params;
    for (auto s : model.parameter_shapes()) {
        std::vector<float> t(s.first * s.second);
        for (auto& v : t) v = nd(gen);
        params.push_back(t);
    }
    // LayerNorm gamma = 1 (positions 8, 14 of the block, and the final one)
    const size_t n = params.size();
    for (size_t i : {size_t(2 + 8), size_t(2 + 14), n - 4}) std::fill(params[i].begin(), params[i].end(), 1.f);
    model.load_parameters(params);
    auto logits = model.forward({1, 2, 3, 4, 5}, 1, 5);
    EXPECT(logits.size() == 5 * 30);
    for (float v : logits) EXPECT(std::isfinite(v));
    auto ids = model.generate({1, 2, 3}, 6);
    EXPECT(ids.size() == 6);
    // greedy: the first new id is the argmax of the last row of a forward on the prompt
    auto l3 = model.forward({1, 2, 3}, 1, 3);
    size_t best = 0;
    for (size_t v = 1; v < 30; v++)
        if (l3[2 * 30 + v] > l3[2 * 30 + best]) best = v;
    EXPECT(ids[0] == best);
    threw = false;
    try {
        model.generate({1, 2, 3}, 15);  // 3 + 15 - 1 > block_size
    } catch (const rg::ContextFull&) {
        threw = true;
    }
    EXPECT(threw);
    // Tokenizer trait: the reference's own char-tokenizer checks (src/tokenization/char_tokenizer.rs:113-161)
    auto tok = rg::Tokenizer::chars_of("Hello, world!");
    auto enc = tok.encode("Hello");
    EXPECT(enc.size() == 5 && tok.decode(enc) == "Hello");
    EXPECT(rg::Tokenizer::chars_of("aabbcc").vocab_size() == 3);
    auto abc = rg::Tokenizer::char_vocab({'a', 'b', 'c'});
    EXPECT(abc.encode("cab") == (std::vector<uint32_t>{2, 0, 1}));
    threw = false;
    try {
        rg::Tokenizer::bpe_load("/nonexistent/tokenizer.json");
    } catch (const rg::IoError&) {
        threw = true;
    }
    EXPECT(threw);
    threw = false;
    try {
        model.load_safetensors("/nonexistent/model.safetensors");
    } catch (const rg::IoError&) {
        threw = true;
    }
    EXPECT(threw);
    // TensorV2 / ops_v2: the reference's own unit cases (src/tensor_v2.rs tests, src/ops_v2/basic.rs and matmul.rs tests)
    {
        auto a = rg::TensorV2::ones(be, {2, 2}, false), b = rg::TensorV2::ones(be, {2, 2}, true);
        auto sum = rg::add_op(a, b);
        EXPECT(sum.shape() == (std::vector<size_t>{2, 2}) && sum.requires_grad() && sum.dtype() == rg::DType::F32);
        auto sv = sum.to_cpu_data();
        EXPECT(sv.size() == 4 && sv[0] == 2 && sv[3] == 2);
        auto prod = rg::mul_op(rg::TensorV2::from_slice(be, {2, 3}, {2}, false), rg::TensorV2::from_slice(be, {4, 5}, {2}, false));
        auto pv = prod.to_cpu_data();
        EXPECT(prod.shape() == (std::vector<size_t>{2}) && pv[0] == 8 && pv[1] == 15 && !prod.requires_grad());
        auto mm = rg::matmul_op(rg::TensorV2::zeros(be, {2, 3, 4}, false), rg::TensorV2::zeros(be, {2, 4, 5}, false));
        EXPECT(mm.shape() == (std::vector<size_t>{2, 3, 5}));
        EXPECT(rg::sub_op(sum, a).relu().transpose(0, 1).reshape({4}).shape() == (std::vector<size_t>{4}));
    }
    std::printf("OK\n");
    return 0;
}
