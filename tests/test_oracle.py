"""CPU tests of the oracle: the reference's own known answers, an independent
float64 implementation, the committed golden vectors and the mode bridges."""
import os

import numpy as np
import pytest
import torch

from oracle import gpt_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- the reference's known answers (the only values its tests pin) -----------
def test_reference_kats():
    k = O.reference_kats()
    m = k["matmul_2x2"]
    assert np.abs(m["a"] @ m["b"] - m["out"]).max() <= m["tol"]
    assert np.array_equal(O.relu(k["relu_4"]["x"]), k["relu_4"]["out"])
    assert np.array_equal(O.relu(k["relu_5"]["x"]), k["relu_5"]["out"])
    assert abs(O.sigmoid(k["sigmoid_0"]["x"])[0] - 0.5) <= 1e-6
    ln = k["layernorm_1234"]
    for f in (O.layernorm_two_pass, O.layernorm_welford):
        y = f(ln["x"], ln["gamma"], ln["beta"], ln["eps"])
        assert abs(float(y.mean())) < 1e-3           # src/backend/fused.rs:240-242
        assert abs(float(y.var()) - 1.0) < 0.1       # src/backend/fused.rs:244-246
    g = O.gelu_tanh(k["gelu_01"]["x"])
    assert abs(g[0]) < 1e-6 and 0.8 < g[1] < 0.9     # src/backend/fused.rs:250-259
    # ramps of examples/cuda_kernels_test.rs against float64 arithmetic, at the reference's tolerances
    r = k["ramp_add"]
    assert np.abs((r["a"] + r["b"]) - (r["a"].astype(np.float64) + r["b"])).max() <= r["tol"]
    r = k["ramp_exp"]
    assert np.abs(np.exp(r["x"]) - np.exp(r["x"].astype(np.float64))).max() <= r["tol"]
    r = k["ramp_sigmoid"]
    assert np.abs(O.sigmoid(r["x"]) - 1 / (1 + np.exp(-r["x"].astype(np.float64)))).max() <= r["tol"]
    r = k["ramp_softmax"]
    x64 = r["x"].astype(np.float64)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    assert np.abs(O.softmax_lastaxis(r["x"]) - e / e.sum(-1, keepdims=True)).max() <= r["tol"]


def test_param_order_and_count():
    cfg = O.CONFIGS[1]["cfg"]
    shapes = O.param_shapes(cfg)
    assert len(shapes) == 2 + 16 * cfg.num_layers + 4 == cfg.n_params_tensors
    D, V, C, L = cfg.embedding_dim, cfg.vocab_size, cfg.block_size, cfg.num_layers
    n = sum(int(np.prod(s)) for s in shapes)
    assert n == V * D + C * D + L * (12 * D * D + 13 * D) + 2 * D + D * V + V
    assert shapes[0] == (V, D) and shapes[1] == (C, D)
    assert shapes[2 + 10] == (D, 4 * D) and shapes[2 + 12] == (4 * D, D)
    assert shapes[-2] == (D, V) and shapes[-1] == (1, V)
    p = O.make_params(O.CONFIGS[0]["cfg"], 1)
    assert np.all(p[2 + 8] == 1) and np.all(p[2 + 9] == 0) and np.all(p[-4] == 1)
    assert abs(float(p[0].std()) - 0.02) < 2e-3


# ---- independent implementation: torch, float64, written from the forward spec
def _torch_forward(params, cfg, ids, causal, act):
    P = [torch.from_numpy(p).double() for p in params]
    ids = torch.from_numpy(np.asarray(ids, dtype=np.int64))
    B, T = ids.shape
    H, D = cfg.num_heads, cfg.embedding_dim
    x = P[0][ids] + P[1][torch.arange(T)][None]
    ln = torch.nn.functional.layer_norm
    for l in range(cfg.num_layers):
        p = P[2 + 16 * l: 18 + 16 * l]
        n = ln(x, (D,), p[8][0], p[9][0], 1e-5)
        q, k, v = [(n @ p[2 * i] + p[2 * i + 1][0]).view(B, T, H, D // H).transpose(1, 2) for i in range(3)]
        s = (q @ k.transpose(-1, -2)) / (D // H) ** 0.5
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        a = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, T, D)
        x = x + a @ p[6] + p[7][0]
        n = ln(x, (D,), p[14][0], p[15][0], 1e-5)
        h = n @ p[10] + p[11][0]
        h = torch.relu(h) if act == "relu" else torch.nn.functional.gelu(h, approximate="tanh")
        x = x + h @ p[12] + p[13][0]
    n = ln(x, (D,), P[-4][0], P[-3][0], 1e-5)
    return (n @ P[-2] + P[-1][0]).numpy()


@pytest.mark.parametrize("causal,act", [(False, "relu"), (True, "gelu_tanh"), (False, "gelu_tanh"), (True, "relu")])
def test_oracle_matches_float64(causal, act):
    cfg = O.GptConfig(32, 40, 2, 4, 64)
    params = O.make_params(cfg, 3, stress=True)
    ids = O.make_prompt(cfg, 3, 2, 19)
    got = O.forward(params, cfg, ids, causal=causal, act=act)
    want = _torch_forward(params, cfg, ids, causal, act)
    assert np.abs(got - want).max() < 1e-5


def test_oracle_matches_float64_char_gpt():
    c = O.CONFIGS[0]
    params = O.make_params(c["cfg"], O.config_seed(0))
    ids = O.make_prompt(c["cfg"], O.config_seed(0), 1, 64)
    for causal, act in ((False, "relu"), (True, "gelu_tanh")):
        d = np.abs(O.forward(params, c["cfg"], ids, causal, act) - _torch_forward(params, c["cfg"], ids, causal, act))
        assert d.max() < 1e-5


# ---- bridges between the two modes ------------------------------------------
def test_mode_bridges():
    cfg = O.GptConfig(16, 30, 2, 2, 64)
    params = O.make_params(cfg, 5, stress=True)
    ids = O.make_prompt(cfg, 5, 3, 12)
    # a single-token context has nothing to mask
    a = O.forward(params, cfg, ids[:, :1], causal=False, act="relu")
    b = O.forward(params, cfg, ids[:, :1], causal=True, act="relu")
    assert np.array_equal(a, b)
    # under the causal mask, row t of a long forward equals the last row of a forward on the prefix
    full = O.forward(params, cfg, ids, causal=True, act="gelu_tanh")
    for t in (0, 5, 11):
        pre = O.forward(params, cfg, ids[:, :t + 1], causal=True, act="gelu_tanh", last_only=True)
        assert np.abs(full[:, t] - pre[:, 0]).max() < 2e-6
    # without the mask it does not (the reference cannot use a KV cache)
    nf = O.forward(params, cfg, ids, causal=False, act="relu")
    np_ = O.forward(params, cfg, ids[:, :6], causal=False, act="relu", last_only=True)
    assert np.abs(nf[:, 5] - np_[:, 0]).max() > 1e-4
    # Welford and two-pass LayerNorm agree
    x = np.random.default_rng(0).standard_normal((4, 96)).astype(np.float32) * 3 + 1
    g, bta = params[2 + 8][:, :64], params[2 + 9][:, :64]
    assert np.abs(O.layernorm_welford(x[:, :64], g, bta) - O.layernorm_two_pass(x[:, :64], g, bta)).max() < 2e-6


def test_greedy_is_top_k_one():
    rng = np.random.default_rng(1)
    for _ in range(20):
        lg = rng.standard_normal(37).astype(np.float32)
        for u in (0.0, 0.3, 0.999):
            assert O.sample_topk(lg, 0.8, 1, u) == O.greedy_pick(lg)
    # top_k >= V keeps the whole distribution: the walk follows the CDF
    lg = np.log(np.array([0.1, 0.2, 0.3, 0.4], np.float32))
    assert [O.sample_topk(lg, 1.0, 0, u) for u in (0.05, 0.25, 0.5, 0.95)] == [0, 1, 2, 3]
    assert [O.sample_topk(lg, 1.0, 2, u) for u in (0.1, 0.9)] == [2, 3]


def test_embedding_errors():
    t = np.zeros((5, 4), np.float32)
    with pytest.raises(IndexError):
        O.embedding(np.array([[5.0]]), t)
    with pytest.raises(ValueError):
        O.embedding(np.array([1.0]), t)
    cfg = O.GptConfig(4, 10, 1, 1, 32)
    with pytest.raises(IndexError):
        O.forward(O.make_params(cfg, 0), cfg, np.zeros((1, 5), np.int64))


def test_sliding_window_loop():
    cfg = O.GptConfig(8, 20, 1, 2, 64)
    params = O.make_params(cfg, 9)
    out = O.generate_reference(params, cfg, [1, 2, 3, 4, 5, 6], 6)   # crosses block_size
    assert len(out) == 6 and all(0 <= t < 20 for t in out)
    ids = [1, 2, 3, 4, 5, 6] + out[:5]
    lg = O.forward(params, cfg, np.asarray(ids[-8:])[None], last_only=True)[0, 0]
    assert int(np.argmax(lg)) == out[5]


# ---- the committed golden vectors --------------------------------------------
def test_golden_char_gpt():
    g = np.load(os.path.join(GOLD, "char_gpt.npz"))
    c = O.CONFIGS[0]
    cfg, seed = c["cfg"], O.config_seed(0)
    assert np.array_equal(g["prompt"], O.make_prompt(cfg, seed, 1, c["prompt"]))
    for stress in (False, True):
        tag = "stress" if stress else "plain"
        params = O.make_params(cfg, seed, stress=stress)
        ids = np.concatenate([g["prompt"], g[f"n_{tag}_tokens"]], 1)
        lg = O.teacher_forced_logits(params, cfg, ids, True, "gelu_tanh", c["prompt"])
        assert np.abs(lg - g[f"n_{tag}_logits"]).max() < 2e-5
        assert np.array_equal(lg.argmax(-1), g[f"n_{tag}_tokens"])
        ids = np.concatenate([g["prompt"], g[f"r_{tag}_tokens"]], 1)
        lg = O.teacher_forced_logits(params, cfg, ids[:, :c["prompt"] + 8], False, "relu", c["prompt"])
        assert np.abs(lg - g[f"r_{tag}_logits"][:, :8]).max() < 2e-5


def test_golden_gpt2_small_sample():
    g = np.load(os.path.join(GOLD, "gpt2_small_sample.npz"))
    c = O.CONFIGS[1]
    cfg, seed = c["cfg"], O.config_seed(1)
    params = O.make_params(cfg, seed)
    assert np.array_equal(g["prompt"], O.make_prompt(cfg, seed, 1, c["prompt"]))
    ids = np.concatenate([g["prompt"], g["n_tokens"]], 1)[:, :c["prompt"] + 3]
    lg = O.teacher_forced_logits(params, cfg, ids, True, "gelu_tanh", c["prompt"])
    assert np.abs(lg - g["n_logits"][:, :3]).max() < 5e-5
    assert np.array_equal(lg.argmax(-1), g["n_tokens"][:, :3])


def test_step_bytes_formula():
    # GPT-2-small shape, f32, batch 1, mean context 256: 362.3 MB; roofline 22,084 tok/s at 8 TB/s
    cfg = O.CONFIGS[1]["cfg"]
    b = O.decode_step_bytes(cfg, 1, 256, 4, 4)
    assert abs(b / 1e6 - 362.3) < 0.2
    assert abs(8e12 / b - 22084) < 20
    cfg3 = O.CONFIGS[2]["cfg"]
    assert abs(O.decode_step_bytes(cfg3, 64, 384, 2, 2) / 1e6 - 1153) < 2


def test_bf16_round():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-5, 0.0], np.float32)
    r = O.bf16_round(x)
    t = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(r, t)


def test_weighted_index_draw_is_the_top_k_0_draw():
    """KnowledgeManager::generate (WeightedIndex over exp(l / T)) and WasmGptTrainer::generate with top_k = 0 (normalised
    inverse-CDF walk) draw from the same distribution: for the same uniform number they return the same id unless the
    number falls within f32 rounding of a CDF step, and then the neighbouring id."""
    rng = np.random.default_rng(7)
    V = 97
    same = total = 0
    for trial in range(40):
        logits = (rng.standard_normal(V) * 1.5).astype(np.float32)
        T = (0.7, 1.0, 1.3)[trial % 3]
        for u in rng.random(25):
            a = O.sample_weighted(logits, T, float(u))
            b = O.sample_topk(logits, T, 0, float(u))
            total += 1
            same += a == b
            assert abs(a - b) <= 1
    assert same >= total - 2
    # the edges of the binary search: u = 0 gives the first id with a positive weight, u just below 1 the last id
    w = np.array([0.0, 2.0, 0.0, 1.0, 1.0], np.float32)
    assert O.weighted_index_sample(w, 0.0) == 1
    assert O.weighted_index_sample(w, 0.49) == 1 and O.weighted_index_sample(w, 0.5) == 3
    assert O.weighted_index_sample(w, 0.75) == 4 and O.weighted_index_sample(w, 0.999999) == 4
    # frequencies follow the weights
    draws = np.array([O.weighted_index_sample(w, float(u)) for u in rng.random(4000)])
    freq = np.bincount(draws, minlength=5) / 4000
    assert np.abs(freq - w / w.sum()).max() < 0.03
    with pytest.raises(ValueError):
        O.weighted_index_sample(np.zeros(4, np.float32), 0.3)


def test_folded_layernorm_and_shifted_sums_identities():
    """The algebra the token-loop kernels rely on, checked in float64 against the oracle's LayerNorm + Linear
    (src/ops/norm.rs:41-52, src/nn/linear.rs:50-56):
    LN(x).W + b = rstd * (x.(g*W) - mean * sum_k(g_k W_kn)) + (beta.W + b), and the exact combination of per-warp shifted
    sums (count, sum(x - c), sum((x - c)^2), shift c) into mean and biased variance."""
    rng = np.random.default_rng(3)
    K, N = 768, 40
    x = rng.standard_normal(K) * 3 + 1.5
    g, beta = 1 + 0.1 * rng.standard_normal(K), 0.1 * rng.standard_normal(K)
    W, b = rng.standard_normal((K, N)) * 0.02, rng.standard_normal(N) * 0.02
    mean, var = x.mean(), x.var()
    rstd = 1.0 / np.sqrt(var + 1e-5)
    direct = (((x - mean) * rstd) * g + beta) @ W + b
    folded = rstd * (x @ (g[:, None] * W) - mean * (g @ W)) + (beta @ W + b)
    assert np.abs(direct - folded).max() < 1e-12
    want = O.layernorm_two_pass(x.astype(np.float32)[None, :], g.astype(np.float32), beta.astype(np.float32))[0].astype(np.float64) @ W + b
    assert np.abs(want - folded).max() < 2e-5
    # 8 warps, each with its own shift (its first element); combined with the first warp's shift as the common one
    parts = []
    for w in range(8):
        xs = x[w * 32:(w + 1) * 32] if w < 7 else x[7 * 32:]
        c = xs[0]
        parts.append((len(xs), (xs - c).sum(), ((xs - c) ** 2).sum(), c))
    C0 = parts[0][3]
    S0 = sum(p[0] for p in parts)
    S1 = sum(p[1] + p[0] * (p[3] - C0) for p in parts)
    S2 = sum(p[2] + 2 * (p[3] - C0) * p[1] + p[0] * (p[3] - C0) ** 2 for p in parts)
    m1 = S1 / S0
    assert abs((C0 + m1) - mean) < 1e-12 and abs((S2 / S0 - m1 * m1) - var) < 1e-10
