"""GPU parity of the GPT token loop against the oracle, teacher-forced: same
seeded weights and ids; logits within the stated tolerance on every step, ids and
argmax bit-exact."""
import os

import numpy as np
import pytest

import rustygradients_b200 as rg
from oracle import gpt_oracle as O
from helpers import BF16_REL_TOL, F32_TOL, assert_bf16_close, confident_rows, model_for, teacher_forced

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


# ---- configuration 0: char GPT, every step, against the committed golden vectors
@pytest.mark.parametrize("tag", ["plain", "stress"])
def test_char_gpt_kv_cache_steps_match_golden(backend, tag):
    g = np.load(os.path.join(GOLD, "char_gpt.npz"))
    c = O.CONFIGS[0]
    params = O.make_params(c["cfg"], O.config_seed(0), stress=(tag == "stress"))
    m = model_for(backend, c["cfg"], params)
    ids = np.concatenate([g["prompt"], g[f"n_{tag}_tokens"]], 1)
    logits, picks = teacher_forced(m, ids, c["prompt"])
    want = g[f"n_{tag}_logits"]
    assert logits.shape == want.shape
    assert np.abs(logits - want).max() <= F32_TOL
    assert np.array_equal(picks, logits.argmax(-1))                       # sampling kernel: bit-exact on its own logits
    ok = confident_rows(want, 4 * F32_TOL)
    assert ok.mean() > 0.8 and np.array_equal(picks[ok], g[f"n_{tag}_tokens"][ok])
    # the free-running loop reproduces the ids (ties aside, which the margin check above bounds)
    out = m.generate(g["prompt"], c["gen"])
    first_bad = np.argmin(ok[0]) if not ok[0].all() else c["gen"]
    assert np.array_equal(out[0, :first_bad], g[f"n_{tag}_tokens"][0, :first_bad])


@pytest.mark.parametrize("tag", ["plain", "stress"])
def test_char_gpt_reference_mode_matches_golden(backend, tag):
    """Mode R = the reference's own forward: no mask, ReLU, full re-forward per id."""
    g = np.load(os.path.join(GOLD, "char_gpt.npz"))
    c = O.CONFIGS[0]
    cfg = c["cfg"]
    params = O.make_params(cfg, O.config_seed(0), stress=(tag == "stress"))
    m = model_for(backend, cfg, params, causal=False, act="relu")
    ids = np.concatenate([g["prompt"], g[f"r_{tag}_tokens"]], 1)
    want = g[f"r_{tag}_logits"]
    for i in range(c["gen"]):
        t = c["prompt"] + i
        lg = m.forward(ids[:, :t].astype(np.float32))
        assert np.abs(lg[:, -1] - want[:, i]).max() <= F32_TOL
    full = m.forward(ids[:, :64].astype(np.float32))
    assert np.abs(full - O.forward(params, cfg, ids[:, :64], causal=False, act="relu")).max() <= F32_TOL
    ok = confident_rows(want, 4 * F32_TOL)[0]
    first_bad = np.argmin(ok) if not ok.all() else c["gen"]
    out = m.generate(g["prompt"][0], c["gen"])
    assert np.array_equal(out[:first_bad], g[f"r_{tag}_tokens"][0, :first_bad])
    with pytest.raises(rg.Unsupported):
        m.prefill(g["prompt"])
        m.decode_step(np.array([1]))


def test_reference_mode_slides_its_window(backend):
    """generate past block_size keeps the last block_size ids (src/wasm_api.rs:103-104)."""
    cfg = O.GptConfig(8, 20, 1, 2, 64)
    params = O.make_params(cfg, 9)
    m = model_for(backend, cfg, params, causal=False, act="relu")
    lo = []
    want = O.generate_reference(params, cfg, [1, 2, 3, 4, 5, 6], 6, logits_out=lo)
    got = m.generate(np.array([1, 2, 3, 4, 5, 6]), 6)
    gaps = [np.sort(l)[-1] - np.sort(l)[-2] for l in lo]
    if min(gaps) > 4 * F32_TOL:
        assert list(got) == want


# ---- configuration 1: GPT-2-small shape, vocab 1024, f32 (the benchmark workload)
def test_gpt2_small_every_step(backend):
    c = O.CONFIGS[1]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    params = O.make_params(cfg, O.config_seed(1))
    g = np.load(os.path.join(GOLD, "gpt2_small_sample.npz"))
    m = model_for(backend, cfg, params)
    ids = np.concatenate([g["prompt"], g["n_tokens"]], 1)
    logits, picks = teacher_forced(m, ids, P)
    want = O.teacher_forced_logits(params, cfg, ids, True, "gelu_tanh", P)
    assert logits.shape == (1, G, cfg.vocab_size)
    err = np.abs(logits - want).max(-1)
    assert err.max() <= F32_TOL, (err.max(), int(err.argmax()))
    assert np.abs(logits[:, g["steps"]] - g["n_logits"]).max() <= F32_TOL     # committed fixture
    assert np.array_equal(picks, logits.argmax(-1))
    ok = confident_rows(want, 4 * F32_TOL)
    assert ok.mean() > 0.9 and np.array_equal(picks[ok], g["n_tokens"][ok])
    # device-resident loop == host-driven loop
    m.prefill(g["prompt"])
    m.decode_run(G - 1)
    run = m.read_tokens(P, G, 1)
    first_bad = np.argmin(ok[0]) if not ok[0].all() else G
    assert np.array_equal(run[0, :first_bad], g["n_tokens"][0, :first_bad])
    # rewinding to the prompt and running again is idempotent, bit for bit
    m.rewind(P)
    m.decode_run(G - 1)
    assert np.array_equal(m.read_tokens(P, G, 1), run)
    out = m.generate(g["prompt"][0], G)
    assert np.array_equal(out, run[0])


def test_gpt2_small_reference_mode(backend):
    c = O.CONFIGS[1]
    cfg, P = c["cfg"], c["prompt"]
    params = O.make_params(cfg, O.config_seed(1))
    g = np.load(os.path.join(GOLD, "gpt2_small_sample.npz"))
    m = model_for(backend, cfg, params, causal=False, act="relu")
    lg = m.forward(g["prompt"].astype(np.float32))
    assert np.abs(lg[:, -1] - g["r_prompt_last_logits"]).max() <= F32_TOL
    want = O.forward(params, cfg, g["prompt"], causal=False, act="relu")
    assert np.abs(lg - want).max() <= F32_TOL
    lo = []
    toks = O.generate_reference(params, cfg, g["prompt"][0], 3, logits_out=lo)
    got = m.generate(g["prompt"][0], 3)
    if min(np.sort(l)[-1] - np.sort(l)[-2] for l in lo) > 4 * F32_TOL:
        assert list(got) == toks


# ---- bf16-weight mode and batches (configurations 2-4 at reduced depth / batch)
@pytest.mark.parametrize("shape", [(50257, 768, 12, 2), (50257, 1024, 16, 2), (5003, 1600, 25, 2)])
def test_bf16_batched_steps(backend, shape):
    """bf16 weights, GPT-2 small / medium / XL widths at reduced depth, against the ORACLE for every form of the token
    step: batches 1, 2, 4 run in the persistent kernel, batch 5 as separate launches."""
    V, D, H, L = shape
    cfg = O.GptConfig(64, V, L, H, D)
    P, G = 24, 6
    params = O.make_params(cfg, 77, stress=True, bf16=True)
    m = model_for(backend, cfg, params, dtype="bf16", max_batch=8)
    for B in (1, 2, 4, 5):
        prompt = O.make_prompt(cfg, 77 + B, B, P)
        toks, want = O.generate_causal(params, cfg, prompt, G)
        ids = np.concatenate([prompt, toks], 1)
        logits, picks = teacher_forced(m, ids, P)
        assert_bf16_close(logits, want, f"D={D} H={H} batch {B}")
        assert np.array_equal(picks, logits.argmax(-1))


@pytest.mark.parametrize("shape", [(1024, 16), (1600, 25)])
def test_f32_persistent_kernel_wide_models(backend, shape):
    """The persistent kernel (batches 1, 2, 4) on the medium and XL widths, f32, 2 layers, against the oracle."""
    D, H = shape
    cfg = O.GptConfig(48, 3001, 2, H, D)
    params = O.make_params(cfg, 31, stress=True)
    m = model_for(backend, cfg, params, max_batch=4)
    for B in (1, 2, 4):
        prompt = O.make_prompt(cfg, 31 + B, B, 11)
        toks, want = O.generate_causal(params, cfg, prompt, 8)
        logits, picks = teacher_forced(m, np.concatenate([prompt, toks], 1), 11)
        assert np.abs(logits - want).max() <= F32_TOL, (D, B, float(np.abs(logits - want).max()))
        assert np.array_equal(picks, logits.argmax(-1))
        l0 = backend.launch_count
        m.rewind(11)
        m.decode_run(6)
        backend.synchronize()
        assert backend.launch_count - l0 <= 3          # the persistent kernel took it: one launch for 6 steps


def test_f32_batched_steps_odd_sizes(backend):
    cfg = O.GptConfig(40, 301, 2, 3, 96)   # head_dim 32, nothing a multiple of the tile sizes
    for B in (1, 2, 3, 7, 9):
        params = O.make_params(cfg, 5, stress=True)
        prompt = O.make_prompt(cfg, 5 + B, B, 9)
        toks, want = O.generate_causal(params, cfg, prompt, 31)   # fills the context to the last row
        m = model_for(backend, cfg, params, max_batch=9)
        logits, picks = teacher_forced(m, np.concatenate([prompt, toks], 1), 9)
        assert np.abs(logits - want).max() <= F32_TOL
        assert np.array_equal(picks, logits.argmax(-1))


# ---- size-independent properties at full size (configuration 2: vocab 50257, bf16, batch 64)
def test_full_size_cache_is_consistent_with_recompute(backend):
    c = O.CONFIGS[2]
    cfg = c["cfg"]
    B, P, G = 64, 256, 8
    params = O.make_params(cfg, O.config_seed(2), bf16=True)
    prompt = O.make_prompt(cfg, O.config_seed(2), B, P)
    m = model_for(backend, cfg, params, dtype="bf16", max_batch=B)
    out = m.generate(prompt, G)
    assert out.shape == (B, G) and out.max() < cfg.vocab_size
    assert np.array_equal(out, m.generate(prompt, G))                      # deterministic
    # a fresh prompt pass over prompt+generated reproduces the step logits (cache == recompute)
    ids = np.concatenate([prompt, out], 1)
    lg_pre, pk_pre = m.prefill(ids[:, :P + G - 1])
    m.prefill(ids[:, :P])
    for t in range(P, P + G - 1):
        lg_step, pk_step = m.decode_step(ids[:, t])
    assert_bf16_close(lg_step, lg_pre, "batch 64: cached step vs prompt pass")
    # shards of the batch are independent: sequence b alone gives the same ids
    solo = m.generate(prompt[7:9], G)
    assert np.array_equal(solo, out[7:9])
    # the oracle on two of the 64 sequences, first step
    want = O.forward(params, cfg, prompt[:2], causal=True, act="gelu_tanh", last_only=True)[:, 0]
    lg0, _ = m.prefill(prompt[:2])
    assert_bf16_close(lg0, want, "full-size prompt pass")


# ---- error behaviour of the model interface
def test_model_errors(backend):
    cfg = O.GptConfig(16, 30, 1, 2, 64)
    params = O.make_params(cfg, 1)
    with pytest.raises(rg.InvalidInput):        # assert embed_dim % num_heads == 0, src/nn/attention.rs:38-41
        rg.GPTModel(backend, rg.GptConfig(16, 30, 1, 3, 64))
    m = rg.GPTModel(backend, rg.GptConfig(16, 30, 1, 2, 64, max_batch=2))
    with pytest.raises(rg.InvalidInput):        # parameters not loaded
        m.forward(np.zeros((1, 4), np.float32))
    with pytest.raises(rg.ShapeError):          # "Mismatch in number of parameter tensors", src/wasm_api.rs:186
        m.load_parameters(params[:-1])
    bad = list(params)
    bad[2] = np.zeros((64, 63), np.float32)
    with pytest.raises(rg.ShapeError):          # "Mismatch in tensor shape", src/wasm_api.rs:190
        m.load_parameters(bad)
    m.load_parameters(params)
    with pytest.raises(rg.InvalidInput):        # id >= vocab, src/ops/embedding.rs:51-56
        m.forward(np.array([[30.0]], np.float32))
    with pytest.raises(rg.InvalidInput):        # T > block_size: position lookup out of range
        m.forward(np.zeros((1, 17), np.float32))
    with pytest.raises(rg.InvalidInput):
        m.prefill(np.zeros((3, 4), np.uint32))  # batch > max_batch
    with pytest.raises(rg.InvalidInput):
        m.decode_step(np.array([1]))            # no context yet
    m.prefill(np.zeros((1, 15), np.uint32))
    with pytest.raises(rg.InvalidInput):
        m.decode_step(np.array([1, 2]))         # two ids for a context of one sequence
    m.prefill(np.zeros((1, 16), np.uint32))
    with pytest.raises(rg.ContextFull):
        m.decode_step(np.array([1]))
    with pytest.raises(rg.ContextFull):
        m.generate(np.zeros(10, np.uint32), 8)
    assert m.generate(np.zeros(10, np.uint32), 7).shape == (7,)
    # still usable afterwards
    lg = m.forward(np.array([[1, 2, 3]], np.float32))
    assert np.abs(lg - O.forward(params, cfg, np.array([[1, 2, 3]]), causal=True, act="gelu_tanh")).max() <= F32_TOL


# ---- stochastic sampling: top-k filter, temperature, inverse-CDF draw (src/wasm_api.rs:120-156)
def test_topk_temperature_sampling(backend):
    cfg = O.GptConfig(40, 301, 2, 3, 96)
    params = O.make_params(cfg, 5, stress=True)
    B, P, G = 3, 9, 14
    prompt = O.make_prompt(cfg, 8, B, P)
    m = model_for(backend, cfg, params, max_batch=4)
    for temperature, top_k, seed in ((0.9, 7, 5), (1.3, 0, 11), (0.7, 301, 3), (2.0, 40, 99)):
        out = m.generate(prompt, G, temperature=temperature, top_k=top_k, seed=seed)
        assert np.array_equal(out, m.generate(prompt, G, temperature=temperature, top_k=top_k, seed=seed))   # reproducible
        ids = np.concatenate([prompt, out], 1)
        logits, _ = teacher_forced(m, ids, P)            # the rows each draw was made from
        agree = agree_wi = 0
        for b in range(B):
            for i in range(G):
                lg = logits[b, i].astype(np.float64)
                u = O.uniform_draw(seed, b, i)
                keep = np.ones(cfg.vocab_size, bool)
                if 0 < top_k < cfg.vocab_size:
                    keep[:] = False
                    keep[np.argsort(-lg, kind="stable")[:top_k]] = True
                pr = np.where(keep, np.exp((lg - lg.max()) / temperature), 0.0)
                cdf = np.cumsum(pr) / pr.sum()
                tok = int(out[b, i])
                assert keep[tok]
                lo = cdf[tok - 1] if tok else 0.0
                assert lo - 1e-5 <= u <= cdf[tok] + 1e-5          # the inverse-CDF walk stopped at the right id
                agree += O.sample_topk(logits[b, i], temperature, top_k, u) == tok
                if top_k == 0:      # KnowledgeManager::generate's WeightedIndex draw: same CDF, same id away from boundaries
                    agree_wi += O.sample_weighted(logits[b, i], temperature, u) == tok
        assert agree >= B * G - 2                                   # the oracle's f32 walk agrees away from boundaries
        assert top_k != 0 or agree_wi >= B * G - 2
    assert not np.array_equal(m.generate(prompt, G, temperature=1.0, top_k=50, seed=1),
                              m.generate(prompt, G, temperature=1.0, top_k=50, seed=2))
    assert np.array_equal(m.generate(prompt, G, temperature=5.0, top_k=1, seed=7), m.generate(prompt, G))  # top_k 1 is greedy
    with pytest.raises(rg.InvalidInput):
        m.generate(prompt, G, temperature=0.0, top_k=5)
    # the reference's loop (no mask, full re-forward) with sampling
    mr = model_for(backend, cfg, params, causal=False, act="relu", max_batch=4)
    a = mr.generate(prompt, 6, temperature=0.8, top_k=10, seed=4)
    assert a.shape == (B, 6) and np.array_equal(a, mr.generate(prompt, 6, temperature=0.8, top_k=10, seed=4))


# ---- the two token-step implementations compute the same thing
def test_persistent_kernel_equals_graph_step(backend, monkeypatch):
    cfg = O.GptConfig(96, 1024, 3, 4, 256)
    params = O.make_params(cfg, 21, stress=True)
    for B in (1, 2, 4):
        prompt = O.make_prompt(cfg, 21 + B, B, 17)
        monkeypatch.delenv("RG_B200_DECODE", raising=False)
        a = model_for(backend, cfg, params, max_batch=4)        # persistent cooperative kernel
        monkeypatch.setenv("RG_B200_DECODE", "graph")
        b = model_for(backend, cfg, params, max_batch=4)        # CUDA-graph step (the variable is read at load time)
        monkeypatch.delenv("RG_B200_DECODE", raising=False)
        ids = np.concatenate([prompt, a.generate(prompt, 40)], 1)
        la, pa = teacher_forced(a, ids, 17)
        lb, pb = teacher_forced(b, ids, 17)
        assert np.abs(la - lb).max() <= 2e-5
        assert np.array_equal(pa, la.argmax(-1)) and np.array_equal(pb, lb.argmax(-1))
        l0 = backend.launch_count
        a.rewind(17)
        a.decode_run(30)
        backend.synchronize()
        assert backend.launch_count - l0 <= 3                    # one launch for 30 token steps
        tr_rows = a.read_trace()
        assert tr_rows.shape[1] == 12


# ---- the whole context window: every position up to block_size, both token-step implementations
@pytest.mark.parametrize("dtype,B", [("f32", 1), ("bf16", 4)])
def test_full_context_window(backend, monkeypatch, dtype, B):
    """GPT-2-small shape (the benchmark workload) driven to the last position of its 1024-token window: the
    persistent kernel (attention slices grow from one ring chunk to several) against the CUDA-graph step,
    teacher-forced on the persistent kernel's own ids; then the window is full."""
    cfg = O.CONFIGS[1]["cfg"]
    params = O.make_params(cfg, O.config_seed(1), bf16=(dtype == "bf16"))
    P = 24
    prompt = O.make_prompt(cfg, O.config_seed(1), B, P)
    monkeypatch.delenv("RG_B200_DECODE", raising=False)
    a = model_for(backend, cfg, params, dtype=dtype, max_batch=B)
    G = cfg.block_size - P + 1                                  # the last id is picked at position block_size - 1
    out = a.generate(prompt, G)
    assert out.shape == (B, G) and np.array_equal(out, a.generate(prompt, G))
    with pytest.raises(rg.ContextFull):
        a.generate(prompt, G + 1)
    monkeypatch.setenv("RG_B200_DECODE", "graph")
    b = model_for(backend, cfg, params, dtype=dtype, max_batch=B)
    monkeypatch.delenv("RG_B200_DECODE", raising=False)
    ids = np.concatenate([prompt, out], 1)[:, :cfg.block_size]
    lb, pb = teacher_forced(b, ids, P)                          # logits that predict ids[:, P:], graph step
    tol = 1e-4 if dtype == "f32" else 2e-3
    sure = confident_rows(lb, 10 * tol)
    assert np.array_equal(pb[sure], ids[:, P:][sure])           # same picks wherever the top-2 gap is clear
    assert sure.mean() > 0.5
    la, pa = teacher_forced(a, ids, P)                          # the same steps, one launch of the persistent kernel each
    assert np.abs(la - lb).max() <= tol
    assert np.array_equal(pa, la.argmax(-1))
    assert np.array_equal(pa, out[:, :G - 1])                   # stepwise picks == the ids of the single long run


# ---- the GEMM-form token step (batch >= 8, bf16): fused kernels between the projections == one kernel per operation
def test_fused_rows_step_equals_plain_rows_step(backend, monkeypatch):
    cfg = O.GptConfig(64, 1000, 2, 4, 256)
    params = O.make_params(cfg, 23, stress=True, bf16=True)
    for B in (8, 19):
        prompt = O.make_prompt(cfg, 23 + B, B, 9)
        monkeypatch.delenv("RG_B200_ROWS_STEP", raising=False)
        a = model_for(backend, cfg, params, dtype="bf16", max_batch=B)
        ids = np.concatenate([prompt, a.generate(prompt, 20)], 1)
        la, pa = teacher_forced(a, ids, 9)
        monkeypatch.setenv("RG_B200_ROWS_STEP", "plain")
        b = model_for(backend, cfg, params, dtype="bf16", max_batch=B)
        lb, pb = teacher_forced(b, ids, 9)
        monkeypatch.delenv("RG_B200_ROWS_STEP", raising=False)
        scale = np.abs(lb).max(-1, keepdims=True)
        # same arithmetic up to the order of the f32 sums, which moves some activations by one bf16 step (2^-8 relative)
        assert (np.abs(la - lb) / scale).max() <= 8e-3
        assert np.array_equal(pa, la.argmax(-1)) and np.array_equal(pb, lb.argmax(-1))
        want = O.teacher_forced_logits(params, cfg, ids, True, "gelu_tanh", 9)
        assert_bf16_close(la, want, f"fused rows step batch {B}")


# ---- prompt pass in bf16 mode: tensor-core projections and attention against the CUDA-core kernels and the oracle
@pytest.mark.parametrize("causal", [True, False])
def test_prompt_pass_tensor_core_kernels(backend, monkeypatch, causal):
    """Ragged sizes on purpose: prompt lengths that are not multiples of the 128-row tiles, a block_size that is not
    one either (key tiles then run past the end of a head's cache rows), several sequences and heads."""
    cfg = O.GptConfig(330, 777, 2, 4, 256)          # head_dim 64
    act = "gelu_tanh" if causal else "relu"
    params = O.make_params(cfg, 29, stress=True, bf16=True)
    for B, T in ((3, 77), (2, 130), (1, 257), (2, 330)):
        ids = O.make_prompt(cfg, 29 + T, B, T)
        monkeypatch.delenv("RG_B200_PREFILL", raising=False)
        a = model_for(backend, cfg, params, causal=causal, act=act, dtype="bf16", max_batch=B)
        la = a.forward(ids.astype(np.float32))
        monkeypatch.setenv("RG_B200_PREFILL", "simt")
        b = model_for(backend, cfg, params, causal=causal, act=act, dtype="bf16", max_batch=B)
        lb = b.forward(ids.astype(np.float32))
        monkeypatch.delenv("RG_B200_PREFILL", raising=False)
        want = O.forward(params, cfg, ids, causal=causal, act=act)
        assert_bf16_close(lb, want, f"prompt pass CUDA cores B={B} T={T}")
        assert_bf16_close(la, want, f"prompt pass tensor cores B={B} T={T}")
        assert np.isfinite(la).all()
        # launch counts tell that the tensor-core attention ran: one more kernel per block (the Q / V^T preparation)
        l0 = backend.launch_count
        a.forward(ids.astype(np.float32))
        n_tc = backend.launch_count - l0
        l0 = backend.launch_count
        b.forward(ids.astype(np.float32))
        assert n_tc != backend.launch_count - l0
