"""CPU oracle for the GPT token loop of RustyGradients (crate rusty-gradients 0.2.0).

TEST INFRASTRUCTURE ONLY.  This module is the checker: tests, the smoke entry
and the benchmark's CPU-baseline leg may import it; the product path (the CUDA
library and its host mirror) never does.

It is a numpy-f32 restatement of the reference's forward pass and token loop.
Every function names the reference lines it follows.  The reference itself
cannot be built here (no Rust toolchain; its numeric dependencies
ndarray 0.16.1 / matrixmultiply 0.3.10 / rand 0.8.5 are only named in
Cargo.lock), so:

  PARITY UNPINNED at model level - the reference has no test that pins a
  forward logit or a generated token (tests/nn_test.rs only checks that
  gradients are non-zero).  What the reference does pin - the op-level known
  answers in src/backend/cuda.rs:553-570, src/backend/fused.rs:228-259,
  src/backend/simd.rs:167-187 and the ramp inputs with tolerances of
  examples/cuda_kernels_test.rs:146-256 - is reproduced in `reference_kats()`
  and checked by the CPU tests.  GEMM summation order (matrixmultiply's
  micro-kernel vs OpenBLAS here) is not pinned by anything in the reference.

Two switches separate the reference's model from the path a KV cache needs:
  causal=False, act="relu"      -> "mode R": exactly GPTModel::forward
  causal=True,  act="gelu_tanh" -> "mode N": causal mask + tanh-GELU, the only
                                    two deltas; everything else is shared code.
"""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

F32 = np.float32
LN_EPS = F32(1e-5)  # src/nn/norm.rs:8,53-57


# ----------------------------------------------------------------------------
# configuration and seeded parameters
# ----------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class GptConfig:
    """Field names follow src/models/gpt.rs:8-14."""
    block_size: int
    vocab_size: int
    num_layers: int
    num_heads: int
    embedding_dim: int

    @property
    def head_dim(self) -> int:
        return self.embedding_dim // self.num_heads

    @property
    def hidden_dim(self) -> int:  # src/models/gpt.rs:37
        return 4 * self.embedding_dim

    @property
    def n_params_tensors(self) -> int:
        return 2 + 16 * self.num_layers + 4


# The five workload shapes (index = position in the list of configurations).
CONFIGS = {
    0: dict(cfg=GptConfig(64, 52, 4, 4, 128), batch=1, prompt=16, gen=48, dtype="f32"),
    1: dict(cfg=GptConfig(1024, 1024, 12, 12, 768), batch=1, prompt=128, gen=256, dtype="f32"),
    2: dict(cfg=GptConfig(1024, 50257, 12, 12, 768), batch=64, prompt=256, gen=256, dtype="bf16"),
    3: dict(cfg=GptConfig(1024, 50257, 24, 16, 1024), batch=256, prompt=512, gen=512, dtype="bf16"),
    4: dict(cfg=GptConfig(1024, 50257, 48, 25, 1600), batch=32, prompt=512, gen=256, dtype="bf16"),
}


def config_seed(cfg_index: int) -> int:
    return 20240 + cfg_index


def param_shapes(cfg: GptConfig) -> List[Tuple[int, ...]]:
    """Shapes in `parameters()` order: src/models/gpt.rs:85-93 ->
    src/nn/transformer.rs:68-75 -> src/nn/attention.rs:107-114,
    src/nn/norm.rs:60-62, src/nn/feedforward.rs:51-56, src/nn/linear.rs:59-61."""
    V, D, C, F = cfg.vocab_size, cfg.embedding_dim, cfg.block_size, cfg.hidden_dim
    shapes: List[Tuple[int, ...]] = [(V, D), (C, D)]
    for _ in range(cfg.num_layers):
        shapes += [(D, D), (1, D)] * 4          # Wq bq Wk bk Wv bv Wo bo
        shapes += [(1, D), (1, D)]              # ln1 gamma beta
        shapes += [(D, F), (1, F), (F, D), (1, D)]  # W1 b1 W2 b2
        shapes += [(1, D), (1, D)]              # ln2 gamma beta
    shapes += [(1, D), (1, D), (D, V), (1, V)]  # final ln, head W, head b
    return shapes


def _is_ln_gamma(i: int, cfg: GptConfig) -> bool:
    n = cfg.n_params_tensors
    if i == n - 4:
        return True
    if 2 <= i < n - 4:
        return (i - 2) % 16 in (8, 14)
    return False


def _is_ln_beta(i: int, cfg: GptConfig) -> bool:
    n = cfg.n_params_tensors
    if i == n - 3:
        return True
    if 2 <= i < n - 4:
        return (i - 2) % 16 in (9, 15)
    return False


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round f32 -> bf16 (nearest even) and return the value up-cast to f32."""
    u = np.ascontiguousarray(a, dtype=F32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(F32)


def make_params(cfg: GptConfig, seed: int, stress: bool = False,
                bf16: bool = False) -> List[np.ndarray]:
    """Seeded stand-in for a trained model.  Every embedding table, Linear
    weight and Linear bias ~ N(0, 0.02); LayerNorm gamma=1, beta=0 (the
    reference's defaults, src/nn/norm.rs:37-39).  `stress` perturbs gamma and
    beta so that a kernel that ignores them cannot pass.  `bf16` rounds every
    tensor the engine keeps in bf16 (all matrices and embedding tables) to
    bf16 and returns them as f32."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for i, shp in enumerate(param_shapes(cfg)):
        if _is_ln_gamma(i, cfg):
            a = np.ones(shp, F32)
            if stress:
                a = (a + rng.standard_normal(shp, dtype=F32) * F32(0.02)).astype(F32)
        elif _is_ln_beta(i, cfg):
            a = np.zeros(shp, F32)
            if stress:
                a = (rng.standard_normal(shp, dtype=F32) * F32(0.02)).astype(F32)
        else:
            a = (rng.standard_normal(shp, dtype=F32) * F32(0.02)).astype(F32)
            if bf16 and shp[0] != 1:
                a = bf16_round(a)
        out.append(np.ascontiguousarray(a))
    return out


def make_prompt(cfg: GptConfig, seed: int, batch: int, length: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed + 7919))
    return rng.integers(0, cfg.vocab_size, size=(batch, length), dtype=np.uint32)


# ----------------------------------------------------------------------------
# ops (forward halves only)
# ----------------------------------------------------------------------------
def embedding(ids: np.ndarray, table: np.ndarray) -> np.ndarray:
    """src/ops/embedding.rs:25-66: ids [B,T] (f32-valued in the reference, cast
    `as usize`), table [V,D] -> [B,T,D]; id >= V is InvalidInput."""
    if ids.ndim != 2 or table.ndim != 2:
        raise ValueError("DimensionError: embedding expects 2-D ids and 2-D table")
    idx = ids.astype(np.int64)
    if idx.size and (idx.max() >= table.shape[0] or idx.min() < 0):
        raise IndexError("InvalidInput: index out of bounds for vocabulary size")
    return table[idx]


def layernorm_two_pass(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray,
                       eps: float = LN_EPS) -> np.ndarray:
    """src/ops/norm.rs:41-52: mean, biased variance of (x-mean), eps inside the
    sqrt, then 1/sqrt, times gamma plus beta; gamma/beta are [1,D]."""
    x = x.astype(F32, copy=False)
    mean = x.mean(axis=-1, keepdims=True, dtype=F32)
    xm = x - mean
    var = (xm * xm).mean(axis=-1, keepdims=True, dtype=F32)
    inv = F32(1.0) / np.sqrt(var + F32(eps))
    return (xm * inv * gamma.reshape(-1) + beta.reshape(-1)).astype(F32)


def layernorm_welford(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray,
                      eps: float = LN_EPS) -> np.ndarray:
    """src/backend/fused.rs:22-144: one-pass Welford mean / M2 per row, then
    the same normalisation.  Pure-Python inner loop: small inputs only."""
    x2 = x.reshape(-1, x.shape[-1]).astype(F32)
    out = np.empty_like(x2)
    g, b = gamma.reshape(-1), beta.reshape(-1)
    for r in range(x2.shape[0]):
        mean, m2 = F32(0), F32(0)
        for i, v in enumerate(x2[r]):
            d = v - mean
            mean = F32(mean + d / F32(i + 1))
            m2 = F32(m2 + d * (v - mean))
        var = F32(m2 / F32(x2.shape[1]))
        inv = F32(1.0) / np.sqrt(F32(var + F32(eps)))
        out[r] = (x2[r] - mean) * inv * g + b
    return out.reshape(x.shape)


def linear(x: np.ndarray, w: np.ndarray, b: np.ndarray) -> np.ndarray:
    """src/nn/linear.rs:50-56 + src/ops/matmul.rs:51-72: y = x . W + b with
    W [in,out] and b [1,out] broadcast over rows (src/ops/basic_ops.rs:45-54)."""
    return (x.astype(F32, copy=False) @ w + b.reshape(-1)).astype(F32)


def softmax_lastaxis(s: np.ndarray) -> np.ndarray:
    """src/ops/elementwise.rs:144-157: subtract the row max, exp, divide by sum."""
    m = s.max(axis=-1, keepdims=True)
    e = np.exp((s - m).astype(F32)).astype(F32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)


def relu(x: np.ndarray) -> np.ndarray:
    """src/ops/elementwise.rs:61-62."""
    return np.maximum(x, F32(0)).astype(F32)


GELU_C0 = F32(0.7978845608)  # src/backend/fused.rs:152
GELU_C1 = F32(0.044715)      # src/backend/fused.rs:153


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """src/backend/fused.rs:151-175 / src/backend/cuda_kernels.cu:120-131."""
    x = x.astype(F32, copy=False)
    inner = GELU_C0 * (x + GELU_C1 * x * x * x)
    return (F32(0.5) * x * (F32(1.0) + np.tanh(inner).astype(F32))).astype(F32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    """src/backend/simd.rs (sigmoid_simd) / cuda_kernels.cu:107-116."""
    return (F32(1.0) / (F32(1.0) + np.exp(-x.astype(F32)))).astype(F32)


def activation(x: np.ndarray, act: str) -> np.ndarray:
    if act == "relu":
        return relu(x)
    if act == "gelu_tanh":
        return gelu_tanh(x)
    raise ValueError(act)


# ----------------------------------------------------------------------------
# model forward
# ----------------------------------------------------------------------------
def attention(n: np.ndarray, p: Sequence[np.ndarray], H: int, causal: bool,
              k_out: Optional[list] = None) -> np.ndarray:
    """src/nn/attention.rs:57-105.  p = [Wq,bq,Wk,bk,Wv,bv,Wo,bo]."""
    B, T, D = n.shape
    hd = D // H
    q = linear(n, p[0], p[1]).reshape(B, T, H, hd).transpose(0, 2, 1, 3)
    k = linear(n, p[2], p[3]).reshape(B, T, H, hd).transpose(0, 2, 1, 3)
    v = linear(n, p[4], p[5]).reshape(B, T, H, hd).transpose(0, 2, 1, 3)
    if k_out is not None:
        k_out.append((k.copy(), v.copy()))
    # scores, then the scale as a separate multiply (attention.rs:78-87)
    s = np.matmul(q, k.transpose(0, 1, 3, 2)).astype(F32)
    s = (s * F32(1.0 / math.sqrt(hd))).astype(F32)
    if causal:
        mask = np.triu(np.ones((T, T), dtype=bool), k=1)
        s = np.where(mask, F32(-np.inf), s)
    pr = softmax_lastaxis(s)
    a = np.matmul(pr, v).astype(F32).transpose(0, 2, 1, 3).reshape(B, T, D)
    return linear(a, p[6], p[7])


def block(x: np.ndarray, p: Sequence[np.ndarray], H: int, causal: bool, act: str,
          k_out: Optional[list] = None) -> np.ndarray:
    """src/nn/transformer.rs:51-65 (pre-LN residual block); p = the block's 16
    tensors in parameters() order."""
    n1 = layernorm_two_pass(x, p[8], p[9])
    x = (x + attention(n1, p[0:8], H, causal, k_out)).astype(F32)
    n2 = layernorm_two_pass(x, p[14], p[15])
    h = activation(linear(n2, p[10], p[11]), act)     # src/nn/feedforward.rs:40-48
    return (x + linear(h, p[12], p[13])).astype(F32)


def forward(params: Sequence[np.ndarray], cfg: GptConfig, ids: np.ndarray,
            causal: bool = False, act: str = "relu", last_only: bool = False,
            kv_out: Optional[list] = None, hidden_out: Optional[list] = None) -> np.ndarray:
    """src/models/gpt.rs:58-83: ids [B,T] -> logits [B,T,V] (or [B,1,V] when
    last_only, which computes only the row the token loop uses)."""
    ids = np.asarray(ids)
    B, T = ids.shape
    if T > cfg.block_size:
        raise IndexError("InvalidInput: position index out of bounds for block_size")
    tok = embedding(ids, params[0])
    pos = embedding(np.arange(T, dtype=np.int64)[None, :], params[1])
    x = (tok + pos).astype(F32)                       # broadcast over B
    for l in range(cfg.num_layers):
        base = 2 + 16 * l
        x = block(x, params[base:base + 16], cfg.num_heads, causal, act, kv_out)
        if hidden_out is not None:
            hidden_out.append(x.copy())
    n = cfg.n_params_tensors
    if last_only:
        x = x[:, -1:, :]
    x = layernorm_two_pass(x, params[n - 4], params[n - 3])
    return linear(x, params[n - 2], params[n - 1])


# ----------------------------------------------------------------------------
# token loop
# ----------------------------------------------------------------------------
def sample_topk(logits: np.ndarray, temperature: float, top_k: int, u: float) -> int:
    """src/wasm_api.rs:120-156 for one row of logits and one uniform draw u in
    [0,1): keep the top_k logits (others -> -inf), exp(l/temperature) with NO
    max subtraction, normalise when the sum is positive, inverse-CDF walk;
    falls through to id 0 when the walk never crosses u."""
    l = logits.astype(F32).copy()
    V = l.shape[0]
    if 0 < top_k < V:
        order = np.argsort(-l, kind="stable")
        l[order[top_k:]] = F32(-np.inf)
    with np.errstate(over="ignore"):
        p = np.exp((l / F32(temperature)).astype(F32)).astype(F32)
    s = F32(0)
    for v in p:
        s = F32(s + v)
    if s > 0:
        p = (p / s).astype(F32)
    c = F32(0)
    for i in range(V):
        c = F32(c + p[i])
        if F32(u) < c:
            return i
    return 0


def weighted_index_sample(weights: np.ndarray, u: float) -> int:
    """`WeightedIndex::new(&probs).sample(rng)` as src/bin/knowledge_manager.rs:196-198 uses it.  The algorithm
    lives in the `rand` crate (Cargo.toml pins rand 0.8.5; not vendored in the reference tree), restated from its
    published description: `new` keeps the running f32 sums of all weights but the last and the total; `sample` draws
    `chosen` uniformly in [0, total) and returns the number of kept sums that are <= chosen (a binary search).  `u` in
    [0,1) stands for the reference's unseeded `thread_rng` draw (chosen = u * total).  The weights are
    `exp(logit / temperature)` without normalisation or max subtraction."""
    w = np.asarray(weights, F32)
    c = F32(0)
    cum = np.empty(w.shape[0], F32)
    for i, v in enumerate(w):
        c = F32(c + v)
        cum[i] = c
    total = cum[-1]
    if not (total > 0) or not np.isfinite(total):
        raise ValueError("WeightedIndex::new fails on an all-zero, negative or non-finite weight vector")
    chosen = F32(F32(u) * total)
    return int(np.searchsorted(cum[:-1], chosen, side="right"))


def sample_weighted(logits: np.ndarray, temperature: float, u: float) -> int:
    """One step of KnowledgeManager::generate's draw (src/bin/knowledge_manager.rs:196-198) from a row of logits."""
    with np.errstate(over="ignore"):
        w = np.exp((logits.astype(F32) / F32(temperature)).astype(F32)).astype(F32)
    return weighted_index_sample(w, u)


_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_draw(seed: int, seq: int, step: int) -> float:
    """The engine's stand-in for the reference's unseeded `rng.gen::<f32>()`
    (src/wasm_api.rs:145): a counter-based draw in [0,1) with 24 random bits, keyed
    by (seed, sequence, step)."""
    h = _splitmix64((_splitmix64((seed ^ ((0xD1B54A32D192ED03 * (seq + 1)) & _M64)) & _M64) + step) & _M64)
    return float(np.float32(h >> 40) * np.float32(1.0 / 16777216.0))


def greedy_pick(logits_row: np.ndarray) -> int:
    """top_k = 1 in src/wasm_api.rs:123-156: only the maximum survives with
    probability 1.  Ties: lowest index (the reference's unstable sort leaves
    the tie order unspecified)."""
    return int(np.argmax(logits_row))


def generate_reference(params, cfg: GptConfig, prompt: Sequence[int], max_new: int,
                       causal: bool = False, act: str = "relu",
                       logits_out: Optional[list] = None) -> List[int]:
    """src/wasm_api.rs:97-163 with top_k=1: every step re-runs the full forward
    on the last block_size ids and reads the last row."""
    ids = [int(t) for t in prompt]
    out = []
    for _ in range(max_new):
        ctx = ids[max(0, len(ids) - cfg.block_size):]
        lg = forward(params, cfg, np.asarray(ctx, dtype=np.int64)[None, :],
                     causal=causal, act=act, last_only=True)[0, 0]
        if logits_out is not None:
            logits_out.append(lg.copy())
        nxt = greedy_pick(lg)
        ids.append(nxt)
        out.append(nxt)
    return out


def generate_causal(params, cfg: GptConfig, prompt: np.ndarray, max_new: int,
                    act: str = "gelu_tanh") -> Tuple[np.ndarray, np.ndarray]:
    """Greedy loop for mode N on a batch of prompts [B,P].  Under a causal mask
    row t of one full forward equals what a KV-cache step would produce, so the
    loop below (full forward per step, last row) is the exact, if slow, spec.
    Returns (tokens [B,max_new], logits [B,max_new,V])."""
    ids = np.asarray(prompt, dtype=np.int64)
    toks, lgs = [], []
    for _ in range(max_new):
        lg = forward(params, cfg, ids, causal=True, act=act, last_only=True)[:, 0]
        nxt = lg.argmax(axis=-1)
        toks.append(nxt)
        lgs.append(lg)
        ids = np.concatenate([ids, nxt[:, None]], axis=1)
    return np.stack(toks, 1).astype(np.uint32), np.stack(lgs, 1)


def teacher_forced_logits(params, cfg: GptConfig, ids: np.ndarray, causal: bool,
                          act: str, first: int) -> np.ndarray:
    """Logits that predict ids[:, first:], i.e. rows first-1 .. T-2.
    causal: one forward gives all rows.  non-causal (mode R): row t depends on
    the whole window, so each step is its own forward on ids[:, :t+1]."""
    ids = np.asarray(ids, dtype=np.int64)
    T = ids.shape[1]
    if causal:
        return forward(params, cfg, ids[:, :T], causal=True, act=act)[:, first - 1:T - 1]
    rows = [forward(params, cfg, ids[:, :t + 1], causal=False, act=act, last_only=True)[:, 0]
            for t in range(first - 1, T - 1)]
    return np.stack(rows, 1)


# ----------------------------------------------------------------------------
# byte model (algorithmic bytes of one decode step)
# ----------------------------------------------------------------------------
def decode_step_bytes(cfg: GptConfig, batch: int, mean_ctx: float,
                      weight_bytes: int, kv_bytes: int) -> float:
    """Block weights + biases + LN params, untied LM head + bias, final LN, one
    token row and one position row, plus K and V of every layer for every
    cached position of every sequence."""
    D, V, L = cfg.embedding_dim, cfg.vocab_size, cfg.num_layers
    w = L * (12 * D * D + 13 * D) + D * V + V + 2 * D + 2 * D
    return weight_bytes * w + batch * kv_bytes * 2 * L * D * mean_ctx


# ----------------------------------------------------------------------------
# the reference's own known answers
# ----------------------------------------------------------------------------
def reference_kats() -> dict:
    """Inputs and expected outputs that the reference's tests state in text."""
    ramp = np.arange(1024, dtype=F32)
    return {
        # src/backend/cuda.rs:553-570, examples/cuda_demo.rs:86-108
        "matmul_2x2": dict(a=np.array([[1, 2], [3, 4]], F32), b=np.array([[5, 6], [7, 8]], F32),
                           out=np.array([[19, 22], [43, 50]], F32), tol=1e-5),
        # src/backend/simd.rs:167-171
        "relu_4": dict(x=np.array([-2, -1, 1, 2], F32), out=np.array([0, 0, 1, 2], F32), tol=0.0),
        # tests/nn_test.rs:39-55 (forward values implied by the gradient mask)
        "relu_5": dict(x=np.array([-2, -1, 0, 1, 2], F32), out=np.array([0, 0, 0, 1, 2], F32), tol=0.0),
        # src/backend/simd.rs:182-187
        "sigmoid_0": dict(x=np.array([0], F32), out=np.array([0.5], F32), tol=1e-6),
        # src/backend/fused.rs:228-247: mean ~ 0 (1e-3), variance ~ 1 (0.1)
        "layernorm_1234": dict(x=np.array([[1, 2, 3, 4]], F32), gamma=np.ones((1, 4), F32),
                               beta=np.zeros((1, 4), F32), eps=1e-5),
        # src/backend/fused.rs:250-259: gelu(0) ~ 0, 0.8 < gelu(1) < 0.9
        "gelu_01": dict(x=np.array([0, 1], F32)),
        # examples/cuda_kernels_test.rs:146-256: ramps and per-op tolerances
        "ramp_add": dict(a=ramp * F32(0.01), b=ramp * F32(0.02), tol=1e-4),
        "ramp_mul": dict(a=ramp * F32(0.01), b=ramp * F32(0.02), tol=1e-4),
        "ramp_relu": dict(x=ramp * F32(0.01) - F32(0.5), tol=1e-5),
        "ramp_sigmoid": dict(x=ramp * F32(0.01) - F32(0.5), tol=1e-5),
        "ramp_exp": dict(x=ramp * F32(0.001) - F32(0.5), tol=1e-4),
        "ramp_softmax": dict(x=(ramp * F32(0.01)).reshape(8, 128), tol=1e-4),
    }
