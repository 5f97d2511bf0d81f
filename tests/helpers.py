"""Shared helpers of the GPU parity tests."""
import numpy as np

import rustygradients_b200 as rg
from oracle import gpt_oracle as O

F32_TOL = 1e-3      # max |logit difference| in f32 mode, every step
BF16_REL_TOL = 2e-2  # relative to the largest |logit| of the row, bf16-weight mode


def model_for(backend, cfg: O.GptConfig, params, causal=True, act="gelu_tanh", dtype="f32", max_batch=1):
    m = rg.GPTModel(backend, rg.GptConfig(cfg.block_size, cfg.vocab_size, cfg.num_layers, cfg.num_heads,
                                          cfg.embedding_dim, causal=causal, activation=act, weight_dtype=dtype,
                                          max_batch=max_batch))
    m.load_parameters(params)
    return m


def teacher_forced(model, ids: np.ndarray, first: int):
    """Prefill ids[:, :first], then feed ids[:, first:] one token at a time.
    Returns (logits [B, T-first, V], picks [B, T-first]) = what predicts ids[:, first:]
    plus... exactly the rows the oracle's teacher_forced_logits returns."""
    B, T = ids.shape
    lg, pk = model.prefill(ids[:, :first])
    logits, picks = [lg], [pk]
    for t in range(first, T - 1):
        lg, pk = model.decode_step(ids[:, t])
        logits.append(lg)
        picks.append(pk)
    return np.stack(logits, 1), np.stack(picks, 1)


def confident_rows(logits: np.ndarray, margin: float):
    """Rows whose top-2 gap exceeds margin (argmax there must agree bit-exactly)."""
    s = np.sort(logits, axis=-1)
    return (s[..., -1] - s[..., -2]) > margin
