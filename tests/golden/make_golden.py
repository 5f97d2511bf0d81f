"""Writes tests/golden/*.npz from the CPU oracle (oracle/gpt_oracle.py).

The reference cannot be executed here (no Rust toolchain), so these vectors pin
the ORACLE, not the reference: they guard the restatement against accidental
change and give the GPU tests a fixture that does not depend on the BLAS build of
the machine they run on.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import gpt_oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def char_gpt():
    """Configuration 0 (char GPT), both modes, every one of the 48 steps."""
    c = O.CONFIGS[0]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    seed = O.config_seed(0)
    out = {}
    for stress in (False, True):
        tag = "stress" if stress else "plain"
        params = O.make_params(cfg, seed, stress=stress)
        prompt = O.make_prompt(cfg, seed, 1, P)
        toks, logits = O.generate_causal(params, cfg, prompt, G, act="gelu_tanh")
        out[f"n_{tag}_tokens"] = toks
        out[f"n_{tag}_logits"] = logits.astype(np.float32)
        lo = []
        r = O.generate_reference(params, cfg, prompt[0], G, causal=False, act="relu", logits_out=lo)
        out[f"r_{tag}_tokens"] = np.asarray(r, np.uint32)[None, :]
        out[f"r_{tag}_logits"] = np.stack(lo)[None].astype(np.float32)
    out["prompt"] = O.make_prompt(cfg, seed, 1, P)
    np.savez_compressed(os.path.join(HERE, "char_gpt.npz"), **out)


def gpt2_small_sample():
    """Configuration 1 (GPT-2-small shape, vocab 1024): greedy ids of all 256
    steps, logits of 6 of them (mode N), and the last-row logits of the prompt in
    mode R."""
    c = O.CONFIGS[1]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    seed = O.config_seed(1)
    params = O.make_params(cfg, seed)
    prompt = O.make_prompt(cfg, seed, 1, P)
    toks, logits = O.generate_causal(params, cfg, prompt, G, act="gelu_tanh")
    steps = np.array([0, 1, 2, 100, 200, 255])
    r_last = O.forward(params, cfg, prompt, causal=False, act="relu", last_only=True)[:, 0]
    np.savez_compressed(os.path.join(HERE, "gpt2_small_sample.npz"), prompt=prompt, n_tokens=toks, steps=steps,
                        n_logits=logits[:, steps].astype(np.float32), r_prompt_last_logits=r_last.astype(np.float32))


if __name__ == "__main__":
    char_gpt()
    gpt2_small_sample()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
