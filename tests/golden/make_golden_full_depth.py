"""Writes tests/golden/full_depth.npz: oracle logits of the first steps of the two full-depth configurations that are
too slow to run through the oracle inside a GPU test (GPT-2-medium shape: 24 blocks, d_model 1024, 16 heads;
GPT-2-XL shape: 48 blocks, d_model 1600, 25 heads; vocabulary 50257, bf16-rounded weights, 2 sequences).

    python tests/golden/make_golden_full_depth.py        (a few minutes and ~20 GB of host memory for the XL shape)

Stored per shape: the prompt [2,6], the oracle's 5 greedy ids per sequence, every 61st column of the 5 logits rows,
and each row's largest |logit| and arg-max.  The weights are not stored: the test draws them again from the seed."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import gpt_oracle as O  # noqa: E402

SHAPES = {"medium": (1024, 16, 24), "xl": (1600, 25, 48)}
SEED, B, P, G, STRIDE = 41, 2, 6, 5, 61


def main() -> None:
    out = {"stride": np.int64(STRIDE), "seed": np.int64(SEED)}
    for name, (D, H, L) in SHAPES.items():
        cfg = O.GptConfig(32, 50257, L, H, D)
        params = O.make_params(cfg, SEED, bf16=True)
        prompt = O.make_prompt(cfg, SEED, B, P)
        toks, logits = O.generate_causal(params, cfg, prompt, G)
        out[f"{name}_prompt"] = prompt
        out[f"{name}_tokens"] = toks
        out[f"{name}_logits_sampled"] = np.ascontiguousarray(logits[:, :, ::STRIDE])
        out[f"{name}_row_absmax"] = np.abs(logits).max(-1)
        out[f"{name}_row_top2_gap"] = np.sort(logits, -1)[..., -1] - np.sort(logits, -1)[..., -2]
        del params
        print(name, "done", flush=True)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "full_depth.npz"), **out)


if __name__ == "__main__":
    main()
