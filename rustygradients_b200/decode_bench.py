"""Token-step time for a batch of sequences on one GPU.

    python -m rustygradients_b200.decode_bench [--batch 64] [--prompt 256] [--steps 64] [--dtype bf16] [--vocab 50257]
                                               [--layers 12] [--d-model 768] [--heads 12]

GPT-2-small shape by default (full vocabulary, bf16 weights: the batched configuration), seeded random
weights.  Prints one JSON line: microseconds per step, tokens/s and the algorithmic GB/s of the step
(weights once + the KV cache of every sequence) against nothing: the caller compares it with the HBM peak.
Batches of 1, 2 and 4 run in the persistent token-loop kernel, larger ones in the CUDA-graph step."""
from __future__ import annotations

import argparse
import json

import numpy as np


def main() -> None:
    import torch

    from . import B200Backend, GptConfig, GPTModel

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--d-model", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12)
    a = ap.parse_args()
    be = B200Backend(0)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", 0))
    m = GPTModel(be, GptConfig(1024, a.vocab, a.layers, a.heads, a.d_model, weight_dtype=a.dtype, max_batch=a.batch))
    rng = np.random.Generator(np.random.PCG64(9))
    m.load_parameters([(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) if s[0] != 1 or s[1] == a.vocab
                       else np.ones(s, np.float32) for s in m.parameter_shapes()])
    prompt = rng.integers(0, a.vocab, size=(a.batch, a.prompt), dtype=np.uint32)
    m.prefill(prompt, want_logits=False)
    m.decode_run(min(a.steps, 40))  # warm-up: graph capture / placement search
    times = []
    for _ in range(3):
        m.rewind(a.prompt)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        m.decode_run(a.steps)
        e1.record(stream)
        be.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / a.steps)
    us = min(times)
    by = m.decode_step_bytes(a.batch, a.prompt + a.steps / 2)
    print(json.dumps({"batch": a.batch, "dtype": a.dtype, "prompt": a.prompt, "steps": a.steps, "us_per_step": us,
                      "tokens_per_s": a.batch / (us * 1e-6), "algorithmic_gb_per_s": by / (us * 1e-6) / 1e9,
                      "launches": be.launch_count}))


if __name__ == "__main__":
    main()
