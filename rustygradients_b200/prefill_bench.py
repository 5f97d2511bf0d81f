"""Prompt-pass throughput in bf16-weight mode (the tensor-core part of the path).

    python -m rustygradients_b200.prefill_bench [--batch 8] [--prompt 256] [--layers 12] [--iters 3]

Runs the prompt of `batch` sequences through a GPT-2-small-shaped model
(vocabulary 50257, d_model 768, 12 heads) with seeded random bf16 weights and
prints one JSON line with the time of the prompt pass and its TFLOP/s.  Set
RG_B200_PREFILL=simt to time the CUDA-core GEMM instead of the tcgen05 one."""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np

from . import B200Backend, GptConfig, GPTModel


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    V, D, H, C = 50257, 768, 12, 1024
    cfg = GptConfig(C, V, a.layers, H, D, weight_dtype="bf16", max_batch=a.batch)
    be = B200Backend(0)
    m = GPTModel(be, cfg)
    rng = np.random.Generator(np.random.PCG64(7))
    params = []
    for shp in m.parameter_shapes():
        params.append((rng.standard_normal(shp, dtype=np.float32) * np.float32(0.02)) if shp[0] != 1
                      else np.ones(shp, np.float32))
    m.load_parameters(params)
    ids = rng.integers(0, V, size=(a.batch, a.prompt), dtype=np.uint32)
    m.prefill(ids, want_logits=False)
    be.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.iters):
        m.prefill(ids, want_logits=False)
    be.synchronize()
    dt = (time.perf_counter() - t0) / a.iters
    rows = a.batch * a.prompt
    flops = 2.0 * rows * a.layers * 12 * D * D + 2.0 * a.batch * D * V + 4.0 * a.layers * a.batch * a.prompt * a.prompt * D / 2
    print(json.dumps({"prompt_pass_ms": dt * 1e3, "tflops": flops / dt / 1e12, "rows": rows, "layers": a.layers,
                      "gemm": os.environ.get("RG_B200_PREFILL", "tcgen05"), "launches": be.launch_count}))


if __name__ == "__main__":
    main()
