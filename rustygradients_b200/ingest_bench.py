"""Time from a weights file on disk to a model ready to generate.

    python -m rustygradients_b200.ingest_bench [--vocab 50257] [--layers 12] [--names hf_gpt2|rusty] [--dir /tmp]

Writes a GPT-2-small-shaped F32 safetensors file with seeded random weights
(Hugging Face names: fused c_attn, tied head; or the crate's descriptive names),
then times `GPTModel.load_safetensors` (file mapping, header parse, q|k|v split and
head transpose where needed, host-to-device copies, re-packing for the token-loop
kernel) and prints one JSON line.  The file is removed afterwards."""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np

from . import B200Backend, GptConfig, GPTModel
from . import serialization as S


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--names", default="hf_gpt2", choices=["hf_gpt2", "rusty"])
    ap.add_argument("--dir", default="/tmp")
    a = ap.parse_args()
    D, H, C, V, L = 768, 12, 1024, a.vocab, a.layers
    rng = np.random.Generator(np.random.PCG64(3))

    def n(*shape):
        return rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)

    t = {}
    if a.names == "hf_gpt2":
        t["wte.weight"], t["wpe.weight"] = n(V, D), n(C, D)
        for l in range(L):
            h = f"h.{l}."
            t[h + "attn.c_attn.weight"], t[h + "attn.c_attn.bias"] = n(D, 3 * D), n(3 * D)
            t[h + "attn.c_proj.weight"], t[h + "attn.c_proj.bias"] = n(D, D), n(D)
            t[h + "mlp.c_fc.weight"], t[h + "mlp.c_fc.bias"] = n(D, 4 * D), n(4 * D)
            t[h + "mlp.c_proj.weight"], t[h + "mlp.c_proj.bias"] = n(4 * D, D), n(D)
            for ln in ("ln_1", "ln_2"):
                t[h + ln + ".weight"], t[h + ln + ".bias"] = np.ones(D, np.float32), np.zeros(D, np.float32)
        t["ln_f.weight"], t["ln_f.bias"] = np.ones(D, np.float32), np.zeros(D, np.float32)
    be = B200Backend(0)
    m = GPTModel(be, GptConfig(C, V, L, H, D))
    if a.names == "rusty":
        for name, shp in zip(S.rusty_names(L), m.parameter_shapes()):
            t[name] = n(*shp)
    path = os.path.join(a.dir, f"rg_ingest_bench_{os.getpid()}.safetensors")
    S.write_safetensors(path, t)
    size = os.path.getsize(path)
    del t
    try:
        times = []
        for _ in range(3):
            be.synchronize()
            t0 = time.perf_counter()
            m.load_safetensors(path, names=a.names)
            be.synchronize()
            times.append(time.perf_counter() - t0)
        ids = m.generate(np.zeros((1, 4), np.uint32), 4)
        print(json.dumps({"file_bytes": size, "names": a.names, "load_s": times, "best_gb_per_s": size / min(times) / 1e9,
                          "generated": [int(x) for x in np.asarray(ids).ravel()]}))
    finally:
        os.remove(path)


if __name__ == "__main__":
    main()
