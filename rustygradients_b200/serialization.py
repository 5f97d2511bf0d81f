"""Host-side mirror of the reference's on-disk model formats
(src/serialization/mod.rs, src/serialization/safetensors_format.rs).

Reading goes through the C ABI (`rg_model_metadata_read`, `GPTModel.load_safetensors`,
`GPTModel.load_json`).  The writers here produce the same files `save_model` /
`getWeightsAsJson` produce, for callers that prepare checkpoints in Python."""
from __future__ import annotations

import ctypes as C
import json
import struct
from typing import Dict, Mapping, Sequence

import numpy as np

from . import _lib
from ._lib import check
from .gpt import GptConfig


def read_metadata(path: str, **engine_switches) -> GptConfig:
    """ModelMetadata (src/serialization/mod.rs:28-37) -> GptConfig; `engine_switches` set the fields the
    metadata does not carry (causal, activation, weight_dtype, max_batch, ...)."""
    c = _lib.GptConfigC()
    check(_lib.load().rg_model_metadata_read(path.encode(), C.byref(c)))
    return GptConfig(block_size=c.block_size, vocab_size=c.vocab_size, num_layers=c.num_layers,
                     num_heads=c.num_heads, embedding_dim=c.embedding_dim, **engine_switches)


def write_metadata(path: str, cfg: GptConfig, model_type: str = "GPT", dropout: float = 0.0) -> None:
    """The sidecar `save_model` writes next to the weights (safetensors_format.rs:76-81)."""
    meta = {"model_type": model_type, "vocab_size": cfg.vocab_size, "embedding_dim": cfg.embedding_dim,
            "num_layers": cfg.num_layers, "num_heads": cfg.num_heads, "block_size": cfg.block_size,
            "dropout": dropout}
    with open(path, "w") as f:
        json.dump(meta, f, indent=2)


def write_safetensors(path: str, tensors: Mapping[str, np.ndarray]) -> None:
    """F32 safetensors file: u64 little-endian header length, JSON header {name: {dtype, shape,
    data_offsets}}, raw little-endian data; header padded with spaces to 8 bytes like the safetensors crate."""
    header: Dict[str, dict] = {}
    blobs = []
    off = 0
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name], dtype="<f4")
        header[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def write_weights_json(path: str, params: Sequence[np.ndarray]) -> None:
    """`getWeightsAsJson` (src/wasm_api.rs:166-177): [{shape, data}] in parameters() order."""
    with open(path, "w") as f:
        json.dump([{"shape": list(p.shape), "data": [float(x) for x in np.asarray(p, np.float32).ravel()]}
                   for p in params], f)


def rusty_names(num_layers: int) -> list:
    """Tensor names of a GPTModel in parameters() order under the crate's descriptive naming
    (examples/serialization_demo.rs:24-101 extended with the biases and the final LayerNorm)."""
    names = ["token_embedding.weight", "position_embedding.weight"]
    for l in range(num_layers):
        p = f"layer_{l}."
        for w in ("q", "k", "v", "out_proj"):
            names += [p + f"attn.{w}.weight", p + f"attn.{w}.bias"]
        names += [p + "ln1.gamma", p + "ln1.beta", p + "ffn.fc1.weight", p + "ffn.fc1.bias",
                  p + "ffn.fc2.weight", p + "ffn.fc2.bias", p + "ln2.gamma", p + "ln2.beta"]
    return names + ["ln_f.gamma", "ln_f.beta", "output_projection.weight", "output_projection.bias"]
