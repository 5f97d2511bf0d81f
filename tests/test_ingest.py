"""Weight ingest from disk (safetensors F32 + metadata sidecar, the legacy weights JSON,
the crate's descriptive names and the Hugging Face GPT-2 names): every route must put
exactly the same model on the device as `load_parameters` does from memory."""
import json
import os
import struct

import numpy as np
import pytest

import rustygradients_b200 as rg
from oracle import gpt_oracle as O
from rustygradients_b200 import serialization as S
from tests.helpers import F32_TOL, model_for

CFG = O.GptConfig(block_size=24, vocab_size=61, num_layers=2, num_heads=4, embedding_dim=128)


def _params():
    return O.make_params(CFG, seed=31, stress=True)


def _hf_tensors(params, prefix="", block_rows=None):
    """The same model under Hugging Face GPT-2 names: fused c_attn, 1-D vectors, tied head (so the
    parameter list is changed to match: head = wte^T, head bias 0)."""
    p = [np.array(x) for x in params]
    D = CFG.embedding_dim
    p[-2] = np.ascontiguousarray(p[0].T)
    p[-1] = np.zeros_like(p[-1])
    t = {prefix + "wte.weight": p[0], prefix + "wpe.weight": p[1] if block_rows is None else
         np.concatenate([p[1], np.ones((block_rows - p[1].shape[0], D), np.float32)])}
    for l in range(CFG.num_layers):
        b = p[2 + 16 * l: 2 + 16 * (l + 1)]
        h = f"{prefix}h.{l}."
        t[h + "attn.c_attn.weight"] = np.concatenate([b[0], b[2], b[4]], axis=1)
        t[h + "attn.c_attn.bias"] = np.concatenate([b[1], b[3], b[5]], axis=1).reshape(-1)
        t[h + "attn.c_proj.weight"], t[h + "attn.c_proj.bias"] = b[6], b[7].reshape(-1)
        t[h + "ln_1.weight"], t[h + "ln_1.bias"] = b[8].reshape(-1), b[9].reshape(-1)
        t[h + "mlp.c_fc.weight"], t[h + "mlp.c_fc.bias"] = b[10], b[11].reshape(-1)
        t[h + "mlp.c_proj.weight"], t[h + "mlp.c_proj.bias"] = b[12], b[13].reshape(-1)
        t[h + "ln_2.weight"], t[h + "ln_2.bias"] = b[14].reshape(-1), b[15].reshape(-1)
    t[prefix + "ln_f.weight"], t[prefix + "ln_f.bias"] = p[-4].reshape(-1), p[-3].reshape(-1)
    return t, p


# ------------------------------------------------------------------ CPU: metadata and file-level errors
def test_metadata_sidecar_and_checkpoint(tmp_path):
    cfg = rg.GptConfig(128, 100, 2, 4, 64)  # the values of the reference's round-trip test (safetensors_format.rs:205-213)
    side = str(tmp_path / "test_model.safetensors.json")
    S.write_metadata(side, cfg, model_type="TestModel", dropout=0.1)
    got = S.read_metadata(side, causal=False, activation="relu")
    assert (got.block_size, got.vocab_size, got.num_layers, got.num_heads, got.embedding_dim) == (128, 100, 2, 4, 64)
    assert got.causal is False and got.activation == "relu"
    ck = tmp_path / "ck.json"
    ck.write_text(json.dumps({"metadata": json.load(open(side)), "weights": [], "step": 3, "loss": 0.5}))
    got = S.read_metadata(str(ck))
    assert got.embedding_dim == 64 and got.block_size == 128


def test_metadata_errors(tmp_path):
    with pytest.raises(rg.IoError):
        S.read_metadata(str(tmp_path / "nope.json"))
    bad = tmp_path / "bad.json"
    bad.write_text('{"vocab_size": 10, "embedding_dim": 8')
    with pytest.raises(rg.SerializationError):
        S.read_metadata(str(bad))
    bad.write_text('{"vocab_size": 10, "embedding_dim": 8, "num_layers": 1, "num_heads": 2}')
    with pytest.raises(rg.SerializationError, match="block_size"):
        S.read_metadata(str(bad))


# ------------------------------------------------------------------ GPU: every route == load_parameters
def _logits(model, ids):
    return model.forward(ids.astype(np.float32))


@pytest.mark.gpu
def test_safetensors_rusty_names_equal_in_memory_load(backend, tmp_path):
    params = _params()
    ids = O.make_prompt(CFG, 5, 2, 17)
    want = _logits(model_for(backend, CFG, params, max_batch=2), ids)
    assert np.abs(want - O.forward(params, CFG, ids, causal=True, act="gelu_tanh")).max() < F32_TOL
    path = str(tmp_path / "model.safetensors")
    S.write_safetensors(path, dict(zip(S.rusty_names(CFG.num_layers), params)))
    S.write_metadata(path + ".json", rg.GptConfig(CFG.block_size, CFG.vocab_size, CFG.num_layers, CFG.num_heads,
                                                  CFG.embedding_dim))
    m = rg.GPTModel(backend, S.read_metadata(path + ".json", max_batch=2))
    m.load_safetensors(path)
    np.testing.assert_array_equal(_logits(m, ids), want)
    # and through the token loop
    a = m.generate(ids[:1, :8], 10)
    b = model_for(backend, CFG, params, max_batch=2).generate(ids[:1, :8], 10)
    np.testing.assert_array_equal(a, b)


@pytest.mark.gpu
def test_safetensors_fused_qkv_and_defaults(backend, tmp_path):
    """train_gpt_e2e.rs naming: layer_i.attn.qkv.weight [D,3D] + attn.proj.weight; absent biases are zero,
    absent final LayerNorm is gamma 1 / beta 0."""
    params = [np.array(x) for x in _params()]
    names = S.rusty_names(CFG.num_layers)
    t = {}
    for l in range(CFG.num_layers):
        b = 2 + 16 * l
        for j in (1, 3, 5, 7, 11, 13):
            params[b + j][:] = 0
        t[f"layer_{l}.attn.qkv.weight"] = np.concatenate([params[b], params[b + 2], params[b + 4]], axis=1)
        t[f"layer_{l}.attn.proj.weight"] = params[b + 6]
        for j in (8, 9, 10, 12, 14, 15):
            t[names[b + j]] = params[b + j]
    params[-4][:] = 1
    params[-3][:] = 0
    params[-1][:] = 0
    t["token_embedding.weight"], t["position_embedding.weight"] = params[0], params[1]
    t["output_projection.weight"] = params[-2]
    path = str(tmp_path / "fused.safetensors")
    S.write_safetensors(path, t)
    ids = O.make_prompt(CFG, 6, 1, 12)
    m = rg.GPTModel(backend, rg.GptConfig(CFG.block_size, CFG.vocab_size, CFG.num_layers, CFG.num_heads,
                                          CFG.embedding_dim, max_batch=2))
    m.load_safetensors(path, names="rusty")
    np.testing.assert_array_equal(_logits(m, ids), _logits(model_for(backend, CFG, params, max_batch=2), ids))


@pytest.mark.gpu
@pytest.mark.parametrize("prefix,rows", [("", None), ("transformer.", 40)])
def test_safetensors_hf_gpt2_names(backend, tmp_path, prefix, rows):
    t, params = _hf_tensors(_params(), prefix, rows)
    path = str(tmp_path / "hf.safetensors")
    S.write_safetensors(path, t)
    ids = O.make_prompt(CFG, 8, 2, 9)
    m = rg.GPTModel(backend, rg.GptConfig(CFG.block_size, CFG.vocab_size, CFG.num_layers, CFG.num_heads,
                                          CFG.embedding_dim, max_batch=2))
    m.load_safetensors(path)  # auto-detects the naming
    got = _logits(m, ids)
    np.testing.assert_array_equal(got, _logits(model_for(backend, CFG, params, max_batch=2), ids))
    assert np.abs(got - O.forward(params, CFG, ids, causal=True, act="gelu_tanh")).max() < F32_TOL


@pytest.mark.gpu
def test_weights_json_and_checkpoint_json(backend, tmp_path):
    params = _params()
    ids = O.make_prompt(CFG, 9, 1, 11)
    want = _logits(model_for(backend, CFG, params, causal=False, act="relu", max_batch=2), ids)
    path = str(tmp_path / "weights.json")
    S.write_weights_json(path, params)
    cfg = rg.GptConfig(CFG.block_size, CFG.vocab_size, CFG.num_layers, CFG.num_heads, CFG.embedding_dim, causal=False,
                       activation="relu")
    m = rg.GPTModel(backend, cfg)
    m.load_json(path)
    np.testing.assert_array_equal(_logits(m, ids), want)
    ck = str(tmp_path / "checkpoint.json")
    json.dump({"metadata": {"model_type": "GPT", "vocab_size": CFG.vocab_size, "embedding_dim": CFG.embedding_dim,
                            "num_layers": CFG.num_layers, "num_heads": CFG.num_heads, "block_size": CFG.block_size,
                            "dropout": 0.0}, "weights": json.load(open(path)), "step": 7, "loss": 1.25}, open(ck, "w"),
              indent=1)
    m2 = rg.GPTModel(backend, S.read_metadata(ck, causal=False, activation="relu"))
    m2.load_json(ck)
    np.testing.assert_array_equal(_logits(m2, ids), want)


@pytest.mark.gpu
def test_ingest_errors(backend, tmp_path):
    params = _params()
    names = S.rusty_names(CFG.num_layers)
    cfg = rg.GptConfig(CFG.block_size, CFG.vocab_size, CFG.num_layers, CFG.num_heads, CFG.embedding_dim)
    m = rg.GPTModel(backend, cfg)
    path = str(tmp_path / "m.safetensors")
    with pytest.raises(rg.IoError):
        m.load_safetensors(path)
    t = dict(zip(names, params))
    del t["layer_1.ffn.fc2.weight"]
    S.write_safetensors(path, t)
    with pytest.raises(rg.IoError, match="Missing required weight: layer_1.ffn.fc2.weight"):
        m.load_safetensors(path)
    t = dict(zip(names, params))
    t["layer_0.attn.k.weight"] = t["layer_0.attn.k.weight"][:, :-1]
    S.write_safetensors(path, t)
    with pytest.raises(rg.ShapeError, match="Mismatch in tensor shape"):
        m.load_safetensors(path)
    # a dtype other than F32 (the reference reader's "Expected F32 dtype", safetensors_format.rs:111-116)
    hdr = json.dumps({"token_embedding.weight": {"dtype": "BF16", "shape": [2, 2], "data_offsets": [0, 8]}}).encode()
    hdr += b" " * (-len(hdr) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(rg.SerializationError, match="Expected F32 dtype"):
        m.load_safetensors(path)
    # truncated file / offsets beyond the data
    hdr = json.dumps({"token_embedding.weight": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 64]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(rg.SerializationError):
        m.load_safetensors(path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(rg.SerializationError):
        m.load_safetensors(path)
    # a shape whose element count wraps around 64 bits (4 * 2^62 bytes = 0), with and without an aligned header
    for pad in (0, 1):
        hdr = json.dumps({"token_embedding.weight": {"dtype": "F32", "shape": [1 << 62], "data_offsets": [0, 0]}}).encode()
        hdr += b" " * ((-len(hdr) % 8) + pad)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
        with pytest.raises(rg.SerializationError):
            m.load_safetensors(path)
    # JSON: wrong tensor count, wrong shape, data length that does not match the shape
    jpath = str(tmp_path / "w.json")
    S.write_weights_json(jpath, params[:-1])
    with pytest.raises(rg.ShapeError, match="Mismatch in number of parameter tensors"):
        m.load_json(jpath)
    w = [{"shape": list(p.shape), "data": [0.0] * p.size} for p in params]
    w[3]["data"] = w[3]["data"][:-1]
    json.dump(w, open(jpath, "w"))
    with pytest.raises(rg.ShapeError):
        m.load_json(jpath)
    # an unaligned header still loads (data copied out of the mapping)
    tens = dict(zip(names, params))
    S.write_safetensors(path, tens)
    raw = open(path, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", n + 1) + raw[8:8 + n] + b" " + raw[8 + n:])
    m.load_safetensors(path)
    ids = O.make_prompt(CFG, 10, 1, 6)
    np.testing.assert_array_equal(_logits(m, ids), _logits(model_for(backend, CFG, params, max_batch=2), ids))
