"""GPU tests of the persistent forms of the token loop beyond the benchmark workload: the cluster kernel against the
oracle, full-depth GPT-2-medium / GPT-2-XL shapes, and the bounded device waits running out (without any device
fault: a withheld signal, a lowered iteration limit)."""
import numpy as np
import pytest

import rustygradients_b200 as rg
from oracle import gpt_oracle as O
from helpers import F32_TOL, assert_bf16_close, confident_rows, model_for, teacher_forced

pytestmark = pytest.mark.gpu

FORM_DEFAULT, FORM_CLUSTER, FORM_PERSISTENT, FORM_LAUNCHES = 0, 1, 2, 3


def _cluster(model):
    model.debug_hook(4, FORM_CLUSTER)
    return model


# ---- the cluster kernel (thread-block clusters, two grid-wide exchanges per block) against the oracle
def test_cluster_kernel_char_gpt(backend):
    c = O.CONFIGS[0]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    params = O.make_params(cfg, O.config_seed(0), stress=True)
    prompt = O.make_prompt(cfg, O.config_seed(0), 1, P)
    toks, want = O.generate_causal(params, cfg, prompt, G)
    m = _cluster(model_for(backend, cfg, params))
    logits, picks = teacher_forced(m, np.concatenate([prompt, toks], 1), P)
    assert np.abs(logits - want).max() <= F32_TOL
    assert np.array_equal(picks, logits.argmax(-1))


def test_cluster_kernel_gpt2_small_every_step(backend):
    c = O.CONFIGS[1]
    cfg, P, G = c["cfg"], c["prompt"], 96
    params = O.make_params(cfg, O.config_seed(1))
    prompt = O.make_prompt(cfg, O.config_seed(1), 1, P)
    a = model_for(backend, cfg, params)                       # default form
    ids = np.concatenate([prompt, a.generate(prompt, G)], 1)
    want = O.teacher_forced_logits(params, cfg, ids, True, "gelu_tanh", P)
    m = _cluster(model_for(backend, cfg, params))
    logits, picks = teacher_forced(m, ids, P)
    assert np.abs(logits - want).max() <= F32_TOL
    assert np.array_equal(picks, logits.argmax(-1))
    # one launch runs many steps and reproduces the ids wherever the top-2 gap is clear; twice the same, bit for bit
    l0 = backend.launch_count
    m.prefill(prompt)
    m.decode_run(G - 1)
    run = m.read_tokens(P, G, 1)
    assert backend.launch_count - l0 < 200                    # prompt pass + ONE launch for the steps
    ok = confident_rows(want, 4 * F32_TOL)[0]
    first_bad = np.argmin(ok) if not ok.all() else G
    assert np.array_equal(run[0, :first_bad], ids[0, P:P + first_bad])
    m.rewind(P)
    m.decode_run(G - 1)
    assert np.array_equal(m.read_tokens(P, G, 1), run)


@pytest.mark.parametrize("shape", [(768, 12), (1024, 16), (1600, 25)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_cluster_kernel_widths(backend, shape, dtype):
    """Small, medium and XL widths (cluster sizes 8, 6 and 5: one cluster per head must fit), 2 layers, batch 1."""
    D, H = shape
    cfg = O.GptConfig(48, 3001, 2, H, D)
    params = O.make_params(cfg, 37, stress=True, bf16=(dtype == "bf16"))
    prompt = O.make_prompt(cfg, 37, 1, 13)
    toks, want = O.generate_causal(params, cfg, prompt, 10)
    m = _cluster(model_for(backend, cfg, params, dtype=dtype))
    logits, picks = teacher_forced(m, np.concatenate([prompt, toks], 1), 13)
    if dtype == "f32":
        assert np.abs(logits - want).max() <= F32_TOL
    else:
        assert_bf16_close(logits, want, f"cluster kernel D={D}")
    assert np.array_equal(picks, logits.argmax(-1))


# ---- full depth: GPT-2-medium (24 blocks) and GPT-2-XL (48 blocks) shapes, bf16 weights, 2 sequences
@pytest.mark.parametrize("name,shape", [("medium", (1024, 16, 24)), ("xl", (1600, 25, 48))])
def test_full_depth_models_first_steps(backend, name, shape):
    """Prompt pass + 4 cached steps against oracle logits computed ahead of time (tests/golden/make_golden_full_depth.py:
    the oracle needs minutes for these shapes).  The weights are drawn again from the seed; the engine rounds them to
    bf16 (round to nearest even) at load, exactly what the oracle's copy was rounded with."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "full_depth.npz"))
    D, H, L = shape
    cfg = O.GptConfig(32, 50257, L, H, D)
    params = O.make_params(cfg, int(g["seed"]))                # f32 draws, no host-side rounding
    prompt, toks = g[f"{name}_prompt"], g[f"{name}_tokens"]
    m = model_for(backend, cfg, params, dtype="bf16", max_batch=2)
    del params
    logits, picks = teacher_forced(m, np.concatenate([prompt, toks], 1), prompt.shape[1])
    want = g[f"{name}_logits_sampled"]
    got = logits[:, :, ::int(g["stride"])]
    scale = g[f"{name}_row_absmax"][..., None]
    err = np.abs(got - want) / scale
    print(f"bf16 parity full depth {name}: worst sampled |diff| / row max {err.max():.2e}")
    assert err.max() <= 8e-3
    assert np.array_equal(picks, logits.argmax(-1))
    sure = g[f"{name}_row_top2_gap"] > 4 * 8e-3 * g[f"{name}_row_absmax"]
    assert np.array_equal(picks[sure], toks[sure])


# ---- bounded waits that run out: the call reports DeviceTimeout, the context stays usable
def _small_model(backend):
    cfg = O.GptConfig(64, 128, 3, 4, 128)
    params = O.make_params(cfg, 3)
    prompt = O.make_prompt(cfg, 3, 1, 8)
    return model_for(backend, cfg, params), prompt


def test_persistent_kernel_wait_runs_out(backend):
    m, prompt = _small_model(backend)
    good = m.generate(prompt, 12)
    m.debug_hook(5, 20000)          # iteration limit of every wait
    m.debug_hook(6, 1)              # CTA 0 withholds its q|k|v outputs of block 1
    with pytest.raises(rg.DeviceTimeout):
        m.generate(prompt, 12)
    m.debug_hook(6, -1)
    m.debug_hook(5, 0)
    assert np.array_equal(m.generate(prompt, 12), good)       # same model, same context: works again


def test_cluster_kernel_wait_runs_out(backend):
    m, prompt = _small_model(backend)
    good = m.generate(prompt, 12)
    _cluster(m)
    assert np.array_equal(m.generate(prompt, 12), good)       # (builds the cluster kernel's program)
    m.debug_hook(3, 20000)          # iteration limit of every wait
    m.debug_hook(2, 1)              # head cluster 0 withholds its partial vector of block 1
    with pytest.raises(rg.DeviceTimeout):
        m.generate(prompt, 12)
    m.debug_hook(2, -1)
    assert np.array_equal(m.generate(prompt, 12), good)


def test_allreduce_wait_runs_out_and_tensor_core_flag(backend):
    m, prompt = _small_model(backend)
    good = m.generate(prompt, 6)
    with pytest.raises(rg.DeviceTimeout):                      # rank 0 of 2, nobody plays rank 1
        m.debug_hook(7, 20000)
    assert np.array_equal(m.generate(prompt, 6), good)
    m.debug_hook(1)                                            # what a tensor-core kernel's wait raises when it gives up
    with pytest.raises(rg.DeviceTimeout):
        m.prefill(prompt)
    lg, _ = m.prefill(prompt)                                  # reported once, then cleared
    assert np.isfinite(lg).all()
    m.debug_hook(1)
    with pytest.raises(rg.DeviceTimeout):
        backend.synchronize()
    backend.synchronize()
