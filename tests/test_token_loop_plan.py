"""Host logic of the persistent token-loop kernel without a GPU: the op program of every tensor-parallel rank of the
shapes the benchmark runs (rg_token_loop_plan builds it exactly as a launch would) covers every projection column and
every attention (sequence, head, slice) exactly once and fits the SM's shared memory."""
import ctypes as C

import pytest

import rustygradients_b200 as rg
from rustygradients_b200 import _lib

SMS = 148


def plan(D, H, L, V, T, r, bf16, B, sms=SMS):
    out = (C.c_longlong * 8)()
    _lib.check(_lib.load().rg_token_loop_plan(D, H, L, V, T, r, int(bf16), B, sms, out))
    return dict(zip(("slices", "max_ops", "ring_slots", "smem", "head_ctas", "packed_bytes", "ops", "violations"), out))


def _vocab_slice(V, T, r):
    vpad = -(-(-(-V // T)) // 8) * 8
    v0 = min(V, r * vpad)
    return max(0, min(vpad, V - v0))


@pytest.mark.parametrize("T", [1, 2, 4, 8])
@pytest.mark.parametrize("B", [1, 2, 4])
def test_gpt2_xl_shape_every_rank(T, B):
    D, H, L, V = 1600, 25, 48, 50257
    packed = 0
    fits = set()
    for r in range(T):
        p = plan(D, H, L, V, T, r, True, B)
        assert p["violations"] == 0, (r, p)
        # 0 ring slots = the program does not fit shared memory and the step runs as separate launches (one GPU, 4 sequences)
        assert p["ring_slots"] == 0 or (2 <= p["ring_slots"] <= 6 and p["smem"] <= 227 * 1024)
        fits.add(p["ring_slots"] >= 2)
        assert 1 <= p["slices"] <= 4
        # what the consumers of the picks assume about every rank: one pick slot per CTA with LM-head columns
        assert p["head_ctas"] == min(SMS, -(-_vocab_slice(V, T, r) // 8))
        packed += p["packed_bytes"]
    assert len(fits) == 1          # all ranks of a group take the same form of the step (they wait for each other)
    assert fits == {True} or (T, B) == (1, 4)
    # all ranks together stream the model's projection weights once (bf16; + trailers and padding): 12 D^2 per block + D V
    assert 1.0 <= packed / (2 * (L * 12 * D * D + D * V)) < 1.03


@pytest.mark.parametrize("shape", [(768, 12, 12, 1024, False), (768, 12, 12, 50257, True), (1024, 16, 24, 50257, True),
                                   (128, 4, 3, 128, False), (96, 3, 2, 301, False), (320, 5, 3, 1000, True)])
def test_single_gpu_and_two_rank_shapes(shape):
    D, H, L, V, bf16 = shape
    for T in (1, 2):
        for r in range(T):
            for B in (1, 2, 4):
                p = plan(D, H, L, V, T, r, bf16, B)
                assert p["violations"] == 0 and p["ring_slots"] >= 2, (T, r, B, p)


def test_plan_rejects_shapes_outside_the_kernel():
    out = (C.c_longlong * 8)()
    lib = _lib.load()
    with pytest.raises(rg.InvalidInput):
        _lib.check(lib.rg_token_loop_plan(768, 12, 12, 1024, 1, 0, 0, 3, SMS, out))      # 3 sequences: no instance
    with pytest.raises(rg.InvalidInput):
        _lib.check(lib.rg_token_loop_plan(768, 12, 12, 1024, 2, 2, 0, 1, SMS, out))      # rank outside the group
    with pytest.raises(rg.Unsupported):
        _lib.check(lib.rg_token_loop_plan(2048, 8, 2, 1024, 1, 0, 1, 1, SMS, out))       # head size 256
