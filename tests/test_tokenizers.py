"""Tokenizer front-end: the library's entry points (C ABI, host code) against the
oracle restatement, the committed golden cases and the reference's own known answers
(src/tokenization/char_tokenizer.rs:113-161).  No GPU needed."""
import json
import os

import numpy as np
import pytest

import rustygradients_b200 as rg
from oracle import tokenizer_oracle as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# the vocabulary file the reference ships, where its tree sits next to this repository (or RG_REFERENCE_DIR points at it)
REF_BPE = os.path.join(os.environ.get("RG_REFERENCE_DIR", os.path.join(os.path.dirname(GOLDEN), "..", "..", "reference")),
                       "bpe_tokenizer_1024.json")


def test_reference_kats_char():
    k = T.reference_kats()
    for make in (lambda text: T.CharTokenizer(text), lambda text: rg.CharTokenizer(text)):
        t = make(k["char_hello"]["text"])
        ids = t.encode(k["char_hello"]["encode"])
        assert len(ids) == k["char_hello"]["n_ids"]
        assert t.decode(ids) == k["char_hello"]["decode"]
        t = make(k["char_vocab"]["text"])
        assert (t.vocab_size if isinstance(t, T.CharTokenizer) else t.vocab_size()) == k["char_vocab"]["vocab_size"]
        t = make(k["char_roundtrip"]["text"])
        assert t.decode(t.encode(k["char_roundtrip"]["text"])) == k["char_roundtrip"]["text"]
    lib = rg.CharTokenizer.from_vocab(k["char_from_vocab"]["vocab"])
    ora = T.CharTokenizer(vocab=k["char_from_vocab"]["vocab"])
    for c, i in k["char_from_vocab"]["ids"].items():
        assert lib.encode(c) == [i] and ora.encode(c) == [i]
    assert lib.vocab_size() == 3


def test_golden_cases_library_and_oracle():
    d = json.load(open(os.path.join(GOLDEN, "tokenizer_cases.json"), encoding="utf-8"))
    bpe_lib = rg.BPETokenizer(os.path.join(GOLDEN, "bpe_small.json"))
    bpe_ora = T.BPETokenizer.load(os.path.join(GOLDEN, "bpe_small.json"))
    ch_lib, ch_ora = rg.CharTokenizer(d["char_text"]), T.CharTokenizer(d["char_text"])
    assert bpe_lib.vocab_size() == bpe_ora.vocab_size
    assert ch_lib.vocab_size() == ch_ora.vocab_size
    n_ids = 0
    for c in d["cases"]:
        lib, ora = (bpe_lib, bpe_ora) if c["kind"] == "bpe" else (ch_lib, ch_ora)
        assert ora.encode(c["text"]) == c["ids"]
        assert lib.encode(c["text"]) == c["ids"]
        assert ora.decode(c["ids"]) == c["decoded"]
        assert lib.decode(c["ids"]) == c["decoded"]
        n_ids += len(c["ids"])
    assert n_ids > 200


def test_unknown_ids_and_chars_are_dropped():
    t = rg.CharTokenizer("abc")
    assert t.encode("a?b!c") == [0, 1, 2]
    assert t.decode([0, 99, 2]) == "ac"
    b = rg.BPETokenizer(os.path.join(GOLDEN, "bpe_small.json"))
    assert b.decode([10 ** 6]) == ""
    assert b.encode(" \t\n   ") == []  # Unicode white space only


def test_random_texts_against_oracle():
    rng = np.random.Generator(np.random.PCG64(7))
    ora = T.BPETokenizer.load(os.path.join(GOLDEN, "bpe_small.json"))
    lib = rg.BPETokenizer(os.path.join(GOLDEN, "bpe_small.json"))
    alphabet = [t for t in ora.token_to_id if len(t) == 1 and t != "["] + [" ", "\n", "　", "x", "é"]
    for _ in range(50):
        text = "".join(alphabet[int(i)] for i in rng.integers(0, len(alphabet), size=int(rng.integers(0, 300))))
        ids = ora.encode(text)
        assert lib.encode(text) == ids
        assert lib.decode(ids) == ora.decode(ids)


@pytest.mark.skipif(not os.path.exists(REF_BPE), reason="reference tree not mounted")
def test_shipped_vocabulary_file():
    k = T.reference_kats()["bpe_shipped_file"]
    ora, lib = T.BPETokenizer.load(REF_BPE), rg.BPETokenizer(REF_BPE)
    assert ora.vocab_size == lib.vocab_size() == k["vocab_size"]
    assert len(ora.merges) == k["merges"]
    rng = np.random.Generator(np.random.PCG64(11))
    toks = sorted(ora.token_to_id)
    for _ in range(30):
        words = ["".join(toks[int(i)] for i in rng.integers(0, len(toks), size=int(rng.integers(1, 5)))).strip() or "a"
                 for _ in range(int(rng.integers(1, 40)))]
        text = " ".join(words)
        ids = ora.encode(text)
        assert lib.encode(text) == ids
        assert lib.decode(ids) == ora.decode(ids)


def test_errors(tmp_path):
    with pytest.raises(rg.IoError):
        rg.BPETokenizer(str(tmp_path / "missing.json"))
    bad = tmp_path / "bad.json"
    bad.write_text('{"token_to_id": {"a": 0}, "merges": [["a"]], "vocab_size": 1')
    with pytest.raises(rg.SerializationError):
        rg.BPETokenizer(str(bad))
    bad.write_text('{"token_to_id": {"a": 0}, "id_to_token": {"0": "a"}, "merges": [["a"]], "vocab_size": 1}')
    with pytest.raises(rg.SerializationError):
        rg.BPETokenizer(str(bad))
    # text that is not UTF-8, and an output buffer that is too small, through the C ABI directly
    import ctypes as C
    from rustygradients_b200 import _lib
    lib = _lib.load()
    t = rg.CharTokenizer("ab")
    n = C.c_size_t()
    assert lib.rg_tokenizer_encode(t._h, b"\xff\xfe", 2, None, 0, C.byref(n)) == _lib.RG_ERR_INVALID_INPUT
    ids = (C.c_uint32 * 1)()
    assert lib.rg_tokenizer_encode(t._h, b"abab", 4, ids, 1, C.byref(n)) == _lib.RG_ERR_INVALID_INPUT
    assert n.value == 4
