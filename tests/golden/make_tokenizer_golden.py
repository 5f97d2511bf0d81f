"""Writes tests/golden/bpe_small.json (a tokenizer file in the format of
BPETokenizer::save, src/tokenization/bpe_tokenizer.rs:207-221) and
tests/golden/tokenizer_cases.json (texts with the ids and the decoded strings the
oracle gives for them).  The training text is synthetic: seeded pseudo-words.

Run from the repository root:  python tests/golden/make_tokenizer_golden.py"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import tokenizer_oracle as T  # noqa: E402


def synthetic_text(seed: int = 20240, n_words: int = 600) -> str:
    rng = np.random.Generator(np.random.PCG64(seed))
    syll = ["ka", "to", "mi", "ren", "sol", "va", "qu", "esh", "dor", "lin", "pa", "um", "zé", "ñi", "ör"]
    lexicon = ["".join(syll[i] for i in rng.integers(0, len(syll), size=int(rng.integers(1, 4)))) for _ in range(60)]
    words = [lexicon[int(i)] for i in rng.zipf(1.3, size=n_words) % len(lexicon)]
    seps = [" ", " ", " ", "\n", "\t", "  ", " ", " "]
    out = []
    for w in words:
        out.append(w)
        out.append(seps[int(rng.integers(0, len(seps)))])
    return "".join(out) + "end."


def main() -> None:
    text = synthetic_text()
    tok = T.bpe_train(text, 120, ["[UNK]"])
    tok.save(os.path.join(HERE, "bpe_small.json"))
    loaded = T.BPETokenizer.load(os.path.join(HERE, "bpe_small.json"))
    cases = []
    probes = [text[:200], "katomi  renren sol\nzzz unknown-chars-are-dropped ñiör", "", "   ", "a", "kakaka kaka ka",
              "esh" * 7, text[-120:]]
    for p in probes:
        ids = loaded.encode(p)
        cases.append({"kind": "bpe", "text": p, "ids": ids, "decoded": loaded.decode(ids)})
    ct = T.CharTokenizer(text)
    for p in [text[:100], "zé ñi ör   xyz", ""]:
        ids = ct.encode(p)
        cases.append({"kind": "char", "text": p, "ids": ids, "decoded": ct.decode(ids)})
    json.dump({"char_text": text, "cases": cases}, open(os.path.join(HERE, "tokenizer_cases.json"), "w", encoding="utf-8"),
              ensure_ascii=False, indent=1)
    print("vocab", tok.vocab_size, "merges", len(tok.merges), "cases", len(cases))


if __name__ == "__main__":
    main()
