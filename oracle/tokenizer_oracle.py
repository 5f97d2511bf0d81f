"""CPU restatement of the reference's tokenizers.  TEST INFRASTRUCTURE ONLY: used by
tests/ and by tests/golden/make_tokenizer_golden.py as the checker of the library's
tokenizer entry points; nothing in the product imports it.

Pinned against the reference's own known-answer tests (`reference_kats()`):
src/tokenization/char_tokenizer.rs:113-161 (encode("Hello") has 5 ids and decodes back;
"aabbcc" has vocabulary 3; from_vocab(['a','b','c']) gives ids 0, 1, 2; the pangram
round-trips) and, for the BPE encoder, against the vocabulary file the reference ships
(bpe_tokenizer_1024.json: 433 tokens, 380 merges) when the reference tree is present.
`bpe_train` cannot be pinned: the reference picks the most frequent pair with
`max_by_key` over a HashMap (src/tokenization/bpe_tokenizer.rs:139-155), so ties
are broken by hash order; here the first pair in word order wins."""
from __future__ import annotations

import json
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

# char::is_whitespace (Unicode White_Space), the separator set of str::split_whitespace
_WS = set([0x09, 0x0A, 0x0B, 0x0C, 0x0D, 0x20, 0x85, 0xA0, 0x1680, 0x2028, 0x2029, 0x202F, 0x205F, 0x3000]
          + list(range(0x2000, 0x200B)))


def split_whitespace(text: str) -> List[str]:
    words, cur = [], []
    for ch in text:
        if ord(ch) in _WS:
            if cur:
                words.append("".join(cur))
                cur = []
        else:
            cur.append(ch)
    if cur:
        words.append("".join(cur))
    return words


class CharTokenizer:
    """src/tokenization/char_tokenizer.rs:34-107"""

    def __init__(self, text: Optional[str] = None, vocab: Optional[Sequence[str]] = None):
        chars = sorted(set(text)) if vocab is None else list(vocab)
        self.char_to_idx = {c: i for i, c in enumerate(chars)}   # a repeated char keeps its last id (collect into HashMap)
        self.idx_to_char = {i: c for i, c in enumerate(chars)}
        self.vocab_size = len(chars)

    def encode(self, text: str) -> List[int]:
        return [self.char_to_idx[c] for c in text if c in self.char_to_idx]

    def decode(self, ids: Sequence[int]) -> str:
        return "".join(self.idx_to_char[i] for i in ids if i in self.idx_to_char)


class BPETokenizer:
    """src/tokenization/bpe_tokenizer.rs:186-275 (a loaded tokenizer: no [UNK] id, :241-246)"""

    def __init__(self, token_to_id: Dict[str, int], id_to_token: Dict[int, str], merges: List[Tuple[str, str]],
                 vocab_size: int):
        self.token_to_id, self.id_to_token, self.merges, self.vocab_size = token_to_id, id_to_token, merges, vocab_size

    @classmethod
    def load(cls, path: str) -> "BPETokenizer":
        d = json.load(open(path, encoding="utf-8"))
        return cls({k: int(v) for k, v in d["token_to_id"].items()}, {int(k): v for k, v in d["id_to_token"].items()},
                   [(a, b) for a, b in d["merges"]], int(d["vocab_size"]))

    def save(self, path: str) -> None:  # :207-221
        json.dump({"token_to_id": self.token_to_id, "id_to_token": {str(k): v for k, v in self.id_to_token.items()},
                   "merges": [list(m) for m in self.merges], "vocab_size": self.vocab_size},
                  open(path, "w", encoding="utf-8"), ensure_ascii=False, indent=2)

    def tokenize_word(self, word: str) -> List[str]:  # :186-205
        tokens = list(word)
        for left, right in self.merges:
            i = 0
            while i + 1 < len(tokens):
                if tokens[i] == left and tokens[i + 1] == right:
                    tokens[i] = left + right
                    del tokens[i + 1]
                else:
                    i += 1
        return tokens

    def encode(self, text: str) -> List[int]:  # :250-267
        ids = []
        for word in split_whitespace(text):
            for tok in self.tokenize_word(word):
                if tok in self.token_to_id:
                    ids.append(self.token_to_id[tok])
        return ids

    def decode(self, ids: Sequence[int]) -> str:  # :269-275
        return " ".join(self.id_to_token[i] for i in ids if i in self.id_to_token)


def bpe_train(text: str, vocab_size: int, special_tokens: Sequence[str] = ()) -> BPETokenizer:
    """src/tokenization/bpe_tokenizer.rs:48-123 with a deterministic tie-break (see the module docstring)."""
    token_to_id: Dict[str, int] = {}
    id_to_token: Dict[int, str] = {}
    cur = 0
    for i, t in enumerate(special_tokens):
        token_to_id[t], id_to_token[i] = i, t
        cur = i + 1
    for c in sorted(set(text)):
        if c not in token_to_id:
            token_to_id[c], id_to_token[cur] = cur, c
            cur += 1
    base = cur
    word_freqs: "OrderedDict[Tuple[str, ...], int]" = OrderedDict()
    for w in split_whitespace(text):
        k = tuple(w)
        word_freqs[k] = word_freqs.get(k, 0) + 1
    merges: List[Tuple[str, str]] = []
    for _ in range(base, vocab_size):
        pair_freqs: "OrderedDict[Tuple[str, str], int]" = OrderedDict()
        for w, f in word_freqs.items():
            for i in range(len(w) - 1):
                pair_freqs[(w[i], w[i + 1])] = pair_freqs.get((w[i], w[i + 1]), 0) + f
        if not pair_freqs:
            break
        best = max(pair_freqs.items(), key=lambda kv: kv[1])[0]   # first of the most frequent pairs
        new = best[0] + best[1]
        token_to_id[new], id_to_token[cur] = cur, new
        cur += 1
        merges.append(best)
        nxt: "OrderedDict[Tuple[str, ...], int]" = OrderedDict()
        for w, f in word_freqs.items():
            out, i = [], 0
            while i < len(w):
                if i < len(w) - 1 and w[i] == best[0] and w[i + 1] == best[1]:
                    out.append(new)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            nxt[tuple(out)] = nxt.get(tuple(out), 0) + f
        word_freqs = nxt
    return BPETokenizer(token_to_id, id_to_token, merges, cur)


def reference_kats() -> dict:
    """The values the reference's tokenizer tests pin (src/tokenization/char_tokenizer.rs:113-161)."""
    return {
        "char_hello": {"text": "Hello, world!", "encode": "Hello", "n_ids": 5, "decode": "Hello"},
        "char_vocab": {"text": "aabbcc", "vocab_size": 3},
        "char_from_vocab": {"vocab": ["a", "b", "c"], "ids": {"a": 0, "b": 1, "c": 2}},
        "char_roundtrip": {"text": "The quick brown fox jumps over the lazy dog."},
        "bpe_shipped_file": {"vocab_size": 433, "merges": 380},
    }
