"""Host-side mirror of the `Tokenizer` trait (src/tokenization/mod.rs) with its two
implementations on the token loop's path, over the C ABI:
`CharTokenizer` (src/tokenization/char_tokenizer.rs) and `BPETokenizer` as loaded
from its JSON file (src/tokenization/bpe_tokenizer.rs:224-275)."""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import numpy as np

from . import _lib
from ._lib import check


class _Tokenizer:
    def __init__(self, handle: C.c_void_p):
        self._lib = _lib.load()
        self._h = handle

    def close(self) -> None:
        if self._h:
            self._lib.rg_tokenizer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def vocab_size(self) -> int:
        n = C.c_size_t()
        check(self._lib.rg_tokenizer_vocab_size(self._h, C.byref(n)))
        return int(n.value)

    def encode(self, text: str) -> List[int]:
        raw = text.encode("utf-8")
        n = C.c_size_t()
        check(self._lib.rg_tokenizer_encode(self._h, raw, len(raw), None, 0, C.byref(n)))
        ids = np.zeros(max(1, n.value), np.uint32)
        check(self._lib.rg_tokenizer_encode(self._h, raw, len(raw), ids.ctypes.data_as(_lib._U32P), ids.size,
                                            C.byref(n)))
        return [int(x) for x in ids[:n.value]]

    def decode(self, ids: Sequence[int]) -> str:
        arr = np.ascontiguousarray(ids, dtype=np.uint32)
        n = C.c_size_t()
        check(self._lib.rg_tokenizer_decode(self._h, arr.ctypes.data_as(_lib._U32P), arr.size, None, 0, C.byref(n)))
        buf = C.create_string_buffer(max(1, n.value))
        check(self._lib.rg_tokenizer_decode(self._h, arr.ctypes.data_as(_lib._U32P), arr.size, buf, n.value,
                                            C.byref(n)))
        return buf.raw[:n.value].decode("utf-8")


class CharTokenizer(_Tokenizer):
    """`CharTokenizer::new(text)`; `CharTokenizer.from_vocab(chars)` for an explicit vocabulary."""

    def __init__(self, text: str):
        raw = text.encode("utf-8")
        h = C.c_void_p()
        check(_lib.load().rg_tokenizer_char_from_text(raw, len(raw), C.byref(h)))
        super().__init__(h)

    @classmethod
    def from_vocab(cls, vocab: Sequence[str]) -> "CharTokenizer":
        cps = np.array([ord(c) for c in vocab], dtype=np.uint32)
        h = C.c_void_p()
        check(_lib.load().rg_tokenizer_char_from_vocab(cps.ctypes.data_as(_lib._U32P), cps.size, C.byref(h)))
        self = cls.__new__(cls)
        _Tokenizer.__init__(self, h)
        return self


class BPETokenizer(_Tokenizer):
    """`BPETokenizer::load(path)`."""

    def __init__(self, path: str):
        h = C.c_void_p()
        check(_lib.load().rg_tokenizer_bpe_load(path.encode(), C.byref(h)))
        super().__init__(h)

    @classmethod
    def load(cls, path: str) -> "BPETokenizer":
        return cls(path)
