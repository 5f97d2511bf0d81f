"""Host-side mirror of `GptConfig` / `GPTModel` (src/models/gpt.rs) and of the
token loop `WasmGptTrainer::generate` (src/wasm_api.rs:97-163) over the C ABI."""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import check
from .backend import B200Backend


@dataclasses.dataclass
class GptConfig:
    """src/models/gpt.rs:8-14, plus the engine switches of rg_gpt_config."""
    block_size: int
    vocab_size: int
    num_layers: int
    num_heads: int
    embedding_dim: int
    causal: bool = True
    activation: str = "gelu_tanh"   # or "relu" (the reference's FeedForward)
    weight_dtype: str = "f32"       # or "bf16"
    max_batch: int = 1
    tp_rank: int = 0
    tp_size: int = 1


class GPTModel:
    """`GPTModel::new(config)` (gpt.rs:27-54).  Parameters are not initialised:
    load them with `load_parameters` in `parameters()` order (gpt.rs:85-93)."""

    def __init__(self, backend: B200Backend, config: GptConfig):
        self.backend = backend
        self.config = config
        self._lib = _lib.load()
        c = _lib.GptConfigC(config.block_size, config.vocab_size, config.num_layers, config.num_heads,
                            config.embedding_dim, 1 if config.causal else 0,
                            {"relu": _lib.RG_ACT_RELU, "gelu_tanh": _lib.RG_ACT_GELU_TANH}[config.activation],
                            {"f32": _lib.RG_DTYPE_F32, "bf16": _lib.RG_DTYPE_BF16}[config.weight_dtype],
                            config.max_batch, config.tp_rank, config.tp_size)
        h = C.c_void_p()
        check(self._lib.rg_gpt_create(backend._ctx, C.byref(c), C.byref(h)))
        self._h = h

    # -- tensor parallelism: one NCCL communicator over the ranks that hold the model's shards
    @staticmethod
    def tp_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(_lib.load().rg_gpt_tp_unique_id(buf))
        return bytes(buf)

    def tp_init(self, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128)(*unique_id)
        check(self._lib.rg_gpt_tp_init(self._h, buf))

    def tp_fused(self) -> bool:
        """True when the token step's all-reduces run as the one-shot kernel over peer memory (not NCCL)."""
        return bool(self._lib.rg_gpt_tp_fused(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.rg_gpt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- parameters()
    def parameter_shapes(self) -> List[tuple]:
        n = self._lib.rg_gpt_num_params(self._h)
        out = []
        s = (C.c_size_t * 2)()
        for i in range(n):
            check(self._lib.rg_gpt_param_shape(self._h, i, s))
            out.append((int(s[0]), int(s[1])))
        return out

    def load_parameters(self, params: Sequence[np.ndarray]) -> None:
        """Shape asserts of loadWeightsFromJson (src/wasm_api.rs:182-199)."""
        arrs = [np.ascontiguousarray(p, dtype=np.float32) for p in params]
        n = len(arrs)
        data = (_lib._FP * n)(*[a.ctypes.data_as(_lib._FP) for a in arrs])
        shape_bufs = [(C.c_size_t * max(1, a.ndim))(*a.shape) for a in arrs]
        shapes = (_lib._SZP * n)(*[C.cast(s, _lib._SZP) for s in shape_bufs])
        ndims = (C.c_int * n)(*[a.ndim for a in arrs])
        check(self._lib.rg_gpt_load_params(self._h, data, shapes, ndims, n))

    def load_safetensors(self, path: str, names: str = "auto") -> None:
        """`load_model` (src/serialization/safetensors_format.rs:89-138) followed by the copy into the model;
        names: "auto", "rusty" (the crate's descriptive names) or "hf_gpt2" (src/models/hf_loader.rs:256-276)."""
        code = {"auto": _lib.RG_NAMES_AUTO, "rusty": _lib.RG_NAMES_RUSTY, "hf_gpt2": _lib.RG_NAMES_HF_GPT2}[names]
        check(self._lib.rg_gpt_load_safetensors(self._h, path.encode(), code))

    def load_json(self, path: str) -> None:
        """`loadWeightsFromJson` (src/wasm_api.rs:179-199) / `load_json` (src/serialization/mod.rs:104-113)."""
        check(self._lib.rg_gpt_load_json(self._h, path.encode()))

    # -- Module::forward (gpt.rs:58-83)
    def forward(self, idx: np.ndarray) -> np.ndarray:
        idx = np.ascontiguousarray(idx, dtype=np.float32)
        if idx.ndim != 2:
            raise _lib.DimensionError(f"Operation requires a tensor with 2 dimensions, but got {idx.ndim}")
        B, T = idx.shape
        out = np.empty((B, T, self.config.vocab_size), dtype=np.float32)
        check(self._lib.rg_gpt_forward(self._h, idx.ctypes.data_as(_lib._FP), B, T, out.ctypes.data_as(_lib._FP)))
        return out

    # -- KV-cache halves of the loop
    def prefill(self, ids: np.ndarray, want_logits: bool = True):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        B, T = ids.shape
        logits = np.empty((B, self.config.vocab_size), dtype=np.float32) if want_logits else None
        pick = np.empty(B, dtype=np.uint32)
        self._batch = B                      # sequences of the cached context: decode_step / rewind take one id each
        check(self._lib.rg_gpt_prefill(self._h, ids.ctypes.data_as(_lib._U32P), B, T,
                                       logits.ctypes.data_as(_lib._FP) if want_logits else None,
                                       pick.ctypes.data_as(_lib._U32P)))
        return logits, pick

    def decode_step(self, tok: np.ndarray, want_logits: bool = True):
        tok = np.ascontiguousarray(tok, dtype=np.uint32).reshape(-1)
        B = tok.size
        cached = getattr(self, "_batch", None)
        if cached is not None and B != cached:   # the library reads one id per cached sequence from this array
            raise _lib.InvalidInput(f"decode_step got {B} ids for a context of {cached} sequences")
        logits = np.empty((B, self.config.vocab_size), dtype=np.float32) if want_logits else None
        pick = np.empty(B, dtype=np.uint32)
        check(self._lib.rg_gpt_decode_step(self._h, tok.ctypes.data_as(_lib._U32P),
                                           logits.ctypes.data_as(_lib._FP) if want_logits else None,
                                           pick.ctypes.data_as(_lib._U32P)))
        return logits, pick

    def decode_run(self, n_steps: int) -> None:
        check(self._lib.rg_gpt_decode_run(self._h, int(n_steps)))

    def rewind(self, T: int, tok: Optional[np.ndarray] = None) -> None:
        if tok is not None:
            tok = np.ascontiguousarray(tok, dtype=np.uint32).reshape(-1)
            cached = getattr(self, "_batch", None)
            if cached is not None and tok.size != cached:
                raise _lib.InvalidInput(f"rewind got {tok.size} ids for a context of {cached} sequences")
        check(self._lib.rg_gpt_rewind(self._h, int(T), tok.ctypes.data_as(_lib._U32P) if tok is not None else None))

    def read_tokens(self, start: int, n: int, batch: int) -> np.ndarray:
        out = np.empty((batch, n), dtype=np.uint32)
        check(self._lib.rg_gpt_read_tokens(self._h, int(start), int(n), out.ctypes.data_as(_lib._U32P)))
        return out

    @property
    def position(self) -> int:
        return int(self._lib.rg_gpt_position(self._h))

    def reset(self) -> None:
        check(self._lib.rg_gpt_reset(self._h))

    # -- WasmGptTrainer::generate (wasm_api.rs:97-163), batched
    def generate(self, prompt_ids, max_new_tokens: int, temperature: float = 1.0, top_k: int = 1,
                 seed: int = 0) -> np.ndarray:
        p = np.ascontiguousarray(prompt_ids, dtype=np.uint32)
        single = p.ndim == 1
        if single:
            p = p[None, :]
        B, P = p.shape
        out = np.empty((B, max_new_tokens), dtype=np.uint32)
        check(self._lib.rg_gpt_generate(self._h, p.ctypes.data_as(_lib._U32P), B, P, int(max_new_tokens),
                                        float(temperature), int(top_k), int(seed), out.ctypes.data_as(_lib._U32P)))
        return out[0] if single else out

    def trace(self, on: bool = True) -> None:
        """Record per-stage device timestamps of the last token step of each decode_run."""
        check(self._lib.rg_gpt_trace_enable(self._h, 1 if on else 0))

    def read_trace(self, cap_rows: int = 1 << 16) -> np.ndarray:
        """Rows [cta, op, stage, layer, t_start, t_input, t_dots, t_stored (ns), chunk-wait cycles, poll cycles,
        t_fetched, t_loop (ns)]."""
        out = np.zeros((cap_rows, 12), dtype=np.uint64)
        n = C.c_size_t(0)
        check(self._lib.rg_gpt_trace_read(self._h, out.ctypes.data_as(C.POINTER(C.c_uint64)), cap_rows, C.byref(n)))
        return out[: n.value]

    def debug_hook(self, what: int, value: int = 0) -> None:
        """Test hook of the bounded device waits (rg_debug_hook; the header lists the values of `what`)."""
        check(self._lib.rg_debug_hook(self.backend._ctx, self._h, int(what), int(value)))

    def decode_step_bytes(self, batch: int, mean_ctx: float) -> float:
        return float(self._lib.rg_gpt_decode_step_bytes(self._h, int(batch), float(mean_ctx)))
