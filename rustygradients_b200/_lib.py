"""ctypes binding of librg_b200.so (the C ABI declared in include/rg_b200.h).

There is no CPU fallback: if the shared library is missing, or a call needs a
GPU and none is present, the error is raised to the caller."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "librg_b200.so")

# rg_status values (include/rg_b200.h)
RG_OK, RG_ERR_SHAPE, RG_ERR_DIMENSION, RG_ERR_INVALID_INPUT, RG_ERR_BACKEND, \
    RG_ERR_UNSUPPORTED, RG_ERR_CONTEXT_FULL, RG_ERR_TIMEOUT, RG_ERR_SERIALIZATION, RG_ERR_IO = range(10)
RG_NAMES_AUTO, RG_NAMES_RUSTY, RG_NAMES_HF_GPT2 = 0, 1, 2
RG_ACT_RELU, RG_ACT_GELU_TANH = 0, 1
RG_DTYPE_F32, RG_DTYPE_BF16 = 0, 1


class RustyGradientsError(Exception):
    """Base of the error variants of src/error.rs:13-50."""
    status = -1


class ShapeError(RustyGradientsError):
    status = RG_ERR_SHAPE


class DimensionError(RustyGradientsError):
    status = RG_ERR_DIMENSION


class InvalidInput(RustyGradientsError):
    status = RG_ERR_INVALID_INPUT


class BackendError(RustyGradientsError):
    status = RG_ERR_BACKEND


class Unsupported(RustyGradientsError):
    status = RG_ERR_UNSUPPORTED


class ContextFull(RustyGradientsError):
    status = RG_ERR_CONTEXT_FULL


class DeviceTimeout(RustyGradientsError):
    status = RG_ERR_TIMEOUT


class SerializationError(RustyGradientsError):
    status = RG_ERR_SERIALIZATION


class IoError(RustyGradientsError):
    status = RG_ERR_IO


_ERRORS = {c.status: c for c in (ShapeError, DimensionError, InvalidInput, BackendError,
                                 Unsupported, ContextFull, DeviceTimeout, SerializationError, IoError)}


class GptConfigC(C.Structure):
    _fields_ = [("block_size", C.c_size_t), ("vocab_size", C.c_size_t), ("num_layers", C.c_size_t),
                ("num_heads", C.c_size_t), ("embedding_dim", C.c_size_t), ("causal", C.c_int),
                ("activation", C.c_int), ("weight_dtype", C.c_int), ("max_batch", C.c_size_t),
                ("tp_rank", C.c_int), ("tp_size", C.c_int)]


_P = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_SZ = C.c_size_t
_SZP = C.POINTER(C.c_size_t)
_FP = C.POINTER(C.c_float)
_U32P = C.POINTER(C.c_uint32)

# name -> (restype, argtypes); restype None means rg_status
SIGNATURES = {
    "rg_last_error": (C.c_char_p, []),
    "rg_version": (C.c_char_p, []),
    "rg_device_count": (C.c_int, []),
    "rg_ctx_create": (None, [C.c_int, _PP]),
    "rg_ctx_destroy": (None, [_P]),
    "rg_synchronize": (None, [_P]),
    "rg_ctx_stream": (C.c_void_p, [_P]),
    "rg_ctx_launch_count": (C.c_uint64, [_P]),
    "rg_zeros": (None, [_P, _SZP, C.c_int, _PP]),
    "rg_ones": (None, [_P, _SZP, C.c_int, _PP]),
    "rg_from_slice": (None, [_P, _FP, _SZ, _SZP, C.c_int, _PP]),
    "rg_to_vec": (None, [_P, _P, _FP, _SZ]),
    "rg_shape": (None, [_P, _SZP, C.c_int, C.POINTER(C.c_int)]),
    "rg_storage_len": (C.c_size_t, [_P]),
    "rg_storage_free": (None, [_P]),
    "rg_add": (None, [_P, _P, _P, _PP]),
    "rg_sub": (None, [_P, _P, _P, _PP]),
    "rg_mul": (None, [_P, _P, _P, _PP]),
    "rg_matmul": (None, [_P, _P, _P, _PP]),
    "rg_relu": (None, [_P, _P, _PP]),
    "rg_sigmoid": (None, [_P, _P, _PP]),
    "rg_exp": (None, [_P, _P, _PP]),
    "rg_log": (None, [_P, _P, _PP]),
    "rg_powf": (None, [_P, _P, C.c_float, _PP]),
    "rg_gelu": (None, [_P, _P, _PP]),
    "rg_softmax": (None, [_P, _P, _PP]),
    "rg_sum": (None, [_P, _P, _PP]),
    "rg_sum_axis": (None, [_P, _P, _SZ, _PP]),
    "rg_reshape": (None, [_P, _P, _SZP, C.c_int, _PP]),
    "rg_transpose": (None, [_P, _P, _SZ, _SZ, _PP]),
    "rg_embedding": (None, [_P, _P, _P, _PP]),
    "rg_layer_norm": (None, [_P, _P, _P, _P, C.c_float, _PP]),
    "rg_sparse_cross_entropy": (None, [_P, _P, _P, _PP]),
    "rg_gpt_create": (None, [_P, C.POINTER(GptConfigC), _PP]),
    "rg_gpt_destroy": (None, [_P]),
    "rg_gpt_num_params": (C.c_int, [_P]),
    "rg_gpt_param_shape": (None, [_P, C.c_int, _SZP]),
    "rg_gpt_load_params": (None, [_P, C.POINTER(_FP), C.POINTER(_SZP), C.POINTER(C.c_int), C.c_int]),
    "rg_gpt_forward": (None, [_P, _FP, _SZ, _SZ, _FP]),
    "rg_gpt_prefill": (None, [_P, _U32P, _SZ, _SZ, _FP, _U32P]),
    "rg_gpt_decode_step": (None, [_P, _U32P, _FP, _U32P]),
    "rg_gpt_generate": (None, [_P, _U32P, _SZ, _SZ, _SZ, C.c_float, _SZ, C.c_uint64, _U32P]),
    "rg_gpt_decode_run": (None, [_P, _SZ]),
    "rg_gpt_rewind": (None, [_P, _SZ, _U32P]),
    "rg_gpt_read_tokens": (None, [_P, _SZ, _SZ, _U32P]),
    "rg_gpt_position": (C.c_size_t, [_P]),
    "rg_gpt_reset": (None, [_P]),
    "rg_gpt_decode_step_bytes": (C.c_double, [_P, _SZ, C.c_double]),
    "rg_gpt_tp_unique_id": (None, [C.POINTER(C.c_uint8)]),
    "rg_gpt_tp_init": (None, [_P, C.POINTER(C.c_uint8)]),
    "rg_gpt_tp_fused": (C.c_int, [_P]),
    "rg_gpt_trace_enable": (None, [_P, C.c_int]),
    "rg_gpt_trace_read": (None, [_P, C.POINTER(C.c_uint64), _SZ, _SZP]),
    "rg_debug_hook": (None, [_P, _P, C.c_int, C.c_longlong]),
    "rg_token_loop_plan": (None, [C.c_int] * 9 + [C.POINTER(C.c_longlong)]),
    "rg_linear_row_noalloc": (None, [_P, _P, _P, _P, _SZ, _SZ, _P]),
    "rg_model_metadata_read": (None, [C.c_char_p, C.POINTER(GptConfigC)]),
    "rg_gpt_load_safetensors": (None, [_P, C.c_char_p, C.c_int]),
    "rg_gpt_load_json": (None, [_P, C.c_char_p]),
    "rg_tokenizer_char_from_text": (None, [C.c_char_p, _SZ, _PP]),
    "rg_tokenizer_char_from_vocab": (None, [_U32P, _SZ, _PP]),
    "rg_tokenizer_bpe_load": (None, [C.c_char_p, _PP]),
    "rg_tokenizer_vocab_size": (None, [_P, _SZP]),
    "rg_tokenizer_encode": (None, [_P, C.c_char_p, _SZ, _U32P, _SZ, _SZP]),
    "rg_tokenizer_decode": (None, [_P, _U32P, _SZ, C.c_char_p, _SZ, _SZP]),
    "rg_tokenizer_free": (C.c_int, [_P]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and declare every entry point.  Raises if the
    library has not been built (`python -m rustygradients_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(f"{LIB_PATH} is missing: build it with `python -m rustygradients_b200.build`; "
                           "there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = C.c_int if res is None else res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != RG_OK:
        msg = load().rg_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(status, RustyGradientsError)(msg)
