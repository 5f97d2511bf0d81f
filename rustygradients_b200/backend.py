"""Host-side mirror of the reference's `Backend` trait (src/backend/mod.rs:130-227)
over the C ABI: same method names, argument meaning and error variants as
`CudaBackend` (src/backend/cuda.rs) so tests read like the reference's own."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib
from ._lib import check


def _shape_arr(shape: Sequence[int]):
    return (C.c_size_t * max(1, len(shape)))(*[int(s) for s in shape])


class Storage:
    """CudaStorage {data, shape, device} (src/backend/cuda.rs:29-33): an immutable
    device buffer owned by the library; freed when the Python object dies."""

    def __init__(self, backend: "B200Backend", handle: int):
        self._backend = backend
        self._h = C.c_void_p(handle)

    @property
    def shape(self):
        lib = _lib.load()
        nd = C.c_int(0)
        buf = (C.c_size_t * 8)()
        check(lib.rg_shape(self._h, buf, 8, C.byref(nd)))
        return [int(buf[i]) for i in range(nd.value)]

    def __len__(self) -> int:
        return int(_lib.load().rg_storage_len(self._h))

    def __del__(self):
        try:
            if self._h and self._backend._ctx:
                _lib.load().rg_storage_free(self._h)
        except Exception:
            pass
        self._h = None


class B200Backend:
    """`CudaBackend::new(device_index)` (cuda.rs:87-125)."""

    def __init__(self, device_index: int = 0):
        lib = _lib.load()
        ctx = C.c_void_p()
        check(lib.rg_ctx_create(int(device_index), C.byref(ctx)))
        self._ctx = ctx
        self._lib = lib
        self.device_index = device_index

    # -- CudaBackend::device_count / is_available (cuda.rs:127-135)
    @staticmethod
    def device_count() -> int:
        return int(_lib.load().rg_device_count())

    @staticmethod
    def is_available() -> bool:
        return B200Backend.device_count() > 0

    def device_type(self):
        return ("cuda", self.device_index)

    def synchronize(self) -> None:
        check(self._lib.rg_synchronize(self._ctx))

    @property
    def stream(self) -> int:
        return int(self._lib.rg_ctx_stream(self._ctx) or 0)

    @property
    def launch_count(self) -> int:
        return int(self._lib.rg_ctx_launch_count(self._ctx))

    def close(self) -> None:
        if self._ctx:
            self._lib.rg_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        # storages may outlive the backend object in GC order; keep the context
        # until the process exits rather than risk a use-after-free
        pass

    # -- memory operations
    def _wrap(self, h: C.c_void_p) -> Storage:
        return Storage(self, h.value)

    def zeros(self, shape) -> Storage:
        h = C.c_void_p()
        check(self._lib.rg_zeros(self._ctx, _shape_arr(shape), len(shape), C.byref(h)))
        return self._wrap(h)

    def ones(self, shape) -> Storage:
        h = C.c_void_p()
        check(self._lib.rg_ones(self._ctx, _shape_arr(shape), len(shape), C.byref(h)))
        return self._wrap(h)

    def from_slice(self, data, shape) -> Storage:
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        h = C.c_void_p()
        check(self._lib.rg_from_slice(self._ctx, a.ctypes.data_as(_lib._FP), a.size, _shape_arr(shape), len(shape),
                                      C.byref(h)))
        return self._wrap(h)

    def to_vec(self, st: Storage) -> np.ndarray:
        out = np.empty(len(st), dtype=np.float32)
        check(self._lib.rg_to_vec(self._ctx, st._h, out.ctypes.data_as(_lib._FP), out.size))
        return out

    def to_array(self, st: Storage) -> np.ndarray:
        return self.to_vec(st).reshape(st.shape)

    def shape(self, st: Storage):
        return st.shape

    # -- ops
    def _bin(self, fn, a, b):
        h = C.c_void_p()
        check(fn(self._ctx, a._h, b._h, C.byref(h)))
        return self._wrap(h)

    def _un(self, fn, a):
        h = C.c_void_p()
        check(fn(self._ctx, a._h, C.byref(h)))
        return self._wrap(h)

    def add(self, a, b): return self._bin(self._lib.rg_add, a, b)
    def sub(self, a, b): return self._bin(self._lib.rg_sub, a, b)
    def mul(self, a, b): return self._bin(self._lib.rg_mul, a, b)
    def matmul(self, a, b): return self._bin(self._lib.rg_matmul, a, b)
    def relu(self, a): return self._un(self._lib.rg_relu, a)
    def sigmoid(self, a): return self._un(self._lib.rg_sigmoid, a)
    def exp(self, a): return self._un(self._lib.rg_exp, a)
    def log(self, a): return self._un(self._lib.rg_log, a)
    def gelu(self, a): return self._un(self._lib.rg_gelu, a)
    def softmax(self, a): return self._un(self._lib.rg_softmax, a)
    def sum(self, a): return self._un(self._lib.rg_sum, a)
    def embedding(self, indices, weights): return self._bin(self._lib.rg_embedding, indices, weights)
    def sparse_cross_entropy(self, logits, targets): return self._bin(self._lib.rg_sparse_cross_entropy, logits, targets)

    def powf(self, a, power: float):
        h = C.c_void_p()
        check(self._lib.rg_powf(self._ctx, a._h, float(power), C.byref(h)))
        return self._wrap(h)

    def sum_axis(self, a, axis: int):
        h = C.c_void_p()
        check(self._lib.rg_sum_axis(self._ctx, a._h, int(axis), C.byref(h)))
        return self._wrap(h)

    def reshape(self, a, new_shape):
        h = C.c_void_p()
        check(self._lib.rg_reshape(self._ctx, a._h, _shape_arr(new_shape), len(new_shape), C.byref(h)))
        return self._wrap(h)

    def transpose(self, a, axis1: int, axis2: int):
        h = C.c_void_p()
        check(self._lib.rg_transpose(self._ctx, a._h, int(axis1), int(axis2), C.byref(h)))
        return self._wrap(h)

    def layer_norm(self, x, gamma, beta, epsilon: float):
        h = C.c_void_p()
        check(self._lib.rg_layer_norm(self._ctx, x._h, gamma._h, beta._h, float(epsilon), C.byref(h)))
        return self._wrap(h)
