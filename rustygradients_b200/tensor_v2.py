"""Host-side mirror of the reference's device-aware tensor (`TensorV2`, `DType`: src/tensor_v2.rs:16-23, 64-83,
85-305, 335-351), its `Device` handle (src/backend/mod.rs:25-125) and the free functions of `ops_v2`
(src/ops_v2/basic.rs:15-118, src/ops_v2/matmul.rs:15-50), over this library's `B200Backend`.

The wrapper adds no arithmetic of its own: every operation forwards to the `Backend` method of the same name, exactly as
the reference's does.  Two differences, both forced by what this library is:

* the reference computes every `TensorV2` operation on the host (its non-CPU arms are `unimplemented!`); here the
  arithmetic exists only on the GPU, so an operation needs its operands on `Device.cuda(i)` and raises `Unsupported`
  for host tensors instead of computing on the CPU.  `to_device` moves data either way;
* gradients are outside this library (forward path only): `requires_grad` is carried and propagated like the
  reference does (`a.requires_grad || b.requires_grad`), `grad()` is always None and no backward context is attached.
"""
from __future__ import annotations

import enum
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from ._lib import ShapeError, Unsupported
from .backend import B200Backend, Storage


class DType(enum.Enum):
    """src/tensor_v2.rs:16-23.  Tensors are created as F32, like the reference's constructors."""
    F32 = "F32"
    F16 = "F16"
    BF16 = "BF16"
    I32 = "I32"
    U32 = "U32"


class Device:
    """src/backend/mod.rs:41-125: `Device::cpu()`, `Device::cuda(index)`, `default_device()`, `device_type()`."""
    _backends: Dict[int, B200Backend] = {}

    def __init__(self, kind: str, index: int = 0):
        self._kind, self._index = kind, int(index)

    @staticmethod
    def cpu() -> "Device":
        return Device("cpu")

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        """Fails like the reference's (BackendError) when the device cannot be opened."""
        d = Device("cuda", index)
        d.backend()
        return d

    @staticmethod
    def default_device() -> "Device":
        """CUDA device 0 when one is visible, else the host (mod.rs:98-113)."""
        return Device.cuda(0) if B200Backend.is_available() else Device.cpu()

    def device_type(self) -> Tuple:
        return ("cuda", self._index) if self._kind == "cuda" else ("cpu",)

    def is_cuda(self) -> bool:
        return self._kind == "cuda"

    def backend(self) -> B200Backend:
        if self._kind != "cuda":
            raise Unsupported("the host device has no Backend in this library; use Device.cuda(i)")
        if self._index not in Device._backends:
            Device._backends[self._index] = B200Backend(self._index)
        return Device._backends[self._index]

    def __eq__(self, other) -> bool:
        return isinstance(other, Device) and self.device_type() == other.device_type()

    def __hash__(self) -> int:
        return hash(self.device_type())

    def __repr__(self) -> str:
        return f"Device{self.device_type()}"


class TensorV2:
    """src/tensor_v2.rs:64-83.  `data` is a host array (`TensorData::Cpu`) or a device `Storage`."""

    def __init__(self, data, requires_grad: bool = False, device: Optional[Device] = None):
        device = device or Device.cpu()
        if isinstance(data, Storage):
            if not device.is_cuda():
                raise Unsupported("a device Storage belongs to a cuda Device")
            self._data = data
        else:
            arr = np.ascontiguousarray(np.asarray(data, dtype=np.float32))
            self._data = device.backend().from_slice(arr.reshape(-1), arr.shape) if device.is_cuda() else arr
        self._device = device
        self._dtype = DType.F32
        self._requires_grad = bool(requires_grad)
        self.ctx = None

    # ---- constructors (tensor_v2.rs:87-157, 337-351)
    @staticmethod
    def new(data, requires_grad: bool, device: Device) -> "TensorV2":
        return TensorV2(data, requires_grad, device)

    @staticmethod
    def new_cpu(data, requires_grad: bool) -> "TensorV2":
        return TensorV2(data, requires_grad, Device.cpu())

    @staticmethod
    def zeros(shape: Sequence[int], requires_grad: bool, device: Device) -> "TensorV2":
        if device.is_cuda():
            return TensorV2(device.backend().zeros(shape), requires_grad, device)
        return TensorV2(np.zeros(tuple(shape), np.float32), requires_grad, device)

    @staticmethod
    def ones(shape: Sequence[int], requires_grad: bool, device: Device) -> "TensorV2":
        if device.is_cuda():
            return TensorV2(device.backend().ones(shape), requires_grad, device)
        return TensorV2(np.ones(tuple(shape), np.float32), requires_grad, device)

    @staticmethod
    def randn(shape: Sequence[int], requires_grad: bool) -> "TensorV2":
        """Standard-normal host tensor (unseeded, as in the reference)."""
        return TensorV2.new_cpu(np.random.standard_normal(tuple(shape)).astype(np.float32), requires_grad)

    @staticmethod
    def from_slice(data, shape: Sequence[int], requires_grad: bool) -> "TensorV2":
        flat = np.asarray(data, dtype=np.float32).reshape(-1)
        if flat.size != int(np.prod(tuple(shape), dtype=np.int64)):
            raise ShapeError(f"{flat.size} values do not fill shape {list(shape)}")
        return TensorV2.new_cpu(flat.reshape(tuple(shape)), requires_grad)

    # ---- accessors (tensor_v2.rs:159-204)
    def shape(self):
        return list(self._data.shape)

    def device(self) -> Device:
        return self._device

    def dtype(self) -> DType:
        return self._dtype

    def requires_grad(self) -> bool:
        return self._requires_grad

    def to_device(self, target: Device) -> "TensorV2":
        if target == self._device:
            return self
        return TensorV2(self.to_cpu_data(), self._requires_grad, target)

    def to_cpu_data(self) -> np.ndarray:
        if self._device.is_cuda():
            return self._device.backend().to_array(self._data)
        return self._data.copy()

    def grad(self):
        return None

    def zero_grad(self) -> None:
        pass

    # ---- operations (tensor_v2.rs:208-304): one Backend call each
    def _backend_with(self, *others: "TensorV2") -> B200Backend:
        for t in (self,) + others:
            if not t._device.is_cuda():
                raise Unsupported("TensorV2 arithmetic runs on Device.cuda(i) in this library: call to_device first")
            if t._device != self._device:
                raise Unsupported("operands live on different devices")
        return self._device.backend()

    def _wrap(self, st: Storage, *parents: "TensorV2") -> "TensorV2":
        return TensorV2(st, any(p._requires_grad for p in parents), self._device)

    def add(self, other: "TensorV2") -> "TensorV2":
        return self._wrap(self._backend_with(other).add(self._data, other._data), self, other)

    def sub(self, other: "TensorV2") -> "TensorV2":
        return self._wrap(self._backend_with(other).sub(self._data, other._data), self, other)

    def mul(self, other: "TensorV2") -> "TensorV2":
        return self._wrap(self._backend_with(other).mul(self._data, other._data), self, other)

    def matmul(self, other: "TensorV2") -> "TensorV2":
        return self._wrap(self._backend_with(other).matmul(self._data, other._data), self, other)

    def relu(self) -> "TensorV2":
        return self._wrap(self._backend_with().relu(self._data), self)

    def softmax(self) -> "TensorV2":
        return self._wrap(self._backend_with().softmax(self._data), self)

    def reshape(self, new_shape: Sequence[int]) -> "TensorV2":
        return self._wrap(self._backend_with().reshape(self._data, new_shape), self)

    def transpose(self, axis1: int, axis2: int) -> "TensorV2":
        return self._wrap(self._backend_with().transpose(self._data, axis1, axis2), self)

    # ---- identity semantics of tensor_v2.rs:307-319 (two handles are equal when they share the data)
    def __eq__(self, other) -> bool:
        return isinstance(other, TensorV2) and self._data is other._data

    def __hash__(self) -> int:
        return id(self._data)

    def __repr__(self) -> str:
        return (f"TensorV2 {{ shape: {self.shape()}, device: {self._device.device_type()}, dtype: {self._dtype.name}, "
                f"requires_grad: {str(self._requires_grad).lower()} }}")


# ---- ops_v2 (src/ops_v2/basic.rs:15, 56, 94; src/ops_v2/matmul.rs:15): forward through the backend
def add_op(a: TensorV2, b: TensorV2) -> TensorV2:
    return a.add(b)


def mul_op(a: TensorV2, b: TensorV2) -> TensorV2:
    return a.mul(b)


def sub_op(a: TensorV2, b: TensorV2) -> TensorV2:
    return a.sub(b)


def matmul_op(a: TensorV2, b: TensorV2) -> TensorV2:
    return a.matmul(b)
