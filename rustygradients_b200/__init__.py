"""B200-native GPT token loop behind RustyGradients' Backend / GPT model interface.

The arithmetic lives in lib/librg_b200.so (CUDA, sm_100a, C ABI in
include/rg_b200.h); this package is the thin host-side mirror of the reference's
`Backend` trait, `TensorV2` / `DType`, `GptConfig`, `GPTModel` and `generate`."""
from ._lib import (BackendError, ContextFull, DeviceTimeout, DimensionError, InvalidInput, IoError,
                   RustyGradientsError, SerializationError, ShapeError, Unsupported)
from .backend import B200Backend, Storage
from .gpt import GptConfig, GPTModel
from .tensor_v2 import Device, DType, TensorV2
from .tokenization import BPETokenizer, CharTokenizer

__all__ = ["B200Backend", "Storage", "GptConfig", "GPTModel", "RustyGradientsError", "ShapeError",
           "DimensionError", "InvalidInput", "BackendError", "Unsupported", "ContextFull", "DeviceTimeout",
           "SerializationError", "IoError", "CharTokenizer", "BPETokenizer", "TensorV2", "DType", "Device"]
