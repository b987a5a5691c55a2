"""Drop-in ``tesseract`` package: the reference's Python surface (python/tesseract/__init__.py:19-52) served by
``tesseract_b200``."""
from . import _core
from ._core import DType, Device, Tensor, backward, io, models, nn, ops, optim

float32 = DType.float32
float64 = DType.float64
int64 = DType.int64
int32 = DType.int32

__all__ = ["Tensor", "DType", "Device", "backward", "ops", "nn", "optim", "models", "io", "float32", "float64",
           "int64", "int32"]
__version__ = "0.1.0"
