"""tesseract_b200 -- a Blackwell-native (sm_100a) LLM training and serving framework with the public
surface of Scifan/Tesseract. PyTorch is the framework layer; the hot ops are hand-written CUDA kernels
in ``csrc/`` (tcgen05 / TMEM / TMA), loaded from ``_lib/``."""
from . import _native, ops  # noqa: F401

__version__ = "0.1.0"


def native_available() -> bool:
    """True when the built sm_100a kernel library is present."""
    return _native.available()
