"""ctypes binding of ``libtesseract_b200_cuda.so`` (the sm_100a kernels) and import of the host runtime.

The CUDA library exports a plain C ABI: every entry point takes raw device pointers, sizes and a
``cudaStream_t`` and returns 0 or an error code. On a machine with a GPU a missing library is an error
(``require()`` raises); nothing here falls back silently.
"""
from __future__ import annotations

import ctypes
import importlib.util
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "_lib"
_CUDA_LIB_PATH = _LIB_DIR / "libtesseract_b200_cuda.so"

_lock = threading.Lock()
_lib = None
_host = None
_launch_count = 0  # kernels launched through this binding (bench.py reports it)

P, I, L, F = c_void_p, c_int, c_longlong, c_float

# name -> argtypes (restype is always int unless listed in _RESTYPES)
_SIGNATURES = {
    "tsb_read_status": [P],
    "tsb_sm_count": [],
    "tsb_probe": [P, P],
    "tsb_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, I, I, P],
    "tsb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, I, P],
    "tsb_rmsnorm_bwd_parts": [I],
    "tsb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "tsb_swiglu_fwd": [P, P, L, I, I, P],
    "tsb_swiglu_bwd": [P, P, P, L, I, I, P],
    "tsb_rope_qkv": [P, P, P, P, L, I, I, I, I, I, F, I, P],
    "tsb_embedding_fwd": [P, P, P, L, I, I, I, P],
    "tsb_embedding_bwd": [P, P, P, L, I, I, I, I, P],
    "tsb_ce_stats": [P, P, P, L, I, L, I, I, P],
    "tsb_ce_loss_grad": [P, P, P, P, L, I, L, I, F, I, I, P],
    "tsb_adam_flat": [P, P, P, P, P, L, F, F, F, F, F, F, F, P, I, I, P],
    "tsb_adam_chunk_elems": [],
    "tsb_adam_multi": [P, P, I, F, F, F, F, F, F, F, P, I, I, P],
    "tsb_sumsq": [P, L, P, I, P],
    "tsb_clip_coef": [P, P, F, F, P],
}
_RESTYPES = {"tsb_error_string": c_char_p}
_OPTIONAL_SIGNATURES: dict = {}  # filled by later translation units via register_signatures()


def register_signatures(sigs: dict) -> None:
    """Declare further entry points (called by the op modules that own them)."""
    _SIGNATURES.update(sigs)
    if _lib is not None:
        _bind(_lib, sigs)


def _bind(lib, sigs):
    for name, argtypes in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, c_int)
    try:
        lib.tsb_error_string.argtypes = [c_int]
        lib.tsb_error_string.restype = c_char_p
    except AttributeError:
        pass


def cuda_lib_path() -> Path:
    return _CUDA_LIB_PATH


def available() -> bool:
    """True when the built CUDA library exists on disk (it may still need a GPU to run)."""
    return _CUDA_LIB_PATH.exists()


def lib():
    """The loaded CUDA library (ctypes.CDLL). Raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not _CUDA_LIB_PATH.exists():
                    raise RuntimeError(
                        f"{_CUDA_LIB_PATH} is missing: run `python -m tesseract_b200.build` "
                        "(CUDA tensors are only served by the native sm_100a kernels)")
                loaded = ctypes.CDLL(str(_CUDA_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
                _bind(loaded, _SIGNATURES)
                _lib = loaded
    return _lib


def host():
    """The pybind11 host runtime module (``_tsb_host``), or None if it has not been built."""
    global _host
    if _host is None:
        cands = sorted(_LIB_DIR.glob("_tsb_host*.so"))
        if not cands:
            return None
        spec = importlib.util.spec_from_file_location("_tsb_host", cands[0])
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _host = mod
    return _host


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    """Raise on a non-zero return code of a native entry point."""
    global _launch_count
    if rc == 0:
        _launch_count += 1
        return
    if rc == -2:
        raise NativeError(f"{what}: bad argument (shape, alignment or dtype not supported by the kernel)")
    if rc == -3:
        raise NativeError(f"{what}: TMA descriptor encoding failed")
    try:
        msg = lib().tsb_error_string(rc).decode()
    except Exception:  # pragma: no cover
        msg = "?"
    raise NativeError(f"{what}: CUDA error {rc} ({msg})")


def launch_count() -> int:
    return _launch_count


def add_launches(n: int) -> None:
    """Entry points that launch more than one kernel account for the extra ones here."""
    global _launch_count
    _launch_count += n


def read_status(stream_ptr: int = 0) -> int:
    """Status word of the current device: 0, or the code a bounded wait recorded (then cleared)."""
    return int(lib().tsb_read_status(stream_ptr))


DTYPE_CODES = {}


def dtype_code(dtype) -> int:
    import torch

    if not DTYPE_CODES:
        DTYPE_CODES.update({torch.float32: 0, torch.bfloat16: 1, torch.float16: 2})
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported by the native kernels (fp32 / bf16 / fp16)") from None


def stream_ptr(device=None) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
