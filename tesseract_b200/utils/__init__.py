"""Auxiliary subsystems: environment registry, structured metrics, NVTX ranges, rank watchdog, checkpoints."""
from . import checkpoint, env, metrics, nvtx, watchdog  # noqa: F401
from .errors import DeviceError, ShapeError, TesseractError, check

__all__ = ["checkpoint", "env", "metrics", "nvtx", "watchdog", "TesseractError", "ShapeError", "DeviceError", "check"]
