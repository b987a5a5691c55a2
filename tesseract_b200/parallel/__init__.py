"""Parallelism: communication backends, tensor / sequence / data / expert parallel layers, and the
factory that wires a model and a Trainer for a given world size."""
from .factory import build_parallel_trainer

__all__ = ["build_parallel_trainer"]
