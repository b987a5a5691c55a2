"""Parallelism: communication backends, tensor / sequence / data / expert parallel layers, and the factory that
wires a model and a Trainer for a given world size."""
from .comm import CommBackend, NcclCommBackend, SimCommBackend
from .data_parallel import GradReducer
from .factory import build_parallel_trainer
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

__all__ = ["CommBackend", "NcclCommBackend", "SimCommBackend", "GradReducer", "build_parallel_trainer",
           "ColumnParallelLinear", "RowParallelLinear"]
