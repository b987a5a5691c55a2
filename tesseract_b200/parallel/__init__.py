"""Parallelism: communication backends, tensor / sequence / data / expert parallel layers, and the factory that
wires a model and a Trainer for a given world size."""
from .comm import CommBackend, NcclCommBackend, SimCommBackend
from .data_parallel import GradReducer
from .factory import build_parallel_trainer
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .zero import ShardedAdam, shard_ranges

__all__ = ["ShardedAdam", "shard_ranges", "CommBackend", "NcclCommBackend", "SimCommBackend", "GradReducer", "build_parallel_trainer",
           "ColumnParallelLinear", "RowParallelLinear"]
