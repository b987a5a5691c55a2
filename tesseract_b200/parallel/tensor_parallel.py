"""Megatron-style tensor-parallel Linear layers in ONE process (every rank's shard lives in the module), driven by
a shard-list ``CommBackend``: the reference's simulation harness (src/distributed/TensorParallel.cpp:63-215).

Parameter names: ``shard.{r}.weight`` / ``shard.{r}.bias`` and, for the row-parallel layer, a replicated ``bias``
added once after the reduction. ``from_dense`` slices a dense layer the way a sharded checkpoint load does.
The rank-local (one process per GPU) layers with fused communication are in ``parallel/tp_layers.py``.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
from torch import nn

from ..nn.modules import Linear, Module
from .comm import CommBackend, SimCommBackend


def _uniform(shape, bound, dtype):
    return nn.Parameter(torch.empty(shape, dtype=dtype).uniform_(-bound, bound))


class _ShardHolder(Module):
    """Registers parameters under dotted names ``shard.{r}.weight`` like the reference."""

    def _register(self, name: str, p: nn.Parameter) -> None:
        self._parameters[name] = p

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for n, p in self._parameters.items():
            if p is not None:
                yield (prefix + ("." if prefix else "") + n, p)


class ColumnParallelLinear(_ShardHolder):
    def __init__(self, in_features: int, out_features: int, comm: Optional[CommBackend] = None, bias: bool = True,
                 gather_output: bool = True, dtype=torch.float32):
        super().__init__()
        comm = comm or SimCommBackend(1)
        w = comm.world_size()
        if in_features <= 0 or out_features <= 0:
            raise ValueError("ColumnParallelLinear: features must be positive")
        if out_features % w:
            raise ValueError(f"ColumnParallelLinear: out_features {out_features} not divisible by world_size {w}")
        self.in_features, self.out_features, self.comm, self.gather_output = in_features, out_features, comm, gather_output
        self.world = w
        self.out_per_rank = out_features // w
        bound = 1.0 / math.sqrt(in_features)
        self.weight_shards: List[nn.Parameter] = []
        self.bias_shards: List[nn.Parameter] = []
        for r in range(w):
            p = _uniform((self.out_per_rank, in_features), bound, dtype)
            self._register(f"shard.{r}.weight", p)
            self.weight_shards.append(p)
            if bias:
                b = _uniform((self.out_per_rank,), bound, dtype)
                self._register(f"shard.{r}.bias", b)
                self.bias_shards.append(b)

    def forward_shards(self, x: torch.Tensor) -> List[torch.Tensor]:
        return [torch.nn.functional.linear(x, self.weight_shards[r], self.bias_shards[r] if self.bias_shards else None)
                for r in range(self.world)]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.comm.all_gather(self.forward_shards(x), -1)

    @classmethod
    def from_dense(cls, dense: Linear, comm: CommBackend, gather_output: bool = True) -> "ColumnParallelLinear":
        out_f, in_f = dense.weight.shape
        layer = cls(in_f, out_f, comm, dense.bias is not None, gather_output, dense.weight.dtype)
        n = layer.out_per_rank
        with torch.no_grad():
            for r in range(layer.world):
                layer.weight_shards[r].copy_(dense.weight[r * n:(r + 1) * n])
                if dense.bias is not None:
                    layer.bias_shards[r].copy_(dense.bias[r * n:(r + 1) * n])
        return layer


class RowParallelLinear(_ShardHolder):
    def __init__(self, in_features: int, out_features: int, comm: Optional[CommBackend] = None, bias: bool = True,
                 dtype=torch.float32):
        super().__init__()
        comm = comm or SimCommBackend(1)
        w = comm.world_size()
        if in_features <= 0 or out_features <= 0:
            raise ValueError("RowParallelLinear: features must be positive")
        if in_features % w:
            raise ValueError(f"RowParallelLinear: in_features {in_features} not divisible by world_size {w}")
        self.in_features, self.out_features, self.comm, self.world = in_features, out_features, comm, w
        self.in_per_rank = in_features // w
        bound = 1.0 / math.sqrt(in_features)
        self.weight_shards: List[nn.Parameter] = []
        for r in range(w):
            p = _uniform((out_features, self.in_per_rank), bound, dtype)
            self._register(f"shard.{r}.weight", p)
            self.weight_shards.append(p)
        self.bias = None
        if bias:
            self.bias = _uniform((out_features,), bound, dtype)

    def forward_shards(self, x_shards: List[torch.Tensor]) -> torch.Tensor:
        if len(x_shards) != self.world:
            raise ValueError(f"RowParallelLinear.forward_shards: expected {self.world} input shards, got {len(x_shards)}")
        partials = [torch.nn.functional.linear(x_shards[r], self.weight_shards[r]) for r in range(self.world)]
        y = self.comm.all_reduce_sum(partials)
        return y + self.bias if self.bias is not None else y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_shards(list(torch.split(x, self.in_per_rank, dim=-1)))

    @classmethod
    def from_dense(cls, dense: Linear, comm: CommBackend) -> "RowParallelLinear":
        out_f, in_f = dense.weight.shape
        layer = cls(in_f, out_f, comm, dense.bias is not None, dense.weight.dtype)
        n = layer.in_per_rank
        with torch.no_grad():
            for r in range(layer.world):
                layer.weight_shards[r].copy_(dense.weight[:, r * n:(r + 1) * n])
            if dense.bias is not None:
                layer.bias.copy_(dense.bias)
        return layer
