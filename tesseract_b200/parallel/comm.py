"""Communication backends.

``CommBackend`` keeps the reference's shard-list signature (include/tesseract/distributed/CommBackend.hpp:28-45):
``all_reduce_sum(shards)`` and ``all_gather(shards, dim)`` over a list holding every rank's tensor in one address
space. ``SimCommBackend`` implements it in-process (left-fold add, cat: src/distributed/CommBackend.cpp:9-40), with
autograd flowing through, and is what the CPU tests use to check tensor-parallel layers against dense ones.

``NcclCommBackend`` is the rank-local counterpart of the reference's NCCL wrapper
(src/distributed/NcclCommBackend.cpp:84-203): one process per GPU, all-reduce / all-gather / barrier on the tensor's
current stream. Unlike the reference it does not synchronise the host after each collective, it is asynchronous on
the stream, and it also offers reduce-scatter and all-to-all. It runs over any torch.distributed group, so the same
code is exercised with ``gloo`` CPU ranks in the tests.
"""
from __future__ import annotations

from typing import List, Optional

import torch


class CommBackend:
    def world_size(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def all_reduce_sum(self, shards: List[torch.Tensor]) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def all_gather(self, shards: List[torch.Tensor], dim: int) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError


class SimCommBackend(CommBackend):
    def __init__(self, world_size: int):
        if world_size < 1:
            raise ValueError("SimCommBackend: world_size must be >= 1")
        self._world = world_size

    def world_size(self) -> int:
        return self._world

    def _check(self, shards):
        if len(shards) != self._world:
            raise ValueError(f"expected {self._world} shards, got {len(shards)}")

    def all_reduce_sum(self, shards):
        self._check(shards)
        out = shards[0]
        for s in shards[1:]:
            out = out + s
        return out

    def all_gather(self, shards, dim):
        self._check(shards)
        return torch.cat(list(shards), dim=dim)

    def reduce_scatter(self, shards, dim):
        """Every rank's full-size partial in, list of per-rank slices of the sum out."""
        total = self.all_reduce_sum(shards)
        return list(torch.chunk(total, self._world, dim=dim))


class NcclCommBackend:
    """Rank-local collectives over a torch.distributed process group (NCCL on GPUs, gloo on CPU ranks)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("NcclCommBackend: torch.distributed is not initialised")
        self.group = group if group is not None else dist.group.WORLD
        self._dist = dist

    def world_size(self) -> int:
        return self._dist.get_world_size(self.group)

    def rank(self) -> int:
        return self._dist.get_rank(self.group)

    @torch.no_grad()
    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        out = t.clone()
        self._dist.all_reduce(out, group=self.group)
        return out

    @torch.no_grad()
    def all_reduce_sum_(self, t: torch.Tensor, async_op: bool = False):
        return self._dist.all_reduce(t, group=self.group, async_op=async_op)

    @torch.no_grad()
    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        w = self.world_size()
        tc = t.contiguous()
        out = torch.empty((w * tc.shape[0],) + tuple(tc.shape[1:]), dtype=tc.dtype, device=tc.device)
        self._dist.all_gather_into_tensor(out, tc, group=self.group)
        d = dim % tc.dim()
        if d == 0:
            return out
        return torch.cat(list(out.view(w, *tc.shape).unbind(0)), dim=d)

    @torch.no_grad()
    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over ranks of ``t`` ([world * n, ...]) scattered along dim 0."""
        w = self.world_size()
        tc = t.contiguous()
        out = torch.empty((tc.shape[0] // w,) + tuple(tc.shape[1:]), dtype=tc.dtype, device=tc.device)
        if tc.is_cuda:
            self._dist.reduce_scatter_tensor(out, tc, group=self.group)
        else:  # gloo has no reduce_scatter: all-reduce then slice
            full = tc.clone()
            self._dist.all_reduce(full, group=self.group)
            n = out.shape[0]
            out.copy_(full[self.rank() * n:(self.rank() + 1) * n])
        return out

    @torch.no_grad()
    def all_to_all(self, t: torch.Tensor, in_splits: Optional[list] = None, out_splits: Optional[list] = None):
        tc = t.contiguous()
        n_out = sum(out_splits) if out_splits is not None else tc.shape[0]
        out = torch.empty((n_out,) + tuple(tc.shape[1:]), dtype=tc.dtype, device=tc.device)
        if tc.is_cuda:
            self._dist.all_to_all_single(out, tc, out_splits, in_splits, group=self.group)
        else:
            w = self.world_size()
            ins = list(tc.split(in_splits if in_splits is not None else [tc.shape[0] // w] * w))
            outs = list(out.split(out_splits if out_splits is not None else [n_out // w] * w))
            reqs = []
            me = self.rank()
            for r in range(w):
                if r == me:
                    outs[r].copy_(ins[r])
                else:
                    reqs.append(self._dist.isend(ins[r].contiguous(), self._dist.get_global_rank(self.group, r), group=self.group))
                    reqs.append(self._dist.irecv(outs[r], self._dist.get_global_rank(self.group, r), group=self.group))
            for q in reqs:
                q.wait()
        return out

    def barrier(self) -> None:
        self._dist.barrier(group=self.group)
