"""Optimizer-state sharding over the data-parallel group (ZeRO stage 1): every rank keeps Adam's fp32 moments for
one contiguous slice of the parameter arena only, updates that slice, and the updated slices are exchanged so that
all replicas hold the same parameters again. Gradients stay all-reduced (overlapped with backward by
``GradReducer``), so each rank sees the full gradient and clips by the same global norm.

Per-rank optimizer memory drops from 8 bytes per parameter to 8 / dp: an 8B-parameter model on 8 data-parallel GPUs
keeps 8 GB of moments per GPU instead of 64 GB. The reference has neither data parallelism nor optimizer sharding.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from ..optim.optimizers import Adam, check, dtype_code, lib, stream_ptr

_SHARD_ALIGN = 64      # elements: keeps every slice start 16-byte aligned for the vectorised update kernel


def shard_ranges(numel: int, world: int) -> List[Tuple[int, int]]:
    """``world`` contiguous [begin, end) slices that tile [0, numel); starts are multiples of 64 elements."""
    per = (numel + world - 1) // world
    per = (per + _SHARD_ALIGN - 1) // _SHARD_ALIGN * _SHARD_ALIGN
    return [(min(numel, r * per), min(numel, (r + 1) * per)) for r in range(world)]


class ShardedAdam(Adam):
    def __init__(self, arena, group, **kw):
        import torch.distributed as dist
        super().__init__(arena, **kw)
        if self.arena is None:
            raise ValueError("ShardedAdam needs a ParamArena (one flat parameter buffer)")
        self._dist, self.group = dist, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ranges = shard_ranges(arena.numel, self.world)
        self.begin, self.end = self.ranges[self.rank]
        self._owners = [dist.get_global_rank(group, r) if group is not None else r for r in range(self.world)]

    def state_bytes(self) -> int:
        return 2 * 4 * (self.end - self.begin)

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["shard"] = (self.begin, self.end)
        return sd

    def load_state_dict(self, sd: dict) -> None:
        if tuple(sd.get("shard", (self.begin, self.end))) != (self.begin, self.end):
            raise ValueError("ShardedAdam: the checkpoint holds a different shard than this rank owns")
        super().load_state_dict(sd)

    def _step_arena(self, bc1, bc2):
        a = self.arena
        b0, b1 = self.begin, self.end
        n = b1 - b0
        if self._flat_state is None:
            self._flat_state = (torch.zeros(n, device=a.device, dtype=torch.float32),
                                torch.zeros(n, device=a.device, dtype=torch.float32))
        m, v = self._flat_state
        if n > 0 and not a.flat.is_cuda:
            gf = a.grad.float()
            if self.max_grad_norm > 0:
                gf = gf * min(1.0, self.max_grad_norm / (gf.norm().item() + 1e-6))
            gf = gf[b0:b1]
            m.mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
            v.mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
            w = a.master[b0:b1] if a.master is not None else a.flat[b0:b1].float()
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            if self.weight_decay:
                upd = upd + self.weight_decay * w
            w = w - self.lr * upd
            if a.master is not None:
                a.master[b0:b1].copy_(w)
            a.flat[b0:b1].copy_(w.to(a.dtype))
        elif n > 0:
            gscale = self._gscale([a.grad], a.device)          # global norm: the gradient is complete on every rank
            master = a.master[b0:b1] if a.master is not None else None
            check(lib().tsb_adam_flat(a.flat[b0:b1].data_ptr(), a.grad[b0:b1].data_ptr(), m.data_ptr(), v.data_ptr(),
                                      master.data_ptr() if master is not None else None, n, self.lr, self.beta1,
                                      self.beta2, self.eps, bc1, bc2, self.weight_decay,
                                      gscale.data_ptr() if gscale is not None else None, dtype_code(a.dtype),
                                      dtype_code(a.grad_dtype), stream_ptr(a.device)), "tsb_adam_flat")
        # every owner publishes its updated slice; the slices differ in length, so one broadcast each
        works = []
        for r, (s0, s1) in enumerate(self.ranges):
            if s1 > s0:
                works.append(self._dist.broadcast(a.flat[s0:s1], src=self._owners[r], group=self.group, async_op=True))
        for w_ in works:
            w_.wait()
