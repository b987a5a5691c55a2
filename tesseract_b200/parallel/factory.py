"""Build a Trainer for ``world`` ranks: picks the mesh (tensor x data parallel), constructs the model on the device
and attaches the gradient reducer.

Modes: ``tp`` (tensor + sequence parallel over ``tp`` ranks, data parallel over the rest), ``dp`` (replicated model,
overlapped gradient all-reduce), ``auto`` = ``tp`` over all ranks, which is the configuration the headline
benchmark names (TP = N with sequence parallelism).
"""
from __future__ import annotations

import os

import torch

from ..models import LlamaConfig, LlamaModel
from ..training import TrainConfig, Trainer
from .data_parallel import GradReducer


def _attach_reducer(model, trainer, group):
    buckets = GradReducer.layer_buckets(model, trainer.arena)
    red = GradReducer(trainer.arena, group, buckets)
    # bucket index of block 0: buckets are sorted by arena offset = registration order; the embedding comes first
    red.block_bucket0 = 1 if len(buckets) > len(model.layers) else 0
    model.grad_reducer = red
    trainer.grad_reducer = red
    trainer.dp_group = None
    if getattr(trainer.cfg, "zero_stage", 0) == 1:
        from .zero import ShardedAdam
        c = trainer.cfg
        trainer.opt = ShardedAdam(trainer.arena, group, lr=c.lr, beta1=c.beta1, beta2=c.beta2, eps=c.eps,
                                  weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm)
    elif getattr(trainer.cfg, "zero_stage", 0) not in (0, 1):
        raise ValueError("zero_stage: 0 (replicated optimizer state) or 1 (sharded Adam moments)")
    return red


def build_parallel_trainer(cfg: LlamaConfig, tcfg: TrainConfig, world: int, rank: int, device, mode: str = "auto",
                           seed: int = 0, tp_size: int = 0):
    """Returns ``(trainer, plan)``; ``plan`` has ``name`` (e.g. "tp8+sp", "dp4"), ``dp``, ``dp_rank``, ``tp``,
    ``tp_rank`` and ``fused_comm``."""
    if world == 1:
        model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        return Trainer(model, tcfg), {"name": "single", "dp": 1, "dp_rank": 0, "tp": 1, "tp_rank": 0,
                                      "fused_comm": False}
    import torch.distributed as dist
    if mode == "dp":
        model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        trainer = Trainer(model, tcfg)
        _attach_reducer(model, trainer, dist.group.WORLD)
        return trainer, {"name": f"dp{world}", "dp": world, "dp_rank": rank, "tp": 1, "tp_rank": 0,
                         "fused_comm": False}
    if mode in ("auto", "tp"):
        from .tp_layers import TPContext
        from .tp_model import TPLlamaModel
        tp = tp_size if tp_size > 0 else world
        if world % tp:
            raise ValueError(f"world size {world} is not a multiple of the tensor-parallel size {tp}")
        dp = world // tp
        tp_rank, dp_rank = rank % tp, rank // tp
        tp_group = dp_group = None
        for d in range(dp):
            g = dist.new_group(list(range(d * tp, (d + 1) * tp)))
            if d == dp_rank:
                tp_group = g
        for t in range(tp):
            g = dist.new_group(list(range(t, world, tp)))
            if t == tp_rank:
                dp_group = g
        impl = os.environ.get("TESSERACT_TP_COMM", "fused")
        ctx = TPContext(tp_group, tp_rank, tp, impl="nccl")
        fused_ok = False
        if impl == "fused" and torch.device(device).type == "cuda":
            try:
                from .fused_tp import FusedTP
                ctx.fused = FusedTP(tp_group, tp_rank, tp, device)
                ctx.impl = "fused"
                fused_ok = True
            except Exception as e:  # the unfused NCCL path is always available
                if rank == 0:
                    print(f"[tesseract_b200] fused TP kernels unavailable ({e}); using NCCL collectives", flush=True)
        model = TPLlamaModel(cfg, ctx, device=device, init_std=0.02, seed=seed)
        trainer = Trainer(model, tcfg)
        if dp > 1:
            _attach_reducer(model, trainer, dp_group)
        name = f"tp{tp}+sp" + (f" x dp{dp}" if dp > 1 else "")
        return trainer, {"name": name, "dp": dp, "dp_rank": dp_rank, "tp": tp, "tp_rank": tp_rank,
                         "fused_comm": fused_ok}
    raise ValueError(f"unknown parallelism mode {mode!r}")
