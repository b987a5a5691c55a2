"""Build a Trainer for ``world`` ranks: picks the mesh (tensor x data parallel), constructs the model on
the device with the same seed on every replica, and attaches the gradient reducer."""
from __future__ import annotations

import torch

from ..models import LlamaConfig, LlamaModel
from ..training import TrainConfig, Trainer


def build_parallel_trainer(cfg: LlamaConfig, tcfg: TrainConfig, world: int, rank: int, device, mode: str = "auto",
                           seed: int = 0):
    """Returns ``(trainer, plan)``; ``plan`` has ``name`` (e.g. "tp8+sp", "dp4"), ``dp``, ``dp_rank``,
    ``tp``, ``tp_rank`` and ``fused_comm``."""
    if world == 1:
        model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        return Trainer(model, tcfg), {"name": "single", "dp": 1, "dp_rank": 0, "tp": 1, "tp_rank": 0}
    import torch.distributed as dist
    if mode in ("auto", "dp"):
        model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        trainer = Trainer(model, tcfg, dp_group=dist.group.WORLD)
        return trainer, {"name": f"dp{world}", "dp": world, "dp_rank": rank, "tp": 1, "tp_rank": 0,
                         "fused_comm": False}
    raise ValueError(f"unknown parallelism mode {mode!r}")
