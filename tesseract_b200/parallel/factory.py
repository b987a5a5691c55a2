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


def _symm_grad_alloc(group, device):
    """Returns ``(grad_alloc, holder)`` for ``Trainer``: the gradient arena goes into peer-mapped memory of the
    data-parallel group so that the all-reduce kernel can work on it in place; ``holder["symm"]`` is the
    ``SymmetricMemory`` afterwards. ``(None, None)`` when the NCCL path is selected or the ranks are not CUDA."""
    if torch.device(device).type != "cuda" or os.environ.get("TESSERACT_DP_COMM", "symm") != "symm":
        return None, None
    import torch.distributed as dist
    from .fused_tp import SymmetricMemory
    if dist.get_world_size(group) > 8:
        return None, None
    holder = {}

    def alloc(numel, dtype, dev):
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        sm = SymmetricMemory(group, dist.get_rank(group), dist.get_world_size(group), (nbytes + 255) // 256 * 256, dev)
        holder["symm"] = sm
        return sm.local[:nbytes].view(dtype)

    return alloc, holder


def _resources(trainer, fused, holder):
    """Objects that own peer-mapped device memory and must be ``close()``d (collectively, after a device synchronise
    and a barrier) when a trainer is torn down before the process ends."""
    out = []
    red = getattr(trainer, "grad_reducer", None)
    if red is not None and getattr(red, "symm", None) is not None:
        out.append(red.symm)
    if holder and "symm" in holder:
        out.append(holder["symm"])
    if fused is not None:
        out.append(fused)
    return out


def _attach_reducer(model, trainer, group, holder=None):
    buckets = GradReducer.layer_buckets(model, trainer.arena)
    symm = None
    if holder and "symm" in holder:
        from .fused_tp import SymmGradAllReduce
        symm = SymmGradAllReduce(holder["symm"])
    red = GradReducer(trainer.arena, group, buckets, symm=symm)
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
                           seed: int = 0, tp_size: int = 0, module_init: bool = False):
    """Returns ``(trainer, plan)``; ``plan`` has ``name`` (e.g. "tp8+sp", "dp4"), ``dp``, ``dp_rank``, ``tp``,
    ``tp_rank``, ``fused_comm``, ``dp_comm`` and ``resources`` (see ``_resources``). Weights are N(0, 0.02) from
    ``seed``; ``module_init`` (single process only) keeps the modules' own initialisers instead -- Linear
    U(+-1/sqrt(in)), Embedding N(0, 1), the reference's rules (src/nn/Linear.cpp:19-60, src/nn/Embedding.cpp:64-85)."""
    if world == 1:
        if module_init:
            torch.manual_seed(seed)
            model = LlamaModel(cfg, device=device)
        else:
            model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        return Trainer(model, tcfg), {"name": "single", "dp": 1, "dp_rank": 0, "tp": 1, "tp_rank": 0,
                                      "fused_comm": False, "dp_comm": None, "resources": []}
    import torch.distributed as dist
    if mode == "dp":
        model = LlamaModel(cfg, device=device, init_std=0.02, seed=seed)
        grad_alloc, holder = _symm_grad_alloc(dist.group.WORLD, device)
        trainer = Trainer(model, tcfg, grad_alloc=grad_alloc)
        _attach_reducer(model, trainer, dist.group.WORLD, holder)
        return trainer, {"name": f"dp{world}", "dp": world, "dp_rank": rank, "tp": 1, "tp_rank": 0,
                         "fused_comm": False, "dp_comm": "symm-twoshot" if holder else "nccl",
                         "resources": _resources(trainer, None, holder)}
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
        grad_alloc, holder = _symm_grad_alloc(dp_group, device) if dp > 1 else (None, None)
        trainer = Trainer(model, tcfg, grad_alloc=grad_alloc)
        if dp > 1:
            _attach_reducer(model, trainer, dp_group, holder)
        name = f"tp{tp}+sp" + (f" x dp{dp}" if dp > 1 else "")
        return trainer, {"name": name, "dp": dp, "dp_rank": dp_rank, "tp": tp, "tp_rank": tp_rank,
                         "fused_comm": fused_ok, "dp_comm": ("symm-twoshot" if holder else "nccl") if dp > 1 else None,
                         "resources": _resources(trainer, ctx.fused, holder)}
    raise ValueError(f"unknown parallelism mode {mode!r}")
