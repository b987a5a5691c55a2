"""Expert-parallel mixture-of-experts Llama: the experts of every layer are split over the ranks of one group, and
everything else (embedding, attention, norms, routers, head) is replicated, with every rank working on its own
sequences. One MoE layer call sends each (token, expert) row to the rank that owns the expert and brings the result
back (``parallel.expert``: device-side exchange over peer memory, or NCCL all-to-all); the gradients of the replicated
parameters are summed over the ranks after the backward pass by the two-shot peer-memory all-reduce
(``csrc/allreduce_twoshot.cu``) on a flat gradient buffer that lives in symmetric memory. Expert gradients are complete
on their owner: every row that used an expert was multiplied, forward and backward, on that rank.

    ep = EPMoELlama(cfg, group, rank, world, device, max_tokens=4096)
    ep.zero_grad()
    for tokens, targets in micro_batches:                 # this rank's sequences
        loss = ep.forward_backward(tokens, targets, scale=1.0 / total_micro_batches)
    ep.reduce_replicated_grads()                          # sum over ranks
    logits = ep.decode_step(next_tokens, caches)

The reference's MoE runs on one device (src/nn/MoEFeedForward.cpp:209-291 for the sparse dispatch whose semantics are
kept; src/cuda/MoeForward.cu:188-298 for its fused inference chain); it has no expert parallelism.
"""
from __future__ import annotations

import dataclasses
import torch

from ..models import LlamaConfig, LlamaModel


class EPMoELlama:
    def __init__(self, cfg: LlamaConfig, group, rank: int, world: int, device, max_tokens: int,
                 exchange: str = "fused", capacity_factor: float = 2.0, init_std: float = 0.02, seed: int = 0):
        """``cfg.num_experts`` experts per layer, ``cfg.num_experts // world`` of them on this rank. ``max_tokens``
        bounds the tokens of one forward call on a rank (it sizes the exchange buffers). ``exchange``: "fused"
        (device-side pushes, CUDA ranks of one node) or "nccl" (all-to-all collectives; also gloo on CPU ranks)."""
        if cfg.num_experts < 1:
            raise ValueError("EPMoELlama: the configuration has no experts")
        if cfg.num_experts % world:
            raise ValueError(f"EPMoELlama: {cfg.num_experts} experts do not divide over {world} ranks")
        self.cfg, self.group, self.rank, self.world = cfg, group, rank, world
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        el = E // world
        # only this rank's experts are ever allocated (a full 32-layer 8 x 14336 model is 90 GB in bf16)
        local_cfg = dataclasses.replace(cfg, num_experts=el, num_experts_per_tok=k if 0 < k <= el else 0)
        self.model = LlamaModel(local_cfg, device=device, init_std=init_std, seed=seed)
        self.model.config = cfg
        self.ep = None
        if world > 1:
            from ..nn.modules import Linear
            from .expert import ExpertParallel, FusedExpertParallel
            if exchange == "fused" and self.device.type == "cuda":
                self.ep = FusedExpertParallel(group, rank, world, self.device, cfg.hidden_size, E, k if 0 < k <= E else E,
                                              max_tokens=max_tokens, capacity_factor=capacity_factor)
            else:
                self.ep = ExpertParallel(group, rank, world)
            gen = torch.Generator(device=self.device).manual_seed(seed + 1000003)   # same router on every rank
            for blk in self.model.layers:
                moe = blk.ffn
                moe.gate = Linear(cfg.hidden_size, E, bias=False, dtype=cfg.dtype, device=device)
                with torch.no_grad():
                    moe.gate.weight.normal_(0.0, init_std, generator=gen)
                moe.num_experts = E
                moe.top_k = E if (k <= 0 or k > E) else k
                self.ep.shard_(moe)
        self.exchange = "local" if world == 1 else ("fused" if type(self.ep).__name__ == "FusedExpertParallel" else "nccl")
        expert_ids = {id(p) for blk in self.model.layers for p in blk.ffn.experts.parameters()}
        self.expert_params = [p for p in self.model.parameters() if id(p) in expert_ids]
        self.replicated_params = [p for p in self.model.parameters() if id(p) not in expert_ids]
        # replicated parameters: one flat gradient buffer (peer-mapped when the ranks are CUDA devices of one node)
        self._symm = self._reducer = None
        grad_alloc = holder = None
        if world > 1 and self.device.type == "cuda":
            from .factory import _symm_grad_alloc
            grad_alloc, holder = _symm_grad_alloc(group, self.device)
        from ..optim import ParamArena
        self.arena = ParamArena(self.replicated_params, grad_alloc=grad_alloc)
        if grad_alloc is not None:
            from .fused_tp import SymmGradAllReduce
            self._symm = holder["symm"]
            self._reducer = SymmGradAllReduce(self._symm)

    def load_full_state_dict(self, state: dict) -> None:
        """Loads the weights of an unsharded model (``LlamaModel.state_dict()`` names, every expert present): the
        replicated tensors as they are, of ``layers.{i}.ffn.experts.{e}.*`` only this rank's experts."""
        el = self.cfg.num_experts // self.world
        own = dict(self.model.named_parameters())
        with torch.no_grad():
            for name, value in state.items():
                parts = name.split(".")
                if "experts" in parts:
                    at = parts.index("experts")
                    e = int(parts[at + 1])
                    if not (self.rank * el <= e < (self.rank + 1) * el):
                        continue
                    parts[at + 1] = str(e - self.rank * el)
                    name = ".".join(parts)
                if name in own:
                    own[name].copy_(value.to(own[name].dtype))

    # ------------------------------------------------------------------ training
    def zero_grad(self) -> None:
        self.arena.zero_grad()
        for p in self.expert_params:
            p.grad = None

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """Loss of this rank's ``tokens`` [B, S] (every rank calls this the same number of times per step: each MoE
        layer call is a collective). ``scale`` multiplies the gradients, not the returned loss."""
        loss = self.model.loss(tokens, targets, loss_scale=scale)      # the scale is folded into the fused head gradients
        loss.backward()
        return loss.detach()

    def reduce_replicated_grads(self, average: bool = False) -> None:
        """Sums the gradients of the replicated parameters over the ranks, in place. With ``scale`` = 1 / (micro-batches
        of ALL ranks) in ``forward_backward`` the sum is the gradient of the global mean loss, on the same footing as
        the expert gradients (which already hold every rank's rows). ``average`` divides by the rank count as well."""
        self.arena.fold_autograd_grads()
        if self.world == 1:
            return
        s = (1.0 / self.world) if average else 1.0
        if self._reducer is not None:
            self._reducer.all_reduce_(0, self.arena.numel, self.arena.grad.dtype, scale=s)   # 128-element aligned arena
        else:
            import torch.distributed as dist
            if average:
                self.arena.grad.div_(self.world)
            dist.all_reduce(self.arena.grad, group=self.group)

    # ------------------------------------------------------------------ inference
    def make_kv_caches(self, batch: int, max_len: int) -> list:
        return self.model.make_kv_caches(batch, max_len)

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, caches: list) -> torch.Tensor:
        """tokens [B, S_new] of this rank's sequences through its caches -> logits [B, S_new, V]; a collective (the
        MoE layers exchange rows), so every rank calls it together, with any B >= 1 of its own."""
        return self.model.forward_step(tokens, caches)

    def param_bytes(self) -> dict:
        size = lambda ps: sum(p.numel() * p.element_size() for p in ps)   # noqa: E731
        return {"experts_local": size(self.expert_params), "replicated": size(self.replicated_params)}

    def close(self) -> None:
        for obj in (self._reducer, self._symm, self.ep if hasattr(self.ep, "close") else None):
            if obj is not None:
                obj.close()
        self._reducer = self._symm = None
