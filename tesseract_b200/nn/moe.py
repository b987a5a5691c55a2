"""Mixture-of-experts SwiGLU feed-forward.

Semantics of the reference (src/nn/MoEFeedForward.cpp:27-98,140-146,192-291): router ``gate`` =
Linear(d_model, E) without bias; probs = softmax(router logits); top-k by value descending, index ascending;
gates = the selected probabilities renormalised to sum 1; output = sum over the selected experts of
gate * expert(x), accumulated in ascending expert order; ``aux_loss`` = E * sum_e mean(mask_e) * mean(probs_e)
(Switch load-balancing loss) is stored on the module after each forward; ``num_experts_per_tok <= 0`` or
``> E`` selects every expert. Parameter names: ``gate.weight``, ``experts.{e}.{gate,up,down}_proj.weight``.

On CUDA bf16 the experts run through the grouped-GEMM path (``ops.moe``): device-side routing, counting
and prefix sum (no host synchronisation in the layer, unlike src/cuda/MoeForward.cu:241-247), one grouped
tcgen05 GEMM per projection over the tokens sorted by expert, and a weighted scatter-add combine.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .modules import FeedForward, Linear, Module, ModuleList


def route_topk(logits: torch.Tensor, k: int):
    """Router: returns (probs [T, E] fp32, top-k expert ids [T, k] sorted by (value desc, index asc),
    renormalised gates [T, k])."""
    if (logits.is_cuda and not torch.is_grad_enabled() and logits.shape[-1] <= 256
            and logits.dtype in (torch.float32, torch.bfloat16, torch.float16)):
        probs, idx, gates, _ = ops.moe.route_native(logits, k)
        return probs, idx, gates
    probs = torch.softmax(logits.float(), dim=-1)
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    idx = order.indices[:, :k]
    val = order.values[:, :k]
    gates = val / val.sum(dim=-1, keepdim=True)
    return probs, idx, gates


class MoEFeedForward(Module):
    def __init__(self, d_model: int, d_ff: int, num_experts: int, num_experts_per_tok: int = 2,
                 dtype=torch.float32, device=None):
        super().__init__()
        if d_model <= 0 or d_ff <= 0:
            raise ValueError("MoEFeedForward: d_model and d_ff must be positive")
        if num_experts < 1:
            raise ValueError("MoEFeedForward: num_experts must be >= 1")
        self.d_model, self.d_ff, self.num_experts = d_model, d_ff, num_experts
        k = num_experts_per_tok
        self.top_k = num_experts if (k <= 0 or k > num_experts) else k
        self.gate = Linear(d_model, num_experts, bias=False, dtype=dtype, device=device)
        self.experts = ModuleList([FeedForward(d_model, d_ff, dtype, device) for _ in range(num_experts)])
        self.aux_loss: Optional[torch.Tensor] = None
        self.ep = None  # an expert-parallel dispatcher may be attached (parallel.expert)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T, E, k = x2.shape[0], self.num_experts, self.top_k
        probs, idx, gates = route_topk(self.gate(x2), k)
        mask = torch.zeros_like(probs).scatter_(1, idx, 1.0)
        self.aux_loss = E * (mask.mean(0) * probs.mean(0)).sum()
        if self.ep is not None:
            out = self.ep.forward(self, x2, idx, gates)
        elif ops.moe.grouped_path_ok(x2, self):
            out = ops.moe.moe_ffn_grouped(x2, idx, gates.to(x2.dtype), self)
        else:
            out = self._sparse_reference(x2, idx, gates)
        return out.view(shape)

    def _sparse_reference(self, x2, idx, gates):
        """Per-expert gather -> FFN -> weighted scatter-add, ascending expert order."""
        out = torch.zeros_like(x2)
        for e in range(self.num_experts):
            hit = (idx == e)
            tok = hit.any(dim=1).nonzero().squeeze(-1)
            if tok.numel() == 0:
                continue
            g = (gates * hit)[tok].sum(dim=1).to(x2.dtype)
            out = out.index_add(0, tok, self.experts[e](x2[tok]) * g[:, None])
        return out

    def forward_dense_reference(self, x: torch.Tensor) -> torch.Tensor:
        """Every expert on every token, weighted by the (sparse) gates: the oracle of the sparse paths."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        probs, idx, gates = route_topk(self.gate(x2), self.top_k)
        dense_gates = torch.zeros_like(probs).scatter_(1, idx, gates)
        out = torch.zeros_like(x2)
        for e in range(self.num_experts):
            out = out + self.experts[e](x2) * dense_gates[:, e:e + 1].to(x2.dtype)
        return out.view(shape)
