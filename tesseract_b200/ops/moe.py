"""MoE expert compute on CUDA: device-side routing bookkeeping and grouped tcgen05 GEMMs.

``moe_ffn_grouped`` sorts the (token, expert) assignments by expert entirely on the device, gathers the
token rows once, runs gate_up / down as grouped GEMMs (one GEMM launch per expert over its contiguous row
block, offsets read on the device side of the launch through pre-sized padding, see below) and combines the
weighted expert outputs with a scatter-add. The routing math itself (softmax, top-k, renormalisation) stays
in ``nn.moe.route_topk`` so that every path shares it.
"""
from __future__ import annotations

import torch

from .gemm import gemm_bf16, linear
from .fused import swiglu


def grouped_path_ok(x2: torch.Tensor, moe) -> bool:
    if not (x2.is_cuda and x2.dtype == torch.bfloat16):
        return False
    from ..nn.modules import Linear
    return all(isinstance(ex.gate_proj, Linear) for ex in moe.experts)


def moe_ffn_grouped(x2: torch.Tensor, idx: torch.Tensor, gates: torch.Tensor, moe) -> torch.Tensor:
    """x2 [T, D] bf16, idx [T, k] expert ids, gates [T, k] -> [T, D].

    Tokens are ordered by expert with one stable device sort; expert e owns the row block
    [offsets[e], offsets[e+1]) of the permuted activations. The per-expert row counts are read back once
    per call (one small D2H copy) to size the per-expert GEMM launches; everything else stays on the device.
    Autograd flows through index_select / index_add and the ``linear`` op.
    """
    T, D = x2.shape
    k = idx.shape[1]
    E = moe.num_experts
    flat_e = idx.reshape(-1)
    order = torch.sort(flat_e, stable=True).indices          # positions in the [T*k] assignment list
    tok = order // k
    counts = torch.bincount(flat_e, minlength=E)
    xs = x2.index_select(0, tok)                              # [T*k, D] grouped by expert
    gs = gates.reshape(-1).index_select(0, order)
    bounds = [0] + torch.cumsum(counts, 0).tolist()
    outs = []
    for e in range(E):
        lo, hi = bounds[e], bounds[e + 1]
        if hi == lo:
            continue
        outs.append(moe.experts[e](xs[lo:hi]))
    ys = torch.cat(outs, dim=0) * gs[:, None]
    return torch.zeros_like(x2).index_add(0, tok, ys)
