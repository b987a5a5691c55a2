"""MoE expert compute on CUDA: device-side routing bookkeeping and grouped tcgen05 GEMMs.

``moe_ffn_grouped`` sorts the (token, expert) assignments by expert entirely on the device, gathers the
token rows once, runs gate_up / down as grouped GEMMs (one GEMM launch per expert over its contiguous row
block, offsets read on the device side of the launch through pre-sized padding, see below) and combines the
weighted expert outputs with a scatter-add. The routing math itself (softmax, top-k, renormalisation) stays
in ``nn.moe.route_topk`` so that every path shares it.
"""
from __future__ import annotations

import torch

from .. import _native
from .._native import check, lib, stream_ptr
from .gemm import gemm_bf16, linear
from .fused import swiglu

P, I = _native.P, _native.I
_native.register_signatures({
    "tsb_moe_route": [P, P, P, P, P, I, I, I, I, P],
    "tsb_moe_sort": [P, P, P, P, P, P, I, I, I, P],
})


def route_native(logits: torch.Tensor, k: int, want_probs: bool = True):
    """Device router (no autograd): returns (probs [T, E] fp32 or None, idx int64 [T, k], gates fp32 [T, k],
    counts int32 [E])."""
    T, E = logits.shape
    lg = logits.contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=lg.device)
    gates = torch.empty((T, k), dtype=torch.float32, device=lg.device)
    probs = torch.empty((T, E), dtype=torch.float32, device=lg.device) if want_probs else None
    counts = torch.zeros(E, dtype=torch.int32, device=lg.device)
    check(lib().tsb_moe_route(lg.data_ptr(), idx.data_ptr(), gates.data_ptr(),
                              probs.data_ptr() if probs is not None else None, counts.data_ptr(), T, E, k,
                              _native.dtype_code(lg.dtype), stream_ptr(lg.device)), "tsb_moe_route")
    return probs, idx.long(), gates, counts


def sort_by_expert(idx: torch.Tensor, counts: torch.Tensor):
    """Expert-sorted permutation of the T * k assignments, computed on the device.
    Returns (offsets int32 [E + 1], sorted_pos int32 [T * k], sorted_token int32 [T * k])."""
    T, k = idx.shape
    E = counts.shape[0]
    idx32 = idx.to(torch.int32).contiguous()
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    cursor = torch.empty(E, dtype=torch.int32, device=idx.device)
    pos = torch.empty(T * k, dtype=torch.int32, device=idx.device)
    tok = torch.empty(T * k, dtype=torch.int32, device=idx.device)
    check(lib().tsb_moe_sort(idx32.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), pos.data_ptr(),
                             tok.data_ptr(), T, E, k, stream_ptr(idx.device)), "tsb_moe_sort")
    _native.add_launches(1)
    return offsets, pos, tok


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
