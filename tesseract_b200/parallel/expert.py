"""Expert parallelism for ``nn.MoEFeedForward``: the experts of a layer are split over the ranks of a group, every
rank routes its own tokens, sends each (token, expert) row to the rank that owns the expert, runs its local experts
over everything it received (one grouped GEMM pair on CUDA), and the results travel back to be combined with the
router gates.

    ep = ExpertParallel(group, rank, world)
    ep.shard_(moe_layer)            # keep experts [rank * E / world, (rank + 1) * E / world); attaches ep to the layer
    y = moe_layer(x)                # x: this rank's tokens

Both exchanges are all-to-alls with per-rank row counts (``torch.distributed.all_to_all_single``: NCCL on GPUs over
NVLink, gloo on CPU ranks in the tests); they are differentiable (the adjoint of an all-to-all is the all-to-all
with the split lists swapped), so the backward pass sends output gradients to the expert owners and input gradients
back. The per-destination counts are exchanged first (a [world, E_local] integer all-to-all) and read on the host,
because the collective needs host-side split sizes: that is the one host synchronisation per layer and direction.
The reference has no expert parallelism (its MoE runs on one device, src/nn/MoEFeedForward.cpp:209-291); the
semantics to preserve are those of its sparse dispatch: out[t] = sum_r gate[t, r] * expert[idx[t, r]](x[t]).
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops


class _AllToAllRows(torch.autograd.Function):
    """Rows [sum(send), D] -> rows [sum(recv), D]; rank j gets my rows [cumsum(send)[j-1], cumsum(send)[j])."""

    @staticmethod
    def forward(ctx, rows, send: List[int], recv: List[int], group):
        import torch.distributed as dist
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = rows.new_empty((sum(recv),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, dout):
        import torch.distributed as dist
        din = dout.new_empty((sum(ctx.send),) + tuple(dout.shape[1:]))
        dist.all_to_all_single(din, dout.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv,
                               group=ctx.group)
        return din, None, None, None


class ExpertParallel:
    def __init__(self, group, rank: int, world: int):
        self.group, self.rank, self.world = group, rank, world
        self.stats = {"rows_sent": 0, "rows_received": 0}

    # ------------------------------------------------------------------ sharding
    def shard_(self, moe) -> None:
        """Keep only this rank's experts in ``moe.experts`` (global expert ids stay in the router) and attach."""
        from ..nn.modules import ModuleList
        E = moe.num_experts
        if E % self.world:
            raise ValueError(f"ExpertParallel: {E} experts do not divide over {self.world} ranks")
        el = E // self.world
        if len(moe.experts) == E:
            moe.experts = ModuleList([moe.experts[i] for i in range(self.rank * el, (self.rank + 1) * el)])
        elif len(moe.experts) != el:
            raise ValueError("ExpertParallel: the layer holds neither all experts nor this rank's share")
        moe.experts_per_rank = el
        moe.ep = self

    # ------------------------------------------------------------------ forward (called by MoEFeedForward.forward)
    def forward(self, moe, x2: torch.Tensor, idx: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        T, D = x2.shape
        k = idx.shape[1]
        E, W = moe.num_experts, self.world
        el = E // W
        flat_e = idx.reshape(-1)
        # sort my assignments by global expert id: that is also by destination rank, experts ascending inside a rank
        order = torch.sort(flat_e, stable=True).indices
        tok = torch.div(order, k, rounding_mode="floor")
        counts = torch.bincount(flat_e, minlength=E).view(W, el)                 # [dest rank, local expert]
        recv_counts = torch.empty_like(counts)                                   # [source rank, local expert]
        dist.all_to_all_single(recv_counts, counts.contiguous(), group=self.group)
        both = torch.stack([counts, recv_counts]).cpu()                          # the one host read
        send = both[0].sum(1).tolist()
        recv = both[1].sum(1).tolist()
        self.stats["rows_sent"] += int(sum(send))
        self.stats["rows_received"] += int(sum(recv))

        xs = x2.index_select(0, tok)                                             # rows in send order
        got = _AllToAllRows.apply(xs, send, recv, self.group)                    # grouped by source, expert ascending
        # local expert id of every received row
        rc = both[1]
        local_e = torch.repeat_interleave(torch.arange(el).repeat(W), rc.reshape(-1)).to(x2.device)
        ys = self._local_experts(moe, got, local_e, el)
        back = _AllToAllRows.apply(ys, recv, send, self.group)                   # rows in my send order again
        g = gates.reshape(-1).index_select(0, order).to(back.dtype)
        return torch.zeros_like(x2).index_add(0, tok, back * g[:, None])

    def _local_experts(self, moe, rows: torch.Tensor, local_e: torch.Tensor, el: int) -> torch.Tensor:
        if rows.shape[0] == 0:
            # keep the parameters in the graph so that every rank's backward runs the same collectives
            return rows + 0 * sum(p.sum() for p in moe.experts.parameters()).to(rows.dtype)
        if rows.is_cuda and rows.dtype == torch.bfloat16 and moe.d_model % 64 == 0 and moe.d_ff % 64 == 0:
            ones = torch.ones((rows.shape[0], 1), dtype=rows.dtype, device=rows.device)
            return ops.moe.moe_ffn_grouped(rows, local_e.view(-1, 1), ones, _LocalView(moe, el))
        out = torch.zeros_like(rows)
        for e in range(el):
            sel = (local_e == e).nonzero().squeeze(-1)
            if sel.numel():
                out = out.index_add(0, sel, moe.experts[e](rows.index_select(0, sel)))
        return out


class _LocalView:
    """What ``ops.moe.moe_ffn_grouped`` needs to know about a layer, for the local experts only."""

    def __init__(self, moe, el: int):
        self.experts, self.num_experts, self.d_model, self.d_ff = moe.experts, el, moe.d_model, moe.d_ff
