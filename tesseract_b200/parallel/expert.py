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


# --------------------------------------------------------------------------------------------------------------
# Device-side expert parallelism over peer memory (CUDA, one NVSwitch domain): csrc/moe_ep.cu
class _FusedEPFn(torch.autograd.Function):
    """One MoE layer call with expert parallelism, nothing read back to the host: publish counts -> plan ->
    push rows to the owners -> grouped GEMMs on the owner -> push results back -> weighted combine."""

    @staticmethod
    def forward(ctx, x2, gates, idx32, ep, moe_view, stride, w_gu0, w_dn0, *weights):
        from .._native import check, lib
        from ..ops import moe as M
        from ..ops.fused import swiglu
        T, D = x2.shape
        k = idx32.shape[1]
        E, W, El = ep.num_experts, ep.world, ep.num_experts // ep.world
        dev = x2.device
        s = torch.cuda.current_stream(dev).cuda_stream
        if T * k > ep.ret_rows:
            raise ValueError(f"FusedExpertParallel: {T * k} assignments exceed the return buffer ({ep.ret_rows} rows)")
        counts = torch.bincount(idx32.view(-1), minlength=E).to(torch.int32)
        check(lib().tsb_ep_fill_i32(ep.tags.local_ptr, ep.cap_rows, -1, s), "tsb_ep_fill_i32")
        check(lib().tsb_ep_publish_counts(ep.cnt.ptr_array, counts.data_ptr(), ep.rank, W, E, s), "tsb_ep_publish_counts")
        ep.barrier()                                            # every rank's counts are here; every tag array is reset
        send_base = torch.empty(E, dtype=torch.int32, device=dev)
        offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
        cursor = torch.empty(E, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        check(lib().tsb_ep_plan(ep.cnt.local_ptr, send_base.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), ep.rank, W,
                                E, 128, s), "tsb_ep_plan")
        x2c = x2.contiguous()
        check(lib().tsb_ep_dispatch(x2c.data_ptr(), idx32.data_ptr(), None, ep.recv.ptr_array, ep.tags.ptr_array,
                                    send_base.data_ptr(), cursor.data_ptr(), dest_row.data_ptr(), T * k, k, D, El, ep.rank, W,
                                    1, ep.cap_rows, s), "tsb_ep_dispatch")
        ep.barrier()                                            # every row this rank owns has landed
        tags = ep.tags_view().clone()
        xs = torch.empty((ep.cap_rows, D), dtype=torch.bfloat16, device=dev)
        check(lib().tsb_ep_clean_copy(ep.recv.local_ptr, tags.data_ptr(), xs.data_ptr(), ep.cap_rows,
                                      offsets[El:].data_ptr(), D, s), "tsb_ep_clean_copy")
        h = M.grouped_gemm_rows(xs, w_gu0, stride, offsets, El)
        a = swiglu(h)
        if ep.scatter_epilogue:
            # the return exchange is the epilogue of the down projection: every result row goes from the accumulator
            # straight to the return buffer of the rank it came from (NVLink stores); no local copy of the results
            M.grouped_gemm_rows_scatter(a, w_dn0, stride, offsets, El, tags, ep.ret.ptr_array, W, ep.ret_rows)
        else:
            ys = M.grouped_gemm_rows(a, w_dn0, stride, offsets, El)
            check(lib().tsb_ep_return(ys.data_ptr(), tags.data_ptr(), ep.ret.ptr_array, ep.cap_rows,
                                      offsets[El:].data_ptr(), D, ep.ret_rows, W, s), "tsb_ep_return")
        ep.barrier()                                            # every result row of this rank's tokens is back
        back = ep.ret_view(T * k, D).clone()
        gates32 = gates.float().contiguous()
        out = M.combine_rows(back, ep.identity(T * k), T, k, gates32)
        ctx.save_for_backward(xs, h, a, back, gates32, offsets, tags, dest_row, idx32, w_gu0, w_dn0)
        ctx.ep, ctx.meta = ep, (T, D, El, k, stride, len(weights), gates.dtype)
        ep.calls += 1
        return out

    @staticmethod
    def backward(ctx, dout):
        from .._native import check, lib
        from ..ops import moe as M
        xs, h, a, back, gates32, offsets, tags, dest_row, idx32, w_gu0, w_dn0 = ctx.saved_tensors
        ep = ctx.ep
        T, D, El, k, stride, nw, gdtype = ctx.meta
        dev = dout.device
        s = torch.cuda.current_stream(dev).cuda_stream
        dout = dout.contiguous()
        ident = ep.identity(T * k)
        dgate = torch.empty(T * k, dtype=torch.float32, device=dev)
        check(lib().tsb_moe_gate_grad(dout.data_ptr(), back.data_ptr(), ident.data_ptr(), dgate.data_ptr(), T, D, k, s),
              "tsb_moe_gate_grad")
        # gate-weighted output gradients travel to the owners along the rows of the forward pass
        check(lib().tsb_ep_dispatch(dout.data_ptr(), idx32.data_ptr(), gates32.data_ptr(), ep.recv.ptr_array,
                                    ep.tags.ptr_array, None, None, dest_row.data_ptr(), T * k, k, D, El, ep.rank, ep.world,
                                    0, ep.cap_rows, s), "tsb_ep_dispatch")
        ep.barrier()
        dys = torch.empty_like(xs)
        check(lib().tsb_ep_clean_copy(ep.recv.local_ptr, tags.data_ptr(), dys.data_ptr(), ep.cap_rows,
                                      offsets[El:].data_ptr(), D, s), "tsb_ep_clean_copy")
        dxs, dw = M.grouped_experts_backward(xs, h, a, dys, offsets, El, stride, w_gu0, w_dn0)
        check(lib().tsb_ep_return(dxs.data_ptr(), tags.data_ptr(), ep.ret.ptr_array, ep.cap_rows, offsets[El:].data_ptr(),
                                  D, ep.ret_rows, ep.world, s), "tsb_ep_return")
        ep.barrier()
        dx = M.combine_rows(ep.ret_view(T * k, D), ident, T, k)
        # no barrier needed here: a peer writes this return buffer again only after two barriers of a later call,
        # and this rank enters the first of them after the kernel above
        grads = M.split_expert_grads(dw, El, stride, h.shape[1] // 2, D) if nw else []
        return (dx, dgate.view(T, k).to(gdtype), None, None, None, None, None, None, *grads)


class FusedExpertParallel(ExpertParallel):
    """Expert parallelism whose token exchange runs on the device over NVLink peer memory (``csrc/moe_ep.cu``):
    counts, row plan, dispatch and return are kernels, synchronised by the flag-barrier kernel; the host never reads
    a count and NCCL is not involved. ``max_tokens`` bounds the tokens of one call on a rank; the receive buffer
    holds ``capacity_factor`` times a rank's fair share of rows (a call that exceeds it sets the status word and
    drops the overflow instead of writing out of bounds)."""

    def __init__(self, group, rank: int, world: int, device, d_model: int, num_experts: int, top_k: int,
                 max_tokens: int, capacity_factor: float = 2.0):
        super().__init__(group, rank, world)
        from .fused_tp import SymmetricMemory
        if world > 8 or num_experts % world or num_experts > 256:
            raise ValueError("FusedExpertParallel: at most 8 ranks, at most 256 experts, experts divisible by ranks")
        self.device = torch.device(device)
        self.num_experts, self.top_k, self.d_model = num_experts, top_k, d_model
        el = num_experts // world
        self.ret_rows = max_tokens * top_k
        want = int(capacity_factor * max_tokens * top_k) + el * 127
        self.cap_rows = (min(want, world * max_tokens * top_k + el * 127) + 127) // 128 * 128
        self.recv = SymmetricMemory(group, rank, world, self.cap_rows * d_model * 2, device)
        self.tags = SymmetricMemory(group, rank, world, self.cap_rows * 4, device)
        self.ret = SymmetricMemory(group, rank, world, self.ret_rows * d_model * 2, device)
        self.cnt = SymmetricMemory(group, rank, world, world * num_experts * 4, device)
        self.pads = SymmetricMemory(group, rank, world, 256, device)
        self.epoch = 0
        self.calls = 0
        import os
        self.scatter_epilogue = os.environ.get("TESSERACT_EP_SCATTER_EPILOGUE", "1") == "1"
        self._ident = torch.arange(self.ret_rows, dtype=torch.int32, device=self.device)

    def barrier(self) -> None:
        from .._native import check, lib
        self.epoch += 1
        check(lib().tsb_symm_barrier(self.pads.ptr_array, self.rank, self.world, self.epoch,
                                     torch.cuda.current_stream(self.device).cuda_stream), "tsb_symm_barrier")

    def identity(self, n: int) -> torch.Tensor:
        return self._ident[:n]

    def tags_view(self) -> torch.Tensor:
        return self.tags.local[:self.cap_rows * 4].view(torch.int32)

    def ret_view(self, rows: int, D: int) -> torch.Tensor:
        return self.ret.local[:rows * D * 2].view(torch.bfloat16).view(rows, D)

    def forward(self, moe, x2: torch.Tensor, idx: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
        if not (x2.is_cuda and x2.dtype == torch.bfloat16 and moe.d_model % 64 == 0 and moe.d_ff % 64 == 0):
            return super().forward(moe, x2, idx, gates)
        view = _LocalView(moe, len(moe.experts))
        ws, stride, w_gu0, w_dn0 = ops.moe.expert_weight_stack(view)
        return _FusedEPFn.apply(x2, gates, idx.to(torch.int32).contiguous(), self, view, stride, w_gu0, w_dn0, *ws)

    def close(self) -> None:
        for m in (self.recv, self.tags, self.ret, self.cnt, self.pads):
            m.close()
