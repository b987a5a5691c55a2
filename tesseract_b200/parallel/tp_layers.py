"""Rank-local tensor-parallel + sequence-parallel building blocks (one process per GPU).

Layout (Megatron sequence parallelism): activations between sub-layers are sharded over the token axis
([T / tp, D] per rank); a column-parallel Linear first all-gathers the tokens and multiplies by its slice of output
features, a row-parallel Linear multiplies its slice of input features and reduce-scatters the partial sums back
to token shards. The two collectives are adjoint: the backward of "all-gather -> GEMM" is "GEMM -> reduce-scatter"
and vice versa, so the same two fused primitives serve both directions.

``TPContext.impl`` selects how the two primitives run:
  * ``"fused"``  -- the single-kernel versions in ``parallel/fused_tp.py`` (GEMM tiles pushed to the owning rank from
                    the epilogue over NVLink peer memory; remote token shards pulled by copy CTAs of the GEMM kernel);
  * ``"nccl"``   -- NCCL collective + GEMM back to back (the unfused baseline; also what CPU/gloo ranks use).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops.gemm import gemm_bf16


@dataclass
class TPContext:
    group: object
    rank: int
    size: int
    impl: str = "nccl"
    fused: object = None      # parallel.fused_tp.FusedTP when impl == "fused"

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        xc = x.contiguous()
        out = torch.empty((xc.shape[0] * self.size,) + tuple(xc.shape[1:]), dtype=xc.dtype, device=xc.device)
        dist.all_gather_into_tensor(out, xc, group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        xc = x.contiguous()
        n = xc.shape[0] // self.size
        if xc.is_cuda:
            out = torch.empty((n,) + tuple(xc.shape[1:]), dtype=xc.dtype, device=xc.device)
            dist.reduce_scatter_tensor(out, xc, group=self.group)
            return out
        full = xc.clone()
        dist.all_reduce(full, group=self.group)
        return full[self.rank * n:(self.rank + 1) * n].clone()

    def all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        dist.all_reduce(x, group=self.group)
        return x


def _mm(a: torch.Tensor, b: torch.Tensor, *, a_mn=False, b_mn=False, out=None, accumulate=False) -> torch.Tensor:
    """op(a) @ op(b)^T through the tcgen05 kernel for CUDA bf16, torch otherwise (same operand conventions)."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        return gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=accumulate)
    A = a.t() if a_mn else a
    Bt = b if b_mn else b.t()
    r = A @ Bt
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r)
        return out
    return r


# Token counts (whole step, all ranks) from which the fused kernels are used; below them the collective + GEMM pair
# wins (measured at TP = 8: the gather kernel loses to NCCL + GEMM at 4096 tokens, the scatter kernel wins from the
# smallest size it can run). Both need whole 128-row tiles per rank.
_FUSED_MIN_TOKENS = {"ag": int(os.environ.get("TESSERACT_TP_FUSED_MIN_AG", "8192")),
                     "rs": int(os.environ.get("TESSERACT_TP_FUSED_MIN_RS", "1024"))}


def _fused_applies(ctx: TPContext, x: torch.Tensor, tokens: int, rows_per_rank: int, kind: str,
                   n_local: int = 0) -> bool:
    ok = (ctx.impl == "fused" and ctx.fused is not None and x.is_cuda and x.dtype == torch.bfloat16
          and rows_per_rank % 128 == 0 and tokens >= _FUSED_MIN_TOKENS[kind])
    # A gather whose product has few columns per rank has little arithmetic to hide the pushes behind: measured at
    # TP = 8 with 512 columns per rank, 16384 tokens, the fused kernel takes 0.37 ms against 0.27 ms for NCCL + GEMM,
    # while 768 columns at 32768 tokens and 1792 columns from 8192 tokens win. A threshold of 0 (benchmarks) lifts
    # this rule too.
    if ok and kind == "ag" and _FUSED_MIN_TOKENS["ag"] > 0 and 0 < n_local < 1024 and tokens < 32768:
        ok = False
    return ok


def ag_matmul(ctx: TPContext, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False, keep: bool = True,
              sync_keep: bool = True):
    """(all-gather rows of x_local) @ op(w)^T. Returns (y [T, N], x_full [T, K]). ``keep=False`` allows x_full to
    be a transient buffer that is only valid until the next gathered matmul. With ``sync_keep=False`` the fused
    path may still be filling x_full on a side stream when this returns; the caller then calls
    ``ctx.fused.wait_keep()`` before it reads x_full."""
    n_local = w.shape[1] if b_mn else w.shape[0]
    if _fused_applies(ctx, x_local, x_local.shape[0] * ctx.size, x_local.shape[0], "ag", n_local):
        out = ctx.fused.ag_gemm(x_local, w, b_mn=b_mn, keep=keep)
        if sync_keep:
            ctx.fused.wait_keep()
        return out
    x_full = ctx.all_gather_rows(x_local)
    return _mm(x_full, w, b_mn=b_mn), x_full


def matmul_rs(ctx: TPContext, x: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
    """reduce-scatter over ranks of x @ op(w)^T along rows. Returns y_local [T / tp, N]."""
    if _fused_applies(ctx, x, x.shape[0], x.shape[0] // ctx.size, "rs"):
        return ctx.fused.gemm_rs(x, w, b_mn=b_mn)
    return ctx.reduce_scatter_rows(_mm(x, w, b_mn=b_mn))


class ColumnParallelSPFn(torch.autograd.Function):
    """y [T, N_local] = all_gather(x_local) @ W_local^T; W_local is [N_local, K]."""

    @staticmethod
    def forward(ctx, x_local, w, wgrad_buf, tp: TPContext):
        need_bwd = any(ctx.needs_input_grad[:2])
        # without a backward pass (evaluation under no_grad) the gathered rows are not copied out at all
        y, x_full = ag_matmul(tp, x_local, w, keep=need_bwd, sync_keep=False)
        if not need_bwd:
            return y
        ctx.save_for_backward(x_full, w)   # the gathered activations are kept for the weight gradient
        ctx.tp, ctx.wgrad_buf = tp, wgrad_buf
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx_local = matmul_rs(tp, dy, w, b_mn=True)                      # (dY @ W) reduce-scattered to token shards
        if tp.fused is not None and x_full.is_cuda:
            tp.fused.wait_keep()                                        # x_full may still be arriving on a side stream
        buf = ctx.wgrad_buf
        dw = None
        if buf is not None:
            _mm(dy, x_full, a_mn=True, b_mn=True, out=buf, accumulate=True)
        else:
            dw = _mm(dy, x_full, a_mn=True, b_mn=True).to(w.dtype)
        return dx_local, dw, None, None


class RowParallelSPFn(torch.autograd.Function):
    """y_local [T / tp, N] = reduce_scatter(x [T, K_local] @ W_local^T); W_local is [N, K_local]."""

    @staticmethod
    def forward(ctx, x, w, wgrad_buf, tp: TPContext):
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.wgrad_buf = tp, wgrad_buf
        return matmul_rs(tp, x.contiguous(), w)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dx, dy_full = ag_matmul(tp, dy_local.contiguous(), w, b_mn=True, keep=False)  # all_gather(dY) @ W
        buf = ctx.wgrad_buf
        dw = None
        if buf is not None:
            _mm(dy_full, x, a_mn=True, b_mn=True, out=buf, accumulate=True)
        else:
            dw = _mm(dy_full, x, a_mn=True, b_mn=True).to(w.dtype)
        return dx, dw, None, None


def column_parallel_sp(x_local, w, tp: TPContext, wgrad_buf: Optional[torch.Tensor] = None):
    return ColumnParallelSPFn.apply(x_local, w, wgrad_buf, tp)


def row_parallel_sp(x, w, tp: TPContext, wgrad_buf: Optional[torch.Tensor] = None):
    return RowParallelSPFn.apply(x, w, wgrad_buf, tp)


class VocabParallelCEFn(torch.autograd.Function):
    """Mean cross-entropy with the lm_head weight sharded over the vocabulary and the hidden states sharded
    over tokens: gathers the hidden states, forms this rank's slice of the logits chunk by chunk, merges the
    per-row (max, sum-exp, target-logit) statistics across ranks (one small all-gather per chunk), writes the logits
    gradient in place, and returns the hidden-state gradient reduce-scattered back to token shards.
    Gradients are formed in the forward pass (for an upstream gradient of ``loss_scale``)."""

    @staticmethod
    def forward(ctx, h_local, w, targets, wgrad_buf, tp: TPContext, chunk_rows, loss_scale):
        import torch.distributed as dist
        h_full = tp.all_gather_rows(h_local)
        T, D = h_full.shape
        Vl = w.shape[0]
        v0 = tp.rank * Vl
        dh_full = torch.empty_like(h_full)
        loss_sum = torch.zeros((), device=h_full.device, dtype=torch.float32)
        dw_local = None if wgrad_buf is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            hc, tc = h_full[r0:r1], targets[r0:r1]
            logits = _mm(hc, w)
            stats = ops.ce_stats(logits, tc, vocab_start=v0)
            gathered = torch.empty((tp.size * stats.shape[0], 3), device=stats.device, dtype=stats.dtype)
            dist.all_gather_into_tensor(gathered, stats, group=tp.group)
            merged = ops.merge_ce_stats(list(gathered.view(tp.size, -1, 3).unbind(0))).contiguous()
            loss_rows = ops.ce_loss_and_grad_(logits, tc, merged, loss_scale / T, vocab_start=v0)
            loss_sum += loss_rows.sum()
            _mm(logits, w, b_mn=True, out=dh_full[r0:r1])
            tgt = wgrad_buf if wgrad_buf is not None else dw_local
            _mm(logits, hc, a_mn=True, b_mn=True, out=tgt, accumulate=True)
            del logits
        dh_local = tp.reduce_scatter_rows(dh_full)
        ctx.save_for_backward(dh_local)
        ctx.dw_local, ctx.wdtype = dw_local, w.dtype
        return loss_sum / T

    @staticmethod
    def backward(ctx, g):
        (dh_local,) = ctx.saved_tensors
        dw = ctx.dw_local.to(ctx.wdtype) * g if ctx.dw_local is not None else None
        return dh_local * g.to(dh_local.dtype), dw, None, None, None, None, None
