"""Data-parallel gradient reduction overlapped with the backward pass.

The gradient arena is cut into buckets that follow the model's layer order (one bucket per transformer block, one
for the embedding, one for the head). A marker autograd node placed at the INPUT of every block fires when the
block's backward has finished (everything that contributes to the block's weight gradients has run), and launches
the all-reduce of that block's bucket on a side stream while the earlier blocks are still being differentiated.
Only the last micro-batch of a step communicates; ``finish_step`` reduces whatever is left and joins the streams.

The all-reduce itself is this repository's two-shot peer-memory kernel (``csrc/allreduce_twoshot.cu``) whenever the
gradient arena lives in symmetric memory (``symm`` given: the factory places it there on CUDA ranks of one node);
NCCL / gloo ``all_reduce`` otherwise (CPU ranks, or ``TESSERACT_DP_COMM=nccl`` for A/B runs).

The reference has no data parallelism (it is mentioned only in a comment, src/ops/cpu/Arithmetic.cpp:270).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


class _BucketMarker(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, reducer, bucket_id):
        ctx.reducer, ctx.bucket_id = reducer, bucket_id
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ids = ctx.bucket_id if isinstance(ctx.bucket_id, (tuple, list)) else (ctx.bucket_id,)
        for bid in ids:
            ctx.reducer._bucket_ready(bid)
        return g, None, None


class GradReducer:
    def __init__(self, arena, group, buckets: List[Tuple[int, int]], average: bool = True, symm=None):
        """``buckets``: [begin, end) element ranges of ``arena.grad`` in forward order. ``symm``: a
        ``fused_tp.SymmGradAllReduce`` over the symmetric buffer that ``arena.grad`` is a view of (offset 0)."""
        import torch.distributed as dist
        self.arena, self.group, self.buckets, self.average = arena, group, buckets, average
        self.symm = symm
        self.block_bucket0 = 0
        self.world = dist.get_world_size(group)
        self._dist = dist
        self._last = False
        self._done = [False] * len(buckets)
        self.stream = torch.cuda.Stream() if arena.grad.is_cuda else None
        self.overlapped_bytes = 0

    @staticmethod
    def layer_buckets(model, arena) -> List[Tuple[int, int]]:
        """One bucket per top-level child in registration order (embedding, each block, final norm + head)."""
        offs = {id(p): (o, o + p.numel()) for p, o in zip(arena.params, arena.offsets)}
        groups: List[List[int]] = []

        def span(mod):
            ids = [offs[id(p)] for p in mod.parameters() if id(p) in offs]
            return (min(a for a, _ in ids), max(b for _, b in ids)) if ids else None

        for name, child in model.named_children():
            if name == "layers":
                for blk in child:
                    s = span(blk)
                    if s:
                        groups.append(s)
            else:
                s = span(child)
                if s:
                    groups.append(s)
        groups.sort()
        # close gaps (alignment padding) so the buckets tile the arena
        out = []
        for i, (a, b) in enumerate(groups):
            end = groups[i + 1][0] if i + 1 < len(groups) else arena.numel
            out.append((a, end))
        if out:
            out[0] = (0, out[0][1])
        return out

    def mark(self, x: torch.Tensor, bucket_id) -> torch.Tensor:
        """Identity whose backward announces that the gradients of bucket ``bucket_id`` (an index or several) are
        complete."""
        if not (torch.is_grad_enabled() and x.requires_grad) or self.world == 1:
            return x
        return _BucketMarker.apply(x, self, bucket_id)

    def tail_buckets(self, num_blocks: int):
        """Buckets behind the last transformer block (final norm, head). With the fused head + loss their gradients are
        complete as soon as the backward pass has left the final norm, so they are reduced under the whole rest of
        the backward pass instead of after it."""
        return tuple(range(self.block_bucket0 + num_blocks, len(self.buckets)))

    def begin_step(self) -> None:
        self._done = [False] * len(self.buckets)
        self._last = False
        self.overlapped_bytes = 0

    def set_last_microbatch(self, flag: bool) -> None:
        self._last = flag

    def _reduce(self, bid: int, overlapped: bool) -> None:
        a, b = self.buckets[bid]
        g = self.arena.grad[a:b]
        if self.symm is not None:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                self.symm.all_reduce_(a * g.element_size(), b - a, g.dtype,
                                      scale=(1.0 / self.world) if self.average else 1.0)
        elif self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                if self.average:
                    g.div_(self.world)
                self._dist.all_reduce(g, group=self.group)
        else:
            if self.average:
                g.div_(self.world)
            self._dist.all_reduce(g, group=self.group)
        self._done[bid] = True
        if overlapped:
            self.overlapped_bytes += g.numel() * g.element_size()

    def _bucket_ready(self, bid: int) -> None:
        if self._last and self.world > 1 and not self._done[bid]:
            self._reduce(bid, overlapped=True)

    def finish_step(self) -> None:
        if self.world > 1:
            self.arena.fold_autograd_grads()
            for bid in range(len(self.buckets)):
                if not self._done[bid]:
                    self._reduce(bid, overlapped=False)
            if self.stream is not None:
                torch.cuda.current_stream().wait_stream(self.stream)
