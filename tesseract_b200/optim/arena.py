"""Parameter / gradient arenas: every parameter of a model becomes a view into one flat buffer, with a
second flat buffer of the same layout for gradients (``param.main_grad``).

Why: (1) the optimizer is ONE kernel launch over the arena instead of one per tensor (the reference
launches Adam once per parameter, src/optim/Adam.cpp:30-67); (2) neighbouring projections (q/k/v,
gate/up) are contiguous and run as one GEMM; (3) the data-parallel gradient all-reduce works on large
contiguous buckets; (4) zeroing gradients is one memset instead of freeing every ``.grad``
(src/optim/Optimizer.cpp:7-12).
"""
from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

_ALIGN_ELEMS = 128  # every parameter starts on a 256-byte (bf16) / 512-byte (fp32) boundary


class ParamArena:
    def __init__(self, params: Iterable[nn.Parameter], grad_dtype: torch.dtype | None = None,
                 master_weights: bool = False, grad_alloc=None):
        """``grad_alloc(numel, dtype, device) -> flat tensor`` lets the caller place the gradient buffer (e.g. in
        peer-mapped memory, so that a data-parallel all-reduce kernel can work on it in place)."""
        self.params = [p for p in params]
        if not self.params:
            raise ValueError("ParamArena: no parameters")
        p0 = self.params[0]
        if any(p.dtype != p0.dtype or p.device != p0.device for p in self.params):
            raise ValueError("ParamArena: all parameters must share dtype and device")
        self.dtype, self.device = p0.dtype, p0.device
        self.grad_dtype = grad_dtype or p0.dtype
        self.offsets = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            n = p.numel()
            off += (n + _ALIGN_ELEMS - 1) // _ALIGN_ELEMS * _ALIGN_ELEMS
        self.numel = off
        self.flat = torch.zeros(off, dtype=self.dtype, device=self.device)
        if grad_alloc is not None:
            self.grad = grad_alloc(off, self.grad_dtype, self.device)
            if self.grad.numel() != off or self.grad.dtype != self.grad_dtype or not self.grad.is_contiguous():
                raise ValueError("ParamArena: grad_alloc returned a buffer of the wrong size, dtype or layout")
            self.grad.zero_()
        else:
            self.grad = torch.zeros(off, dtype=self.grad_dtype, device=self.device)
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                view = self.flat[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
        self.master = self.flat.float() if master_weights and self.dtype != torch.float32 else None

    @classmethod
    def from_module(cls, module: nn.Module, **kw) -> "ParamArena":
        seen, params = set(), []
        for p in module.parameters():
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                params.append(p)
        return cls(params, **kw)

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p in self.params:
            p.grad = None

    def fold_autograd_grads(self) -> None:
        """Add any ``param.grad`` produced by plain autograd into the arena (ops without a fused
        main_grad path), then drop it."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(self.grad_dtype))
                p.grad = None

    def bytes(self) -> int:
        n = self.flat.numel() * self.flat.element_size() + self.grad.numel() * self.grad.element_size()
        if self.master is not None:
            n += self.master.numel() * 4
        return n
