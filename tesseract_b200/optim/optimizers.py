"""SGD and Adam.

``Adam`` follows the reference formula exactly (src/optim/Adam.cpp:70-90; no weight decay by default):
m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p -= lr * (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps).
On CUDA the whole update is ONE kernel launch: over the flat arena when the parameters live in a
``ParamArena``, else over a device table of tensors (``tsb_adam_multi``). State is fp32; an fp32 master
copy of bf16 parameters is optional.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, Optional

import torch

from .. import _native
from .._native import check, dtype_code, lib, stream_ptr
from .arena import ParamArena


class Optimizer:
    def __init__(self, params):
        if isinstance(params, ParamArena):
            self.arena: Optional[ParamArena] = params
            self.params = params.params
        else:
            self.arena = None
            self.params = [p for p in params]
        if not self.params:
            raise ValueError("optimizer got an empty parameter list")

    def zero_grad(self) -> None:
        """Drops every gradient (the reference unsets ``.grad`` rather than zero-filling it)."""
        if self.arena is not None:
            self.arena.zero_grad()
        else:
            for p in self.params:
                p.grad = None

    def _grad_of(self, p):
        g = p.grad
        if g is None:
            g = getattr(p, "main_grad", None) if self.arena is not None else None
        return g


class SGD(Optimizer):
    """p -= lr * (momentum-filtered) g (src/optim/SGD.cpp:18-55)."""

    def __init__(self, params, lr: float, momentum: float = 0.0):
        super().__init__(params)
        self.lr, self.momentum = lr, momentum
        self._vel = {}

    @torch.no_grad()
    def step(self) -> None:
        for p in self.params:
            g = self._grad_of(p)
            if g is None:
                continue
            g = g.to(p.dtype)
            if self.momentum != 0.0:
                v = self._vel.get(id(p))
                v = g.clone() if v is None else v.mul_(self.momentum).add_(g)
                self._vel[id(p)] = v
                g = v
            p.add_(g, alpha=-self.lr)


class Adam(Optimizer):
    def __init__(self, params, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: float = 0.0):
        super().__init__(params)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay, self.max_grad_norm = weight_decay, max_grad_norm
        self.t = 0
        self._state = {}       # id(param) -> (m, v) for the per-tensor paths
        self._flat_state = None
        self._table = None     # cached device table for the multi-tensor launch
        self._scratch = None

    # -- state dict (checkpoint / resume) ------------------------------------------------------------
    def state_dict(self) -> dict:
        if self._flat_state is not None:
            m, v = self._flat_state
            return {"t": self.t, "flat_m": m, "flat_v": v}
        return {"t": self.t, "m": [self._state.get(id(p), (None, None))[0] for p in self.params],
                "v": [self._state.get(id(p), (None, None))[1] for p in self.params]}

    def load_state_dict(self, sd: dict) -> None:
        self.t = int(sd["t"])
        if "flat_m" in sd:
            self._flat_state = (sd["flat_m"], sd["flat_v"])
        else:
            for p, m, v in zip(self.params, sd["m"], sd["v"]):
                if m is not None:
                    self._state[id(p)] = (m, v)
            self._table = None

    # -- update --------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        self.t += 1
        bc1 = 1.0 - self.beta1 ** self.t
        bc2 = 1.0 - self.beta2 ** self.t
        if self.arena is not None:
            self.arena.fold_autograd_grads()
            self._step_arena(bc1, bc2)
            return
        active = [p for p in self.params if p.grad is not None]
        if not active:
            return
        if all(p.is_cuda and p.dtype in (torch.float32, torch.bfloat16, torch.float16) for p in active):
            self._step_multi(active, bc1, bc2)
        else:
            for p in active:
                self._step_torch(p, p.grad, bc1, bc2)

    def _step_torch(self, p, g, bc1, bc2):
        st = self._state.get(id(p))
        if st is None:
            st = (torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32))
            self._state[id(p)] = st
        m, v = st
        gf = g.float()
        m.mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
        upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
        if self.weight_decay:
            upd = upd + self.weight_decay * p.float()
        p.copy_((p.float() - self.lr * upd).to(p.dtype))

    def _gscale(self, grads, device):
        """Device scalar multiplying every gradient: the clipping coefficient (no host sync)."""
        if self.max_grad_norm <= 0:
            return None
        if self._scratch is None:
            self._scratch = torch.zeros(2, device=device, dtype=torch.float32)
        self._scratch.zero_()
        for g in grads:
            check(lib().tsb_sumsq(g.data_ptr(), g.numel(), self._scratch.data_ptr(), dtype_code(g.dtype),
                                  stream_ptr(device)), "tsb_sumsq")
        check(lib().tsb_clip_coef(self._scratch.data_ptr(), self._scratch[1:].data_ptr(), self.max_grad_norm, 1.0,
                                  stream_ptr(device)), "tsb_clip_coef")
        return self._scratch[1:]

    def _step_arena(self, bc1, bc2):
        a = self.arena
        if self._flat_state is None:
            self._flat_state = (torch.zeros(a.numel, device=a.device, dtype=torch.float32),
                                torch.zeros(a.numel, device=a.device, dtype=torch.float32))
        m, v = self._flat_state
        if not a.flat.is_cuda:
            gf = a.grad.float()
            if self.max_grad_norm > 0:
                gf = gf * min(1.0, self.max_grad_norm / (gf.norm().item() + 1e-6))
            m.mul_(self.beta1).add_(gf, alpha=1 - self.beta1)
            v.mul_(self.beta2).addcmul_(gf, gf, value=1 - self.beta2)
            w = a.master if a.master is not None else a.flat.float()
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            if self.weight_decay:
                upd = upd + self.weight_decay * w
            w = w - self.lr * upd
            if a.master is not None:
                a.master.copy_(w)
            a.flat.copy_(w.to(a.dtype))
            return
        gscale = self._gscale([a.grad], a.device)
        check(lib().tsb_adam_flat(a.flat.data_ptr(), a.grad.data_ptr(), m.data_ptr(), v.data_ptr(),
                                  a.master.data_ptr() if a.master is not None else None, a.numel, self.lr, self.beta1,
                                  self.beta2, self.eps, bc1, bc2, self.weight_decay,
                                  gscale.data_ptr() if gscale is not None else None, dtype_code(a.dtype),
                                  dtype_code(a.grad_dtype), stream_ptr(a.device)), "tsb_adam_flat")

    def _step_multi(self, active, bc1, bc2):
        dev = active[0].device
        key = tuple((p.data_ptr(), p.grad.data_ptr()) for p in active)
        if self._table is None or self._table[0] != key:
            chunk = lib().tsb_adam_chunk_elems()
            recs, work = [], []
            for i, p in enumerate(active):
                st = self._state.get(id(p))
                if st is None:
                    st = (torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32))
                    self._state[id(p)] = st
                if not p.is_contiguous() or not p.grad.is_contiguous():
                    raise RuntimeError("Adam: parameters and gradients must be contiguous")
                recs += [p.data_ptr(), p.grad.data_ptr(), st[0].data_ptr(), st[1].data_ptr(), 0, p.numel()]
                work += [(i, c) for c in range((p.numel() + chunk - 1) // chunk)]
            table = torch.tensor(recs, dtype=torch.int64).to(dev)
            workt = torch.tensor(work, dtype=torch.int32).to(dev)
            self._table = (key, table, workt)
        _, table, workt = self._table
        pd = {dtype_code(p.dtype) for p in active}
        gd = {dtype_code(p.grad.dtype) for p in active}
        if len(pd) != 1 or len(gd) != 1:
            for p in active:
                self._step_torch(p, p.grad, bc1, bc2)
            return
        gscale = self._gscale([p.grad for p in active], dev)
        check(lib().tsb_adam_multi(table.data_ptr(), workt.data_ptr(), workt.shape[0], self.lr, self.beta1, self.beta2,
                                   self.eps, bc1, bc2, self.weight_decay,
                                   gscale.data_ptr() if gscale is not None else None, pd.pop(), gd.pop(),
                                   stream_ptr(dev)), "tsb_adam_multi")
