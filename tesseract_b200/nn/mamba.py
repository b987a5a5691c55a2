"""Mamba (S6) block: in_proj -> split(x, z) -> causal conv1d -> SiLU -> x_proj -> split(dt, B, C) ->
softplus(dt_proj) -> A = -exp(A_log) -> selective scan -> y * silu(z) -> out_proj.

Parameters, initialisation and the two entry points follow the reference (src/nn/Mamba.cpp:33-186):
``in_proj`` [2 d_inner, d_model], ``x_proj`` [dt_rank + 2N, d_inner], ``dt_proj`` (with bias), ``out_proj``,
``conv_weight`` [d_inner, d_conv] = 1/d_conv, ``conv_bias`` = 0, ``A_log[d, n]`` = log(n + 1), ``D`` = 1.
``forward`` handles a whole sequence, ``forward_step`` one token with an ``SSMStateCache``.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..ops import ssm
from .kv_cache import SSMStateCache
from .modules import Linear, Module


class Mamba(Module):
    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2, dt_rank: int = 0,
                 dtype=torch.float32, device=None):
        super().__init__()
        if d_model <= 0 or d_state <= 0 or expand < 1 or d_conv < 1:
            raise ValueError("Mamba: d_model, d_state, expand must be > 0 and d_conv >= 1")
        self.d_model, self.d_state, self.d_conv = d_model, d_state, d_conv
        self.d_inner = expand * d_model
        self.dt_rank = dt_rank if dt_rank > 0 else (d_model + 15) // 16
        self.dtype = dtype
        self.in_proj = Linear(d_model, 2 * self.d_inner, bias=False, dtype=dtype, device=device)
        self.x_proj = Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False, dtype=dtype, device=device)
        self.dt_proj = Linear(self.dt_rank, self.d_inner, bias=True, dtype=dtype, device=device)
        self.out_proj = Linear(self.d_inner, d_model, bias=False, dtype=dtype, device=device)
        self.conv_weight = nn.Parameter(torch.full((self.d_inner, d_conv), 1.0 / d_conv, dtype=dtype, device=device))
        self.conv_bias = nn.Parameter(torch.zeros(self.d_inner, dtype=dtype, device=device))
        a = torch.log(torch.arange(1, d_state + 1, dtype=torch.float64)).to(dtype)
        self.A_log = nn.Parameter(a[None, :].repeat(self.d_inner, 1).to(device) if device else a[None, :].repeat(self.d_inner, 1))
        self.D = nn.Parameter(torch.ones(self.d_inner, dtype=dtype, device=device))

    def _ssm_inputs(self, x_conv):
        dbl = self.x_proj(x_conv)
        dt, Bm, Cm = torch.split(dbl, [self.dt_rank, self.d_state, self.d_state], dim=-1)
        delta = torch.nn.functional.softplus(self.dt_proj(dt))
        A = -torch.exp(self.A_log.float())
        return delta, A, Bm, Cm

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 3 or x.shape[2] != self.d_model:
            raise ValueError(f"Mamba.forward: expected [B, L, {self.d_model}]")
        x_in, z = torch.split(self.in_proj(x), [self.d_inner, self.d_inner], dim=-1)
        x_conv = ssm.causal_conv1d(x_in, self.conv_weight, self.conv_bias, silu=True)
        delta, A, Bm, Cm = self._ssm_inputs(x_conv)
        y, _ = ssm.selective_scan(x_conv, delta, A, Bm, Cm, self.D)
        return self.out_proj(y * torch.nn.functional.silu(z))

    @torch.no_grad()
    def forward_step(self, x: torch.Tensor, cache: SSMStateCache) -> torch.Tensor:
        if x.dim() != 3 or x.shape[1] != 1 or x.shape[2] != self.d_model:
            raise ValueError(f"Mamba.forward_step: expected [B, 1, {self.d_model}]")
        K = self.d_conv
        x_in, z = torch.split(self.in_proj(x), [self.d_inner, self.d_inner], dim=-1)
        if K > 1:
            window = torch.cat([cache.conv_state, x_in], dim=1)                # [B, K, d_inner]
            x_conv = ssm.causal_conv1d(window, self.conv_weight, self.conv_bias, silu=True)[:, K - 1:K]
            cache.conv_state = window[:, 1:].contiguous()
        else:
            x_conv = ssm.causal_conv1d(x_in, self.conv_weight, self.conv_bias, silu=True)
        delta, A, Bm, Cm = self._ssm_inputs(x_conv)
        y, st = ssm.selective_scan(x_conv, delta, A, Bm, Cm, self.D, cache.ssm_state)
        cache.ssm_state = st
        return self.out_proj(y * torch.nn.functional.silu(z))

    def make_state_cache(self, batch: int) -> SSMStateCache:
        return SSMStateCache(batch, self.d_inner, self.d_state, self.d_conv, self.dtype, self.conv_weight.device)
