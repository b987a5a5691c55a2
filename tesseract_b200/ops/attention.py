"""Attention entry points.

``flash_attention`` (training / prefill, BSHD layout, causal, GQA-native) runs the tcgen05
FlashAttention forward/backward kernels on CUDA bf16 tensors and the reference's composite
(scale folded into Q, causal key j <= query i, softmax in fp32, fully masked row -> zeros;
src/ops/cpu/Attention.cpp:272-317, src/cuda/FusedAttention.cu:69-80) everywhere else.
"""
from __future__ import annotations

import math
import os

import torch

from .. import _native
from .._native import check, lib, stream_ptr

_native.register_signatures({
    "tsb_flash_fwd": [_native.P] * 5 + [_native.I] * 6 + [_native.L] * 12 + [_native.F, _native.I, _native.P],
    "tsb_flash_fwd_varlen": [_native.P] * 5 + [_native.I] * 6 + [_native.L] * 8 + [_native.F, _native.P],
    "tsb_flash_bwd": [_native.P] * 10 + [_native.I] * 6 + [_native.L] * 12 + [_native.F, _native.I, _native.P],
    "tsb_flash_bwd_scratch_bytes": [_native.I] * 4,
})
_native._RESTYPES["tsb_flash_bwd_scratch_bytes"] = _native.L


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                  scale: float | None = None, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Composite attention on [B, H, S, D] tensors with GQA head mapping h -> h // (H / Hkv).

    Rectangular causal (Sq < Sk) aligns the last query with the last key, which is the chunked-prefill
    rule of the reference (first forbidden key = pos + i + 1, src/nn/MultiHeadAttention.cpp:181-200).
    """
    B, H, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if Hkv != H:
        rep = H // Hkv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    s = (q.float() * scale) @ k.float().transpose(-1, -2)
    if mask is not None:
        s = s + mask.float()
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    m = s.max(-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = (s - m).exp()
    denom = p.sum(-1, keepdim=True)
    p = torch.where(denom > 0, p / denom.clamp_min(1e-30), torch.zeros_like(p))
    return (p @ v.float()).to(q.dtype)


def _native_flash_available() -> bool:
    return hasattr(lib(), "tsb_flash_fwd") and os.environ.get("TESSERACT_ATTN", "tcgen05") == "tcgen05"


class _FlashFn(torch.autograd.Function):
    """q [B,S,H,D], k/v [B,S,Hkv,D] (any batch/seq/head strides, unit stride in D) -> o [B,S,H,D]."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        B, Sq, H, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        o = torch.empty((B, Sq, H, D), device=q.device, dtype=q.dtype)
        lse = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32)
        check(lib().tsb_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                  B, Sq, Sk, H, Hkv, D,
                                  q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
                                  scale, int(causal), stream_ptr(q.device)), "tsb_flash_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        B, Sq, H, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        do = do.contiguous()
        # dq/dk/dv are produced packed as one [B, S, (H + 2 Hkv), D] buffer when Sq == Sk so that the
        # gradient of a packed QKV projection needs no concatenation.
        if Sq == Sk:
            packed = torch.empty((B, Sq, H + 2 * Hkv, D), device=q.device, dtype=q.dtype)
            dq, dk, dv = packed[:, :, :H], packed[:, :, H:H + Hkv], packed[:, :, H + Hkv:]
        else:
            # one allocation with a common (batch, seq, head) stride triple for the three gradients
            Sm = max(Sq, Sk)
            packed = torch.empty((B, Sm, H + 2 * Hkv, D), device=q.device, dtype=q.dtype)
            dq, dk, dv = packed[:, :Sq, :H], packed[:, :Sk, H:H + Hkv], packed[:, :Sk, H + Hkv:]
        scratch = torch.empty(lib().tsb_flash_bwd_scratch_bytes(B, Sq, H, D), device=q.device, dtype=torch.uint8)
        if dk.stride() != dq.stride():
            raise RuntimeError("flash_attention backward: dq/dk/dv must share batch/seq/head strides")
        check(lib().tsb_flash_bwd(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                  lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(),
                                  B, Sq, Sk, H, Hkv, D,
                                  q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), dq.stride(0), dq.stride(1), dq.stride(2),
                                  ctx.scale, int(ctx.causal), stream_ptr(q.device)), "tsb_flash_bwd")
        _native.add_launches(3)
        return dq, dk, dv, None, None


class _FlashPackedFn(torch.autograd.Function):
    """Self-attention over a packed projection output qkv [B, S, H + 2 Hkv, D]; the gradient comes back in
    the same packed layout, ready for the QKV GEMM's backward (no slicing / concatenation passes)."""

    @staticmethod
    def forward(ctx, qkv, H, Hkv, causal, scale):
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        B, S, _, D = qkv.shape
        o = torch.empty((B, S, H, D), device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty((B, H, S), device=qkv.device, dtype=torch.float32)
        check(lib().tsb_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                  B, S, S, H, Hkv, D,
                                  q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
                                  scale, int(causal), stream_ptr(qkv.device)), "tsb_flash_fwd")
        ctx.save_for_backward(qkv, o, lse)
        ctx.args = (H, Hkv, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        H, Hkv, causal, scale = ctx.args
        B, S, _, D = qkv.shape
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :H], dqkv[:, :, H:H + Hkv], dqkv[:, :, H + Hkv:]
        scratch = torch.empty(lib().tsb_flash_bwd_scratch_bytes(B, S, H, D), device=qkv.device, dtype=torch.uint8)
        check(lib().tsb_flash_bwd(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                  lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(),
                                  B, S, S, H, Hkv, D,
                                  q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), dq.stride(0), dq.stride(1), dq.stride(2),
                                  scale, int(causal), stream_ptr(qkv.device)), "tsb_flash_bwd")
        _native.add_launches(3)
        return dqkv, None, None, None, None


def flash_attention_packed(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, causal: bool = True,
                           scale: float | None = None) -> torch.Tensor:
    """Self-attention on a packed [B, S, H + 2 Hkv, D] tensor (queries, then keys, then values along the
    head axis) -> [B, S, H, D]."""
    D = qkv.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    H, Hkv = num_heads, num_kv_heads
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and D in (64, 128) and qkv.is_contiguous()
            and _native_flash_available()):
        return _FlashPackedFn.apply(qkv, H, Hkv, bool(causal), float(scale))
    return flash_attention(qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:], causal=causal, scale=scale)


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                    scale: float | None = None) -> torch.Tensor:
    """Attention over BSHD tensors: q [B,Sq,H,D], k/v [B,Sk,Hkv,D] -> [B,Sq,H,D]."""
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and q.stride(-1) == 1 and _native_flash_available():
        return _FlashFn.apply(q, k, v, bool(causal), float(scale))
    if q.is_cuda and os.environ.get("TESSERACT_ATTN", "") == "sdpa":
        # Library fallback kept for A/B comparisons only (never the default on a GPU).
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=(k.shape[2] != q.shape[2]))
        return o.transpose(1, 2).contiguous()
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
        raise RuntimeError("flash_attention: the native tcgen05 kernel is not in the built library "
                           "(rebuild with `python -m tesseract_b200.build`)")
    o = attention_ref(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal, scale=scale)
    return o.transpose(1, 2).contiguous()


def flash_attention_varlen_packed(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int, num_heads: int,
                                  num_kv_heads: int, scale: float | None = None) -> torch.Tensor:
    """Causal self-attention over sequences of different lengths packed on one token axis (inference, no autograd):
    qkv [T, H + 2 Hkv, D] (queries, keys, values along the head axis), cu_seqlens int32 [n + 1] -> [T, H, D].
    One kernel launch for the whole batch on CUDA bf16; per-sequence calls otherwise."""
    T, _, D = qkv.shape
    H, Hkv = num_heads, num_kv_heads
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    n = cu_seqlens.shape[0] - 1
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and D in (64, 128) and qkv.is_contiguous()
            and _native_flash_available() and hasattr(lib(), "tsb_flash_fwd_varlen")):
        q, k, v = qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]
        o = torch.empty((T, H, D), device=qkv.device, dtype=qkv.dtype)
        cu = cu_seqlens.to(device=qkv.device, dtype=torch.int32).contiguous()
        check(lib().tsb_flash_fwd_varlen(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), cu.data_ptr(), n,
                                         int(max_len), T, H, Hkv, D, q.stride(0), q.stride(1), k.stride(0), k.stride(1),
                                         v.stride(0), v.stride(1), o.stride(0), o.stride(1), float(scale),
                                         stream_ptr(qkv.device)), "tsb_flash_fwd_varlen")
        return o
    bounds = cu_seqlens.tolist()
    outs = [flash_attention_packed(qkv[a:b].unsqueeze(0), H, Hkv, causal=True, scale=scale)[0]
            for a, b in zip(bounds[:-1], bounds[1:])]
    return torch.cat(outs, dim=0)
