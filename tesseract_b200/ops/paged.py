"""Attention over KV caches for decoding: GQA decode over contiguous caches and ragged decode /
chunked prefill over paged pools (full precision and INT8 with per-token scales).

Semantics are the reference's (src/nn/PagedAttention.cpp:15-140, src/ops/cpu/Attention.cpp:320-515):
pool layout [num_blocks, Hkv, block_size, D]; block_tables int32 [A, max_logical]; lens int32 [A];
query head h reads KV head h // (H / Hkv); in chunked prefill query s of S new tokens of a request whose
cache holds kv_len tokens (new ones included) sees keys [0, kv_len - S + s]; out-of-range block ids are
clamped to block 0. CPU tensors (and dtypes the kernels do not take) run the torch statement below, which
is also the oracle for the split-K CUDA kernels in ``csrc/decode_attn.cu``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native
from .._native import check, lib, stream_ptr

P, I, L, F = _native.P, _native.I, _native.L, _native.F
_native.register_signatures({
    "tsb_paged_decode": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P],
    "tsb_paged_decode_mx": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P],
    "tsb_paged_decode_scratch_floats": [I, I, I, I],
    "tsb_paged_decode_static_need_floats": [I, I, I, I, I, I],
    "tsb_kv_append_paged": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
})
_native._RESTYPES["tsb_paged_decode_scratch_floats"] = _native.L
_native._RESTYPES["tsb_paged_decode_static_need_floats"] = _native.L


def _gather_request(pool: torch.Tensor, table: torch.Tensor, length: int) -> torch.Tensor:
    """pool [nb, Hkv, bs, ...] -> [Hkv, length, ...] for one request."""
    nb, Hkv, bs = pool.shape[:3]
    n = (length + bs - 1) // bs
    idx = table[:n].long().clamp(0, nb - 1)
    g = pool.index_select(0, idx).transpose(0, 1)
    return g.reshape(Hkv, n * bs, *pool.shape[3:])[:, :length]


def paged_attention_ref(q: torch.Tensor, k_pool, v_pool, block_tables, lens, scale: Optional[float] = None,
                        k_scale=None, v_scale=None) -> torch.Tensor:
    """q [A, S, H, D] (S new tokens per request, the last of which is the newest) -> [A, S, H, D]."""
    A, S, H, D = q.shape
    Hkv = k_pool.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.zeros_like(q)
    rep = H // Hkv
    for a in range(A):
        L_a = int(lens[a])
        if L_a <= 0:
            continue
        k = _gather_request(k_pool, block_tables[a], L_a).float()
        v = _gather_request(v_pool, block_tables[a], L_a).float()
        if k_scale is not None:
            k = k * _gather_request(k_scale, block_tables[a], L_a).unsqueeze(-1)
            v = v * _gather_request(v_scale, block_tables[a], L_a).unsqueeze(-1)
        k = k.repeat_interleave(rep, dim=0)                      # [H, L, D]
        v = v.repeat_interleave(rep, dim=0)
        qa = q[a].float().transpose(0, 1) * scale               # [H, S, D]
        s = qa @ k.transpose(1, 2)                               # [H, S, L]
        i = torch.arange(S, device=q.device)[:, None] + (L_a - S)
        j = torch.arange(L_a, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        out[a] = (p @ v).transpose(0, 1).to(q.dtype)
    return out


def _native_decode_ok(q: torch.Tensor, k_pool: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and q.shape[-1] in (64, 128)
            and hasattr(lib(), "tsb_paged_decode") and k_pool.shape[2] % 8 == 0)


_scratch_cache: dict = {}
_scratch_retired: list = []   # outgrown buffers stay alive: captured CUDA graphs may still point at them


def _decode_scratch(device, floats: int) -> torch.Tensor:
    t = _scratch_cache.get(device)
    if t is None or t.numel() < floats:
        if t is not None:
            _scratch_retired.append(t)
        t = torch.empty(max(floats, 1 << 20), device=device, dtype=torch.float32)
        _scratch_cache[device] = t
    return t


def _scratch_floats(A: int, H: int, Hkv: int, D: int, max_len: int, int8: bool) -> int:
    """fp32 elements of split scratch the kernel's plan asks for (the worst case over all plans when the library
    has no plan query)."""
    if hasattr(lib(), "tsb_paged_decode_static_need_floats"):
        need = int(lib().tsb_paged_decode_static_need_floats(A, H, Hkv, D, max_len, 1 if int8 else 0))
        if need >= 0:
            return need
    return int(lib().tsb_paged_decode_scratch_floats(A, H, D, max_len))


def paged_decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                           lens: torch.Tensor, scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                           v_scale: Optional[torch.Tensor] = None, max_len_hint: int = 0) -> torch.Tensor:
    """One new token per request: q [A, H, D] -> [A, H, D]. INT8 pools pass ``k_scale`` / ``v_scale``."""
    A, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if _native_decode_ok(q, k_pool) and (k_scale is None or k_pool.dtype == torch.int8):
        nb, Hkv, bs, _ = k_pool.shape
        out = torch.empty_like(q)
        max_len = int(max_len_hint) if max_len_hint > 0 else block_tables.shape[1] * bs
        floats = _scratch_floats(A, H, Hkv, D, max_len, k_scale is not None)
        scratch = _decode_scratch(q.device, floats)
        bt = block_tables if block_tables.dtype == torch.int32 else block_tables.to(torch.int32)
        if bt.stride(1) != 1:
            bt = bt.contiguous()
        ln = lens if lens.dtype == torch.int32 else lens.to(torch.int32)
        check(lib().tsb_paged_decode(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                     k_scale.data_ptr() if k_scale is not None else None,
                                     v_scale.data_ptr() if v_scale is not None else None,
                                     bt.data_ptr(), ln.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                     A, H, Hkv, D, bs, nb, bt.stride(0), float(scale), max_len,
                                     1 if q.dtype == torch.bfloat16 else 2, stream_ptr(q.device)), "tsb_paged_decode")
        _native.add_launches(1)
        return out
    return paged_attention_ref(q.unsqueeze(1), k_pool, v_pool, block_tables, lens, scale, k_scale, v_scale).squeeze(1)


def paged_decode_attention_mx(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor,
                              lens: torch.Tensor, scale: Optional[float] = None,
                              k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
                              max_len_hint: int = 0):
    """``quantize_act_mx(paged_decode_attention(...).view(A, H * D))``: the attention output as the E4M3 +
    power-of-two-scale operand ``(q, sf)`` of the output projection's MX GEMM. With head_dim 128, bf16 and a split
    key range the merge kernel of the splits writes the operand itself (no bf16 round trip, one launch fewer)."""
    from . import fp8
    A, H, D = q.shape
    if not (_native_decode_ok(q, k_pool) and (k_scale is None or k_pool.dtype == torch.int8)
            and q.dtype == torch.bfloat16 and (H * D) % 128 == 0 and hasattr(lib(), "tsb_paged_decode_mx")):
        o = paged_decode_attention(q, k_pool, v_pool, block_tables, lens, scale, k_scale, v_scale, max_len_hint)
        return fp8.quantize_act_mx(o.view(A, H * D))
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    nb, Hkv, bs, _ = k_pool.shape
    out = torch.empty_like(q)
    xq, sf = fp8._mx_buffers(A, H * D, q.device)
    max_len = int(max_len_hint) if max_len_hint > 0 else block_tables.shape[1] * bs
    scratch = _decode_scratch(q.device, _scratch_floats(A, H, Hkv, D, max_len, k_scale is not None))
    bt = block_tables if block_tables.dtype == torch.int32 else block_tables.to(torch.int32)
    if bt.stride(1) != 1:
        bt = bt.contiguous()
    ln = lens if lens.dtype == torch.int32 else lens.to(torch.int32)
    check(lib().tsb_paged_decode_mx(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                    k_scale.data_ptr() if k_scale is not None else None,
                                    v_scale.data_ptr() if v_scale is not None else None,
                                    bt.data_ptr(), ln.data_ptr(), out.data_ptr(), scratch.data_ptr(), xq.data_ptr(),
                                    sf.data_ptr(), A, H, Hkv, D, bs, nb, bt.stride(0), float(scale), max_len, 1,
                                    stream_ptr(q.device)), "tsb_paged_decode_mx")
    _native.add_launches(1)
    return xq, sf


def paged_decode_attention_int8(q, k_pool, v_pool, k_scale, v_scale, block_tables, lens, scale=None):
    return paged_decode_attention(q, k_pool, v_pool, block_tables, lens, scale, k_scale, v_scale)


_PREFILL_QUERIES_PER_LAUNCH = 32768   # pseudo-requests per launch (the request index is a grid z coordinate)


def paged_prefill_attention(q: torch.Tensor, k_pool, v_pool, block_tables, lens, scale: Optional[float] = None,
                            k_scale=None, v_scale=None) -> torch.Tensor:
    """Chunked prefill: q [A, S, H, D] against each request's pooled keys (new tokens already appended).

    On the GPU the pools are read in place by the paged decode kernel (bf16 / fp16 or INT8 with per-token scales;
    no gathered or dequantised views): new token ``s`` of request ``a`` is a decode query with the request's block
    table and its own causal length ``lens[a] - S + s + 1``. The reference's kernels for the same op:
    src/cuda/PagedAttention.cu:275-439."""
    A, S, H, D = q.shape
    if not (_native_decode_ok(q, k_pool) and (k_scale is None or k_pool.dtype == torch.int8)) or A * S == 0:
        return paged_attention_ref(q, k_pool, v_pool, block_tables, lens, scale, k_scale, v_scale)
    qf = q.reshape(A * S, H, D)
    if not qf.is_contiguous():
        qf = qf.contiguous()
    bt = block_tables if block_tables.dtype == torch.int32 else block_tables.to(torch.int32)
    ln = lens if lens.dtype == torch.int32 else lens.to(torch.int32)
    steps = torch.arange(S, device=q.device, dtype=torch.int32)
    q_lens = (ln[:, None] - (S - 1) + steps[None, :]).clamp_min(0).reshape(-1).contiguous()
    q_tables = bt.repeat_interleave(S, dim=0)
    max_len = block_tables.shape[1] * k_pool.shape[2]
    out = torch.empty_like(qf)
    for lo in range(0, A * S, _PREFILL_QUERIES_PER_LAUNCH):
        hi = min(A * S, lo + _PREFILL_QUERIES_PER_LAUNCH)
        out[lo:hi] = paged_decode_attention(qf[lo:hi], k_pool, v_pool, q_tables[lo:hi], q_lens[lo:hi], scale, k_scale,
                                            v_scale, max_len_hint=max_len)
    return out.view(A, S, H, D)


def paged_prefill_attention_int8(q, k_pool, v_pool, k_scale, v_scale, block_tables, lens, scale=None):
    return paged_prefill_attention(q, k_pool, v_pool, block_tables, lens, scale, k_scale, v_scale)


def decode_attention_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None):
    """Single-position decode against a contiguous prefix: q [B, H, 1, D], k/v [B, Hkv, L, D]."""
    from .attention import attention_ref
    return attention_ref(q, k, v, causal=False, scale=scale)


def prefill_attention_gqa(q, k, v, scale: Optional[float] = None):
    """Causal prefill: q [B, H, S, D] with k/v [B, Hkv, L, D], L >= S (last query sees every key)."""
    from .attention import attention_ref
    return attention_ref(q, k, v, causal=True, scale=scale)
