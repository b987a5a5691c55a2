"""Fused bandwidth-bound ops with autograd: RMSNorm (+ residual), SwiGLU, RoPE on packed QKV,
embedding, cross-entropy. CUDA tensors run the sm_100a kernels of ``csrc/fused_norm_act.cu`` and
``csrc/loss_optim.cu``; CPU tensors run the plain torch restatement of the reference's math, which is
also the oracle the kernels are tested against.

Reference semantics: RMSNorm composite (src/ops/cpu/RMSNorm.cpp:49-97), SwiGLU ``silu(gate) * up``
(src/ops/cpu/SwiGLU.cpp:106-115), adjacent-pair RoPE (src/ops/cpu/RotaryEmbedding.cpp,
src/nn/RotaryEmbedding.cpp:35-57), mean cross-entropy with int64 targets (src/ops/cpu/Loss.cpp:154).
"""
from __future__ import annotations

import torch

from .. import _native
from .._native import check, dtype_code, lib, stream_ptr

_NATIVE_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in _NATIVE_DTYPES


# --------------------------------------------------------------------------------------- RMSNorm
def rms_norm_ref(x, weight, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * weight.float()).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    """y = rmsnorm(x [+ residual]) * w. Returns (y, h) where h = x + residual (or x itself)."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps, wgrad_buf):
        ctx.set_materialize_grads(False)
        D = x.shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        y = torch.empty(x.shape, device=x.device, dtype=x.dtype)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        if residual is not None:
            r2 = residual.reshape(-1, D).contiguous()
            h = torch.empty(x.shape, device=x.device, dtype=x.dtype)
            check(lib().tsb_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), weight.data_ptr(), y.data_ptr(), h.data_ptr(),
                                        rstd.data_ptr(), rows, D, eps, dtype_code(x.dtype), stream_ptr(x.device)),
                  "tsb_rmsnorm_fwd")
        else:
            h = x2
            check(lib().tsb_rmsnorm_fwd(x2.data_ptr(), None, weight.data_ptr(), y.data_ptr(), None,
                                        rstd.data_ptr(), rows, D, eps, dtype_code(x.dtype), stream_ptr(x.device)),
                  "tsb_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = residual is not None
        ctx.wgrad_buf = wgrad_buf
        ctx.shape = x.shape
        return y, (h if residual is not None else None)

    @staticmethod
    def backward(ctx, dy, dh):
        h, weight, rstd = ctx.saved_tensors
        D = h.shape[-1]
        h = h.reshape(-1, D)
        rows = h.shape[0]
        if dy is None:
            dy = torch.zeros(ctx.shape, device=h.device, dtype=h.dtype)
        dy2 = dy.reshape(-1, D).contiguous()
        dh2 = dh.reshape(-1, D).contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        parts = lib().tsb_rmsnorm_bwd_parts(rows)
        partial = torch.empty((parts, D), device=h.device, dtype=torch.float32)
        buf = ctx.wgrad_buf
        if buf is not None and buf.dtype == weight.dtype:
            dw_t, acc, dw_ret = buf, 1, None
        else:
            dw_t = torch.empty_like(weight)
            acc, dw_ret = 0, dw_t
        check(lib().tsb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                    dh2.data_ptr() if dh2 is not None else None, dx.data_ptr(), dw_t.data_ptr(),
                                    partial.data_ptr(), rows, D, acc, dtype_code(h.dtype), stream_ptr(h.device)),
              "tsb_rmsnorm_bwd")
        _native.add_launches(1)
        if buf is not None and dw_ret is not None:
            buf.add_(dw_ret.to(buf.dtype))
            dw_ret = None
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw_ret, None, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
             wgrad_buf: torch.Tensor | None = None):
    """RMSNorm over the last dimension. With ``residual`` returns ``(y, x + residual)``; else ``y``."""
    if _native_ok(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192 and weight.dtype == x.dtype:
        y, h = _RMSNormFn.apply(x, residual, weight, float(eps), wgrad_buf)
        return (y, h) if residual is not None else y
    if residual is not None:
        h = x + residual
        return _ref_norm_with_buf(h, weight, eps, wgrad_buf), h
    return _ref_norm_with_buf(x, weight, eps, wgrad_buf)


class _GradToBuf(torch.autograd.Function):
    """Identity on a parameter whose gradient is added into ``buf`` instead of ``param.grad``."""

    @staticmethod
    def forward(ctx, w, buf):
        ctx.buf = buf
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        ctx.buf.add_(g.to(ctx.buf.dtype))
        return None, None


def grad_to_buf(w: torch.Tensor, buf: torch.Tensor | None) -> torch.Tensor:
    if buf is None or not (torch.is_grad_enabled() and w.requires_grad):
        return w
    return _GradToBuf.apply(w, buf)


def _ref_norm_with_buf(x, weight, eps, wgrad_buf):
    return rms_norm_ref(x, grad_to_buf(weight, wgrad_buf), eps)


# --------------------------------------------------------------------------------------- SwiGLU
def swiglu_ref(gate_up: torch.Tensor) -> torch.Tensor:
    F = gate_up.shape[-1] // 2
    g, u = gate_up[..., :F].float(), gate_up[..., F:].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        F = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * F).contiguous()
        out = torch.empty((gu.shape[0], F), device=gu.device, dtype=gu.dtype)
        check(lib().tsb_swiglu_fwd(gu.data_ptr(), out.data_ptr(), gu.shape[0], F, dtype_code(gu.dtype),
                                   stream_ptr(gu.device)), "tsb_swiglu_fwd")
        ctx.save_for_backward(gu)
        ctx.shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        F = gu.shape[-1] // 2
        d2 = dout.reshape(-1, F).contiguous()
        dgu = torch.empty_like(gu)
        check(lib().tsb_swiglu_bwd(d2.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.shape[0], F,
                                   dtype_code(gu.dtype), stream_ptr(gu.device)), "tsb_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu_backward(gate_up: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """Gradient of ``swiglu`` with respect to the packed [rows, 2F] input (CUDA kernel; no autograd)."""
    F = gate_up.shape[-1] // 2
    gu = gate_up.reshape(-1, 2 * F).contiguous()
    d2 = dout.reshape(-1, F).contiguous()
    dgu = torch.empty_like(gu)
    check(lib().tsb_swiglu_bwd(d2.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.shape[0], F, dtype_code(gu.dtype),
                               stream_ptr(gu.device)), "tsb_swiglu_bwd")
    return dgu.view(gate_up.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for a packed [..., 2F] tensor (gate = first half of the last dimension)."""
    F = gate_up.shape[-1] // 2
    if _native_ok(gate_up) and F % 8 == 0:
        return _SwiGLUFn.apply(gate_up)
    return swiglu_ref(gate_up)


def swiglu_silu_gate(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Two-operand form of the reference API (``ops::swiglu_silu_gate``)."""
    if _native_ok(gate) and gate.shape[-1] % 8 == 0:
        return swiglu(torch.cat([gate, up], dim=-1))
    return (torch.nn.functional.silu(gate.float()) * up.float()).to(gate.dtype)


# --------------------------------------------------------------------------------------- RoPE
def rope_tables(max_pos: int, head_dim: int, theta: float, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [max_pos, head_dim/2] (fp32): angle(p, j) = p * theta^(-2j/d)."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = theta ** (-j / head_dim)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Adjacent-pair rotation of x [..., T, H, D] (positions [T] or broadcastable [..., T])."""
    c = cos[positions].unsqueeze(-2)  # [..., T, 1, D/2]
    s = sin[positions].unsqueeze(-2)
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    out = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    return out.to(x.dtype)


class _RopeQKVFn(torch.autograd.Function):
    """In-place rotation of the query and key heads of a packed [T, (Hq + 2 Hkv) * D] buffer."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, seq_len, pos_offset, hq, hkv, D):
        assert qkv.is_contiguous()
        T = qkv.shape[0]
        check(lib().tsb_rope_qkv(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                 positions.data_ptr() if positions is not None else None, T, seq_len, pos_offset,
                                 hq + hkv, hq + 2 * hkv, D, 1.0, dtype_code(qkv.dtype), stream_ptr(qkv.device)),
              "tsb_rope_qkv")
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(cos, sin, positions)
        ctx.args = (seq_len, pos_offset, hq, hkv, D)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        cos, sin, positions = ctx.saved_tensors
        seq_len, pos_offset, hq, hkv, D = ctx.args
        d = dqkv.contiguous()
        if d.data_ptr() == dqkv.data_ptr():
            d = d.clone()
        check(lib().tsb_rope_qkv(d.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                 positions.data_ptr() if positions is not None else None, d.shape[0], seq_len,
                                 pos_offset, hq + hkv, hq + 2 * hkv, D, -1.0, dtype_code(d.dtype),
                                 stream_ptr(d.device)), "tsb_rope_qkv")
        return d, None, None, None, None, None, None, None, None


def rope_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, num_heads: int, num_kv_heads: int,
             head_dim: int, seq_len: int, pos_offset: int = 0, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate the Q and K heads of packed ``qkv`` [T, (Hq + 2 Hkv) * D]; token t sits at position
    ``positions[t]`` (int32) or ``pos_offset + t % seq_len``. V is left untouched."""
    T = qkv.shape[0]
    if _native_ok(qkv) and head_dim % 8 == 0:
        if positions is not None:
            positions = positions.to(torch.int32)
        return _RopeQKVFn.apply(qkv, cos, sin, positions, seq_len, pos_offset, num_heads, num_kv_heads, head_dim)
    if positions is None:
        positions = pos_offset + (torch.arange(T, device=qkv.device) % seq_len)
    x = qkv.view(T, num_heads + 2 * num_kv_heads, head_dim)
    rot = rope_ref(x[:, : num_heads + num_kv_heads], cos, sin, positions.long())
    return torch.cat([rot, x[:, num_heads + num_kv_heads:]], dim=1).reshape(T, -1)


# --------------------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, wgrad_buf):
        flat = ids.reshape(-1).contiguous()
        D = table.shape[1]
        out = torch.empty((flat.numel(), D), device=table.device, dtype=table.dtype)
        check(lib().tsb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), D,
                                      table.shape[0], dtype_code(table.dtype), stream_ptr(table.device)),
              "tsb_embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.wgrad_buf = wgrad_buf
        ctx.tshape = table.shape
        ctx.tdtype = table.dtype
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        V, D = ctx.tshape
        d2 = dy.reshape(-1, D).contiguous()
        buf = ctx.wgrad_buf
        ret = None
        if buf is not None and buf.dtype in (torch.float32, torch.bfloat16):
            tgt = buf
        else:
            tgt = torch.zeros((V, D), device=dy.device, dtype=torch.float32)
            ret = tgt
        check(lib().tsb_embedding_bwd(flat.data_ptr(), d2.data_ptr(), tgt.data_ptr(), flat.numel(), D, V,
                                      dtype_code(d2.dtype), int(tgt.dtype == torch.float32), stream_ptr(dy.device)),
              "tsb_embedding_bwd")
        if ret is not None:
            ret = ret.to(ctx.tdtype)
            if buf is not None:
                buf.add_(ret.to(buf.dtype))
                ret = None
        return None, ret, None


def embedding(ids: torch.Tensor, table: torch.Tensor, wgrad_buf: torch.Tensor | None = None) -> torch.Tensor:
    """Row gather ``table[ids]`` for int64 ids (validated against the vocabulary size)."""
    if ids.dtype != torch.int64:
        raise TypeError("embedding: ids must be int64")
    if _native_ok(table) and table.shape[1] % 8 == 0 and ids.is_cuda:
        return _EmbeddingFn.apply(ids, table, wgrad_buf)
    return torch.nn.functional.embedding(ids, grad_to_buf(table, wgrad_buf))


# --------------------------------------------------------------------------------------- cross-entropy
def cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    lf = logits.float()
    return (torch.logsumexp(lf, -1) - lf.gather(-1, targets[:, None]).squeeze(-1)).mean()


def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Per-row {max, sum exp(x - max), target logit (0 if not in this shard)} -> fp32 [rows, 3]."""
    rows, V = logits.shape
    if _native_ok(logits):
        stats = torch.empty((rows, 3), device=logits.device, dtype=torch.float32)
        check(lib().tsb_ce_stats(logits.data_ptr(), targets.data_ptr(), stats.data_ptr(), rows, V, logits.stride(0),
                                 vocab_start, dtype_code(logits.dtype), stream_ptr(logits.device)), "tsb_ce_stats")
        return stats
    lf = logits.float()
    m = lf.max(-1).values
    s = (lf - m[:, None]).exp().sum(-1)
    loc = targets - vocab_start
    inside = (loc >= 0) & (loc < V)
    tl = torch.where(inside, lf.gather(-1, loc.clamp(0, V - 1)[:, None]).squeeze(-1), torch.zeros_like(m))
    return torch.stack([m, s, tl], dim=-1)


def merge_ce_stats(stats_list: list[torch.Tensor]) -> torch.Tensor:
    """Combine per-shard stats of the same rows (what a vocab-parallel all-reduce computes)."""
    m = torch.stack([s[:, 0] for s in stats_list]).max(0).values
    ssum = sum(s[:, 1] * (s[:, 0] - m).exp() for s in stats_list)
    tl = sum(s[:, 2] for s in stats_list)
    return torch.stack([m, ssum, tl], dim=-1)


def ce_loss_and_grad_(logits: torch.Tensor, targets: torch.Tensor, stats: torch.Tensor, grad_scale: float,
                      vocab_start: int = 0, write_grad: bool = True) -> torch.Tensor:
    """Per-row losses (fp32 [rows]); when ``write_grad`` the logits are overwritten IN PLACE with
    ``(softmax - onehot) * grad_scale``. Rows with a negative target contribute nothing."""
    rows, V = logits.shape
    if _native_ok(logits):
        loss_rows = torch.empty(rows, device=logits.device, dtype=torch.float32)
        check(lib().tsb_ce_loss_grad(logits.data_ptr(), targets.data_ptr(), stats.data_ptr(), loss_rows.data_ptr(),
                                     rows, V, logits.stride(0), vocab_start, float(grad_scale), int(write_grad),
                                     dtype_code(logits.dtype), stream_ptr(logits.device)), "tsb_ce_loss_grad")
        return loss_rows
    m, s, tl = stats[:, 0], stats[:, 1], stats[:, 2]
    ignored = targets < 0
    loss_rows = torch.where(ignored, torch.zeros_like(m), s.log() + m - tl)
    if write_grad:
        p = (logits.float() - m[:, None]).exp() / s[:, None]
        loc = targets - vocab_start
        inside = (loc >= 0) & (loc < V) & ~ignored
        rows_idx = torch.nonzero(inside).squeeze(-1)
        p[rows_idx, loc[rows_idx]] -= 1.0
        p = p * grad_scale
        p[ignored] = 0
        logits.copy_(p.to(logits.dtype))
    return loss_rows


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        work = logits.detach().clone()
        stats = ce_stats(work, targets)
        n = logits.shape[0]
        loss_rows = ce_loss_and_grad_(work, targets, stats, 1.0 / n)
        ctx.save_for_backward(work)
        return loss_rows.sum() / n

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad.float() * g).to(grad.dtype), None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean over rows of ``logsumexp(row) - row[target]``; ``logits`` [N, V], ``targets`` int64 [N]."""
    if logits.dim() != 2 or targets.dim() != 1 or targets.shape[0] != logits.shape[0]:
        raise ValueError("cross_entropy expects logits [N, V] and targets [N]")
    if targets.dtype != torch.int64:
        raise TypeError("cross_entropy: targets must be int64")
    if _native_ok(logits):
        return _CrossEntropyFn.apply(logits.contiguous(), targets.contiguous())
    return cross_entropy_ref(logits, targets)
