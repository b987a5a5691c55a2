"""Core layers: Linear, Embedding, RMSNorm, LayerNorm, RotaryEmbedding, MultiHeadAttention (GQA + RoPE),
FeedForward (SwiGLU), TransformerBlock, containers and activation wrappers.

Class names, constructor arguments and parameter names follow the reference's ``nn`` namespace
(include/tesseract/nn/*.hpp; parameter naming rules in src/nn/Module.cpp:32-137) so that
``named_parameters()`` of a model yields the same dotted keys: ``attn.{q,k,v,o}_proj.weight``,
``ffn.{gate,up,down}_proj.weight``, ``norm_1.weight`` ... The projections are separate parameters (as in
the reference) but, when a model packs its parameters into one arena, q/k/v and gate/up sit next to
each other in memory and the layer runs them as ONE GEMM over the fused view.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .. import ops


def _main_grad(p: torch.Tensor) -> Optional[torch.Tensor]:
    return getattr(p, "main_grad", None)


class Module(nn.Module):
    """torch.nn.Module plus the few reference-API conveniences (``replace_module``)."""

    def replace_module(self, name: str, new: nn.Module) -> None:
        """Swap a registered child, keeping its slot name (src/nn/Module.cpp `replace_module`)."""
        if name not in self._modules:
            raise KeyError(f"no child module named {name!r}")
        self._modules[name] = new


class Linear(Module):
    """y = x W^T (+ b); ``weight`` is [out, in], init U(-1/sqrt(in), 1/sqrt(in)) (src/nn/Linear.cpp:43-83)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=torch.float32, device=None):
        super().__init__()
        if in_features <= 0 or out_features <= 0:
            raise ValueError("Linear: feature counts must be positive")
        self.in_features, self.out_features = in_features, out_features
        bound = 1.0 / math.sqrt(in_features)
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device).uniform_(-bound, bound))
        self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype, device=device).uniform_(-bound, bound)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Linear: expected last dimension {self.in_features}, got {x.shape[-1]}")
        return ops.linear(x, self.weight, self.bias, _main_grad(self.weight))

    @classmethod
    def from_weight(cls, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "Linear":
        m = cls.__new__(cls)
        Module.__init__(m)
        m.out_features, m.in_features = weight.shape
        m.weight = nn.Parameter(weight)
        m.bias = nn.Parameter(bias) if bias is not None else None
        return m


class Embedding(Module):
    """Row lookup with int64 ids; N(0,1) init (src/nn/Embedding.cpp:64-85)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, dtype=torch.float32, device=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.randn(num_embeddings, embedding_dim, dtype=dtype, device=device))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids, self.weight, _main_grad(self.weight))


class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.float32, device=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        return ops.rms_norm(x, self.weight, self.eps, residual, _main_grad(self.weight))


class LayerNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.float32, device=None):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        return torch.nn.functional.layer_norm(x, (self.dim,), self.weight, self.bias, self.eps)


class BatchNorm1d(nn.BatchNorm1d):
    pass


class BatchNorm2d(nn.BatchNorm2d):
    pass


class ReLU(nn.ReLU):
    pass


class Sigmoid(nn.Sigmoid):
    pass


class Tanh(nn.Tanh):
    pass


class CrossEntropyLoss(Module):
    def forward(self, logits, targets):
        return ops.cross_entropy(logits, targets)


class Sequential(nn.Sequential):
    """Accepts a list like the reference binding (``Sequential([a, b])``) and has ``add``."""

    def __init__(self, *mods):
        if len(mods) == 1 and isinstance(mods[0], (list, tuple)):
            mods = tuple(mods[0])
        super().__init__(*mods)

    def add(self, m: nn.Module) -> "Sequential":
        self.append(m)
        return self


class ModuleList(nn.ModuleList):
    pass


class DiTBlock(Module):
    """Placeholder, as in the reference (include/tesseract/nn/DiTBlock.hpp:46-58): constructing is allowed,
    running is not implemented."""

    def forward(self, *a, **k):
        raise NotImplementedError("DiTBlock is a placeholder in the reference and here")


class RotaryEmbedding(Module):
    """Adjacent-pair RoPE with cos/sin tables [max_seq, head_dim/2] (fp32 buffers). One instance is
    shared by every attention layer of a model (the reference keeps one pair per layer,
    src/nn/RotaryEmbedding.cpp:66-88)."""

    def __init__(self, head_dim: int, max_seq_len: int, theta: float = 10000.0, device=None):
        super().__init__()
        if head_dim % 2:
            raise ValueError("RotaryEmbedding: head_dim must be even")
        self.head_dim, self.max_seq_len, self.theta = head_dim, max_seq_len, theta
        cos, sin = ops.rope_tables(max_seq_len, head_dim, theta, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, x: torch.Tensor, pos: int = 0) -> torch.Tensor:
        """x [B, H, S, D] -> rotated, positions pos .. pos+S-1 (``forward_offset`` of the reference)."""
        S = x.shape[-2]
        if pos + S > self.max_seq_len:
            raise ValueError("RotaryEmbedding: position beyond max_seq_len")
        positions = torch.arange(pos, pos + S, device=x.device)
        return ops.rope_ref(x.transpose(1, 2), self.cos, self.sin, positions).transpose(1, 2)

    forward_offset = forward


def _adjacent(views: list[torch.Tensor]) -> bool:
    """True when the tensors are contiguous row blocks laid back to back in one allocation."""
    for a, b in zip(views[:-1], views[1:]):
        if not (a.is_contiguous() and b.is_contiguous()):
            return False
        if a.data_ptr() + a.numel() * a.element_size() != b.data_ptr():
            return False
        if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
            return False
    return True


def fused_rows_view(params: list[torch.Tensor]) -> Optional[torch.Tensor]:
    """One [sum(rows), in] view over row-stacked parameters that sit back to back in an arena, else None."""
    datas = [p.data for p in params]
    if not _adjacent(datas) or len({d.shape[1] for d in datas}) != 1:
        return None
    first = datas[0]
    rows = sum(d.shape[0] for d in datas)
    return torch.as_strided(first, (rows, first.shape[1]), (first.shape[1], 1), first.storage_offset())


class _FusedProj:
    """Runs several row-stacked Linear weights as one GEMM (fused view when available, else a cat)."""

    @staticmethod
    def run(x: torch.Tensor, linears: list[Linear]) -> torch.Tensor:
        ws = [l.weight for l in linears]
        grads = [_main_grad(w) for w in ws]
        if all(g is not None for g in grads):
            wv = fused_rows_view(ws)
            gv = fused_rows_view(grads) if wv is not None else None
            if wv is not None and gv is not None:
                need = torch.is_grad_enabled() and any(w.requires_grad for w in ws)
                return ops.linear(x, wv, None, gv, force_wgrad=need)
        need_grad = torch.is_grad_enabled() and any(w.requires_grad for w in ws)
        if not need_grad:
            # inference: weights that already sit back to back (an arena, or an engine that fused them in place) are one
            # GEMM over a view; nothing is copied
            wv = fused_rows_view(ws)
            if wv is not None:
                return ops.linear(x, wv)
            if not x.is_cuda:
                # separate weights on the CPU: three products and a cat of the (small) outputs, instead of copying all
                # the weights into one matrix for every call
                return torch.cat([ops.linear(x, w) for w in ws], dim=-1)
        w = torch.cat([ops.grad_to_buf(w, g) for w, g in zip(ws, grads)], dim=0)
        return ops.linear(x, w)


class MultiHeadAttention(Module):
    """Multi-head attention with grouped-query KV heads and RoPE.

    Separate ``q_proj/k_proj/v_proj/o_proj`` Linear children without bias (k/v out = Hkv * Dh), GQA head
    map h -> h // (H / Hkv), K rotated before caching (src/nn/MultiHeadAttention.cpp:79-165,234-363).
    ``forward`` is the training / full-sequence path: one fused QKV GEMM, in-place RoPE on the packed
    buffer, FlashAttention (BSHD, causal), output projection.
    """

    def __init__(self, d_model: int, num_heads: int, num_kv_heads: int = 0, max_seq_len: int = 2048,
                 rope_theta: float = 10000.0, dtype=torch.float32, device=None, rope: Optional[RotaryEmbedding] = None,
                 causal: bool = True):
        super().__init__()
        if d_model % num_heads:
            raise ValueError("MultiHeadAttention: d_model must be divisible by num_heads")
        self.d_model, self.num_heads = d_model, num_heads
        self.num_kv_heads = num_kv_heads if num_kv_heads > 0 else num_heads
        if num_heads % self.num_kv_heads:
            raise ValueError("MultiHeadAttention: num_kv_heads must divide num_heads")
        self.head_dim = d_model // num_heads
        self.causal = causal
        kv_out = self.num_kv_heads * self.head_dim
        self.q_proj = Linear(d_model, d_model, bias=False, dtype=dtype, device=device)
        self.k_proj = Linear(d_model, kv_out, bias=False, dtype=dtype, device=device)
        self.v_proj = Linear(d_model, kv_out, bias=False, dtype=dtype, device=device)
        self.o_proj = Linear(d_model, d_model, bias=False, dtype=dtype, device=device)
        # The rotary table is shared; keep it out of the child registry when it is not owned here.
        if rope is None:
            self.rope = RotaryEmbedding(self.head_dim, max_seq_len, rope_theta, device)
        else:
            object.__setattr__(self, "rope", rope)

    def qkv(self, x2: torch.Tensor) -> torch.Tensor:
        projs = [self.q_proj, self.k_proj, self.v_proj]
        if all(isinstance(p, Linear) for p in projs):
            return _FusedProj.run(x2, projs)
        return torch.cat([p(x2) for p in projs], dim=-1)   # quantised projections

    def forward(self, x: torch.Tensor, pos: int = 0) -> torch.Tensor:
        B, S, Dm = x.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv(x.reshape(B * S, Dm))
        qkv = ops.rope_qkv(qkv, self.rope.cos, self.rope.sin, num_heads=H, num_kv_heads=Hkv, head_dim=D, seq_len=S,
                           pos_offset=pos)
        qkv = qkv.view(B, S, H + 2 * Hkv, D)
        o = ops.flash_attention_packed(qkv, H, Hkv, causal=self.causal)
        return self.o_proj(o.reshape(B, S, H * D))


    # ------------------------------------------------------------------ incremental decode
    def _project_step(self, x: torch.Tensor, positions: torch.Tensor):
        """x [T, Dm], positions [T] -> rotated q [T, H, D], rotated k [T, Hkv, D], v [T, Hkv, D]."""
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self.qkv(x)
        qkv = ops.rope_qkv(qkv, self.rope.cos, self.rope.sin, num_heads=H, num_kv_heads=Hkv, head_dim=D,
                           seq_len=1, positions=positions)
        qkv = qkv.view(-1, H + 2 * Hkv, D)
        return qkv[:, :H], qkv[:, H:H + Hkv], qkv[:, H + Hkv:]

    @torch.no_grad()
    def forward_step(self, x: torch.Tensor, cache) -> torch.Tensor:
        """x [B, S_new, Dm]: project, rotate at positions cache.current_len() .., append K/V to ``cache`` and
        attend over the whole prefix (src/nn/MultiHeadAttention.cpp:234-363). S_new == 1 is decode,
        S_new > 1 on an empty cache is prefill, anything else is chunked prefill (last query sees all keys)."""
        B, Sn, Dm = x.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        pos = cache.current_len()
        if pos + Sn > self.rope.max_seq_len:
            raise ValueError("forward_step: position beyond the rotary table")
        positions = (pos + torch.arange(Sn, device=x.device)).repeat(B)
        q, k, v = self._project_step(x.reshape(B * Sn, Dm), positions)
        q = q.reshape(B, Sn, H, D)
        k = k.reshape(B, Sn, Hkv, D).transpose(1, 2)
        v = v.reshape(B, Sn, Hkv, D).transpose(1, 2)
        cache.append(k.contiguous(), v.contiguous())
        keys, vals = cache.keys_view(), cache.values_view()          # [B, Hkv, L, D]
        o = ops.flash_attention(q, keys.transpose(1, 2), vals.transpose(1, 2), causal=Sn > 1)
        return self.o_proj(o.reshape(B, Sn, H * D))

    @torch.no_grad()
    def forward_step_batched(self, x: torch.Tensor, caches: list) -> torch.Tensor:
        """x [A, S_new, Dm] with one (batch-1) cache per sequence, each possibly at a different length.
        Projections run once over all A * S_new rows; attention threads every sequence through its own
        cache, or runs as ONE ragged kernel when all caches are paged views of the same pool
        (src/nn/MultiHeadAttention.cpp:365-649)."""
        from .kv_cache import PagedKVCache
        A, Sn, Dm = x.shape
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        if len(caches) != A:
            raise ValueError("forward_step_batched: one cache per sequence is required")
        starts = [c.current_len() for c in caches]
        positions = torch.cat([s + torch.arange(Sn) for s in starts]).to(x.device)
        q, k, v = self._project_step(x.reshape(A * Sn, Dm), positions)
        q = q.reshape(A, Sn, H, D)
        k = k.reshape(A, Sn, Hkv, D).transpose(1, 2)
        v = v.reshape(A, Sn, Hkv, D).transpose(1, 2)
        for a, c in enumerate(caches):
            c.append(k[a:a + 1].contiguous(), v[a:a + 1].contiguous())
        same_pool = all(isinstance(c, PagedKVCache) for c in caches) and len({id(c.pool) for c in caches}) == 1
        if same_pool:
            pool = caches[0].pool
            max_blocks = max(len(c.block_table) for c in caches)
            tables = torch.zeros((A, max_blocks), dtype=torch.int32)
            for a, c in enumerate(caches):
                tables[a, :len(c.block_table)] = torch.tensor(c.block_table, dtype=torch.int32)
            tables = tables.to(x.device)
            lens = torch.tensor([c.current_len() for c in caches], dtype=torch.int32, device=x.device)
            ks = getattr(pool, "k_scale", None)
            vs = getattr(pool, "v_scale", None)
            if Sn == 1:
                o = ops.paged_decode_attention(q[:, 0].contiguous(), pool.k, pool.v, tables, lens, None, ks, vs).unsqueeze(1)
            else:
                o = ops.paged_prefill_attention(q, pool.k, pool.v, tables, lens, None, ks, vs)
        else:
            outs = []
            for a, c in enumerate(caches):
                keys, vals = c.keys_view(), c.values_view()
                outs.append(ops.flash_attention(q[a:a + 1], keys.transpose(1, 2), vals.transpose(1, 2), causal=Sn > 1))
            o = torch.cat(outs, dim=0)
        return self.o_proj(o.reshape(A, Sn, H * D))

    def quantize_(self, scheme) -> None:
        """Swap the four projections for their weight-only quantised variants (src/nn/MultiHeadAttention.cpp:651-673)."""
        from ..quant import quantize_linear
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            self.replace_module(name, quantize_linear(getattr(self, name), scheme))


class FeedForward(Module):
    """SwiGLU MLP ``down(silu(gate(x)) * up(x))`` (src/nn/FeedForward.cpp:11-72); gate and up run as one GEMM."""

    def __init__(self, d_model: int, d_ff: int, dtype=torch.float32, device=None):
        super().__init__()
        self.d_model, self.d_ff = d_model, d_ff
        self.gate_proj = Linear(d_model, d_ff, bias=False, dtype=dtype, device=device)
        self.up_proj = Linear(d_model, d_ff, bias=False, dtype=dtype, device=device)
        self.down_proj = Linear(d_ff, d_model, bias=False, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if isinstance(self.gate_proj, Linear) and isinstance(self.up_proj, Linear):
            gu = _FusedProj.run(x2, [self.gate_proj, self.up_proj])
        else:
            gu = torch.cat([self.gate_proj(x2), self.up_proj(x2)], dim=-1)
        return self.down_proj(ops.swiglu(gu)).view(shape)

    def quantize_(self, scheme) -> None:
        from ..quant import quantize_linear
        for name in ("gate_proj", "up_proj", "down_proj"):
            self.replace_module(name, quantize_linear(getattr(self, name), scheme))


class TransformerBlock(Module):
    """Pre-norm block: h = x + attn(norm_1(x)); out = h + ffn(norm_2(h)) (src/nn/TransformerBlock.cpp:53-67).

    ``forward(x, residual)`` carries the residual stream separately so that each residual add is fused
    into the following RMSNorm kernel: it returns ``(branch_output, residual_stream)`` and the caller
    (the model) folds the last pair with the final norm.
    """

    def __init__(self, d_model: int, num_heads: int, d_ff: int, num_kv_heads: int = 0, max_seq_len: int = 2048,
                 rope_theta: float = 10000.0, eps: float = 1e-5, dtype=torch.float32, device=None,
                 rope: Optional[RotaryEmbedding] = None, ffn: Optional[nn.Module] = None):
        super().__init__()
        self.norm_1 = RMSNorm(d_model, eps, dtype, device)
        self.attn = MultiHeadAttention(d_model, num_heads, num_kv_heads, max_seq_len, rope_theta, dtype, device, rope)
        self.norm_2 = RMSNorm(d_model, eps, dtype, device)
        self.ffn = ffn if ffn is not None else FeedForward(d_model, d_ff, dtype, device)

    def forward_fused(self, x: torch.Tensor, residual: Optional[torch.Tensor]):
        if residual is None:
            h, res = self.norm_1(x), x
        else:
            h, res = self.norm_1(x, residual)
        a = self.attn(h)
        h2, res = self.norm_2(a, res)
        return self.ffn(h2), res

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out, res = self.forward_fused(x, None)
        return out + res

    @torch.no_grad()
    def forward_step(self, x: torch.Tensor, cache) -> torch.Tensor:
        h = x + self.attn.forward_step(self.norm_1(x), cache)
        return h + self.ffn(self.norm_2(h))

    @torch.no_grad()
    def forward_step_batched(self, x: torch.Tensor, caches: list) -> torch.Tensor:
        h = x + self.attn.forward_step_batched(self.norm_1(x), caches)
        return h + self.ffn(self.norm_2(h))
