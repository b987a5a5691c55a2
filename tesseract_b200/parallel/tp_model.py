"""Tensor-parallel + sequence-parallel Llama for training, one process per GPU.

Every rank holds a 1/tp slice of each projection (query / key / value heads, FFN columns, vocabulary rows of
lm_head) under the SAME parameter names as the dense model (``layers.{i}.attn.q_proj.weight`` ...), so a dense
checkpoint is loaded by slicing (``load_dense_state_dict``, as ``from_dense`` does in
src/distributed/TensorParallel.cpp:116-138,198-215) and saved by gathering (``gather_dense_state_dict``).
Embedding and norm weights are replicated; their gradients (and nothing else) are all-reduced over the
tensor-parallel group once per step (``sync_replicated_grads``).

Activations between sub-layers are token shards [T / tp, D]; attention runs on full sequences for the local heads.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
from torch import nn

from .. import ops
from ..models.llama import LlamaConfig, llama_local_to_hf_name
from ..nn.modules import Embedding, Linear, Module, ModuleList, RMSNorm, RotaryEmbedding, _main_grad, fused_rows_view
from .tp_layers import TPContext, VocabParallelCEFn, column_parallel_sp, row_parallel_sp


def _fused_weight_and_grad(linears: List[Linear]):
    ws = [l.weight for l in linears]
    gs = [_main_grad(w) for w in ws]
    if all(g is not None for g in gs):
        wv, gv = fused_rows_view(ws), fused_rows_view(gs)
        if wv is not None and gv is not None:
            return wv, gv
    return torch.cat([ops.grad_to_buf(w, g) for w, g in zip(ws, gs)], dim=0), None


class TPAttention(Module):
    def __init__(self, c: LlamaConfig, tp: TPContext, rope: RotaryEmbedding, device=None):
        super().__init__()
        H, Hkv, D = c.num_attention_heads, c.kv_heads(), c.head_dim
        if H % tp.size or Hkv % tp.size:
            raise ValueError(f"tensor parallel size {tp.size} must divide the query ({H}) and KV ({Hkv}) head counts")
        self.tp = tp
        self.h_local, self.hkv_local, self.head_dim = H // tp.size, Hkv // tp.size, D
        dm, dt = c.hidden_size, c.dtype
        self.q_proj = Linear(dm, self.h_local * D, bias=False, dtype=dt, device=device)
        self.k_proj = Linear(dm, self.hkv_local * D, bias=False, dtype=dt, device=device)
        self.v_proj = Linear(dm, self.hkv_local * D, bias=False, dtype=dt, device=device)
        self.o_proj = Linear(self.h_local * D, dm, bias=False, dtype=dt, device=device)
        object.__setattr__(self, "rope", rope)

    def forward(self, x_local: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        H, Hkv, D = self.h_local, self.hkv_local, self.head_dim
        w, g = _fused_weight_and_grad([self.q_proj, self.k_proj, self.v_proj])
        qkv = column_parallel_sp(x_local, w, self.tp, g)                       # [T, (H + 2 Hkv) D] full sequence
        qkv = ops.rope_qkv(qkv, self.rope.cos, self.rope.sin, num_heads=H, num_kv_heads=Hkv, head_dim=D, seq_len=seq)
        o = ops.flash_attention_packed(qkv.view(batch, seq, H + 2 * Hkv, D), H, Hkv, causal=True)
        return row_parallel_sp(o.reshape(batch * seq, H * D), self.o_proj.weight, self.tp, _main_grad(self.o_proj.weight))


class TPFeedForward(Module):
    def __init__(self, c: LlamaConfig, tp: TPContext, device=None):
        super().__init__()
        if c.intermediate_size % tp.size:
            raise ValueError("tensor parallel size must divide intermediate_size")
        self.tp = tp
        f = c.intermediate_size // tp.size
        self.gate_proj = Linear(c.hidden_size, f, bias=False, dtype=c.dtype, device=device)
        self.up_proj = Linear(c.hidden_size, f, bias=False, dtype=c.dtype, device=device)
        self.down_proj = Linear(f, c.hidden_size, bias=False, dtype=c.dtype, device=device)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        w, g = _fused_weight_and_grad([self.gate_proj, self.up_proj])
        gu = column_parallel_sp(x_local, w, self.tp, g)
        return row_parallel_sp(ops.swiglu(gu), self.down_proj.weight, self.tp, _main_grad(self.down_proj.weight))


class TPBlock(Module):
    def __init__(self, c: LlamaConfig, tp: TPContext, rope, device=None):
        super().__init__()
        self.norm_1 = RMSNorm(c.hidden_size, c.rms_norm_eps, c.dtype, device)
        self.attn = TPAttention(c, tp, rope, device)
        self.norm_2 = RMSNorm(c.hidden_size, c.rms_norm_eps, c.dtype, device)
        self.ffn = TPFeedForward(c, tp, device)

    def forward(self, x, res, batch, seq):
        if res is None:
            h, res = self.norm_1(x), x
        else:
            h, res = self.norm_1(x, res)
        a = self.attn(h, batch, seq)
        h2, res = self.norm_2(a, res)
        return self.ffn(h2), res


class TPLlamaModel(Module):
    def __init__(self, config: LlamaConfig, tp: TPContext, device=None, init_std: Optional[float] = None, seed: int = 0):
        super().__init__()
        c = config
        if c.vocab_size % tp.size:
            raise ValueError("tensor parallel size must divide vocab_size")
        self.config, self.tp = c, tp
        self.rope = RotaryEmbedding(c.head_dim, c.max_position_embeddings, c.rope_theta, device)
        self.embed_tokens = Embedding(c.vocab_size, c.hidden_size, dtype=c.dtype, device=device)
        self.layers = ModuleList([TPBlock(c, tp, self.rope, device) for _ in range(c.num_hidden_layers)])
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, c.dtype, device)
        self.lm_head = Linear(c.hidden_size, c.vocab_size // tp.size, bias=False, dtype=c.dtype, device=device)
        if init_std is not None:
            self.init_weights(init_std, seed)

    # ------------------------------------------------------------------ initialisation / checkpoints
    def replicated_parameters(self):
        """Parameters that every rank holds in full (their gradients are partial sums over token shards)."""
        out = [self.embed_tokens.weight, self.norm.weight]
        for blk in self.layers:
            out += [blk.norm_1.weight, blk.norm_2.weight]
        return out

    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        """N(0, std): replicated tensors from the same stream on every rank, shards from a rank-specific stream."""
        dev = self.embed_tokens.weight.device
        shared = torch.Generator(device=dev).manual_seed(seed)
        own = torch.Generator(device=dev).manual_seed(seed * 1000003 + 17 + self.tp.rank)
        rep = {id(p) for p in self.replicated_parameters()}
        with torch.no_grad():
            for _, p in self.named_parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, std, generator=shared if id(p) in rep else own)

    def _shard_of(self, name: str, full: torch.Tensor) -> torch.Tensor:
        r, n = self.tp.rank, self.tp.size
        if name.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")) \
                or name == "lm_head.weight":
            k = full.shape[0] // n
            return full[r * k:(r + 1) * k]
        if name.endswith(("o_proj.weight", "down_proj.weight")):
            k = full.shape[1] // n
            return full[:, r * k:(r + 1) * k]
        return full

    def load_dense_state_dict(self, sd: Dict[str, torch.Tensor], hf_names: bool = True) -> None:
        with torch.no_grad():
            for name, p in self.named_parameters():
                key = llama_local_to_hf_name(name) if hf_names else name
                if key not in sd:
                    raise KeyError(f"load: required tensor {key!r} is missing")
                p.copy_(self._shard_of(name, sd[key]).to(device=p.device, dtype=p.dtype))

    def gather_dense_state_dict(self, hf_names: bool = True) -> Dict[str, torch.Tensor]:
        """All ranks call this; every rank receives the full (dense) tensors."""
        import torch.distributed as dist
        out = {}
        n = self.tp.size
        for name, p in self.named_parameters():
            key = llama_local_to_hf_name(name) if hf_names else name
            sharded = name.endswith("_proj.weight") or name == "lm_head.weight"
            if n == 1 or not sharded:
                out[key] = p.detach().clone()
                continue
            parts = [torch.empty_like(p) for _ in range(n)]
            dist.all_gather(parts, p.detach().contiguous(), group=self.tp.group)
            dim = 1 if name.endswith(("o_proj.weight", "down_proj.weight")) else 0
            out[key] = torch.cat(parts, dim=dim)
        return out

    # ------------------------------------------------------------------ forward / loss
    def _local_rows(self, flat: torch.Tensor) -> torch.Tensor:
        T = flat.shape[0]
        if T % self.tp.size:
            raise ValueError(f"token count {T} is not divisible by the tensor-parallel size {self.tp.size}")
        n = T // self.tp.size
        return flat[self.tp.rank * n:(self.tp.rank + 1) * n]

    def hidden_states_local(self, tokens: torch.Tensor) -> torch.Tensor:
        B, S = tokens.shape
        ids_local = self._local_rows(tokens.reshape(-1)).contiguous()
        x = self.embed_tokens(ids_local)                      # [T / tp, D]: sequence-parallel from the start
        res = None
        red = getattr(self, "grad_reducer", None)
        for li, blk in enumerate(self.layers):
            if red is not None:
                x = red.mark(x, red.block_bucket0 + li)
                if res is not None:
                    res = red.mark(res, red.block_bucket0 + li)
            x, res = blk(x, res, B, S)
        if red is not None:
            tail = red.tail_buckets(len(self.layers))
            if tail:
                x = red.mark(x, tail)
        if res is None:
            return self.norm(x)
        h, _ = self.norm(x, res)
        return h

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, chunk_rows: int = 8192, loss_scale: float = 1.0,
             total_rows: int = 0) -> torch.Tensor:
        h_local = self.hidden_states_local(tokens)
        w = self.lm_head.weight
        return VocabParallelCEFn.apply(h_local, w, targets.reshape(-1).contiguous(), _main_grad(w), self.tp, chunk_rows,
                                       float(loss_scale))

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the tensor-parallel group (one flat all-reduce)."""
        if self.tp.size == 1:
            return
        grads = []
        for p in self.replicated_parameters():
            g = _main_grad(p)
            if g is None:
                g = p.grad
            if g is not None:
                grads.append(g)
        if not grads:
            return
        small = [g for g in grads if g.numel() < (1 << 20)]
        for g in grads:
            if g.numel() >= (1 << 20):
                self.tp.all_reduce_(g)                       # in place, in the gradient's own dtype
        if small:
            flat = torch.cat([g.reshape(-1).float() for g in small])
            self.tp.all_reduce_(flat)
            off = 0
            for g in small:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g).to(g.dtype))
                off += n
