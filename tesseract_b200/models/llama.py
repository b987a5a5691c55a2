"""Llama-family decoder: config, model, fused training loss, weight I/O by Hugging Face key names.

Structure and naming follow the reference model (include/tesseract/models/Llama.hpp:27-88,
src/models/Llama.cpp:205-226,293-308): ``embed_tokens -> N x TransformerBlock -> norm -> lm_head`` with
parameters ``embed_tokens.weight``, ``layers.{i}.norm_1.weight``, ``layers.{i}.attn.{q,k,v,o}_proj.weight``,
``layers.{i}.norm_2.weight``, ``layers.{i}.ffn.{gate,up,down}_proj.weight`` (or the MoE names),
``norm.weight``, ``lm_head.weight``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from typing import Optional

import torch
from torch import nn

from .. import ops
from ..nn.modules import (Embedding, FeedForward, Linear, Module, ModuleList, RMSNorm, RotaryEmbedding,
                          TransformerBlock, _main_grad)
from ..ops.gemm import gemm_bf16

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
           "float64": torch.float64}


@dataclass
class LlamaConfig:
    """Hyper-parameters with Hugging Face field names (include/tesseract/models/Llama.hpp:27-62)."""

    vocab_size: int = 32000
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 0          # 0 => equals num_attention_heads
    intermediate_size: int = 11008
    num_experts: int = 0                   # 0 => dense SwiGLU FFN
    num_experts_per_tok: int = 0
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    dtype: torch.dtype = torch.float32
    bos_token_id: int = -1
    eos_token_id: int = -1

    def kv_heads(self) -> int:
        return self.num_key_value_heads if self.num_key_value_heads > 0 else self.num_attention_heads

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @staticmethod
    def llama_3_2_1b() -> "LlamaConfig":
        return LlamaConfig(vocab_size=128256, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                           num_key_value_heads=8, intermediate_size=8192, max_position_embeddings=131072,
                           rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                           bos_token_id=128000, eos_token_id=128001)

    @staticmethod
    def llama_3_8b(dtype: torch.dtype = torch.bfloat16, max_position_embeddings: int = 8192) -> "LlamaConfig":
        return LlamaConfig(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                           num_key_value_heads=8, intermediate_size=14336,
                           max_position_embeddings=max_position_embeddings, rope_theta=500000.0,
                           rms_norm_eps=1e-5, dtype=dtype, bos_token_id=128000, eos_token_id=128001)

    @staticmethod
    def from_json(text: str) -> "LlamaConfig":
        """Parse a Hugging Face ``config.json``; missing fields keep their defaults
        (src/models/Llama.cpp:38-188). ``num_local_experts`` is accepted for ``num_experts``."""
        try:
            obj = json.loads(text)
        except json.JSONDecodeError as e:
            raise ValueError(f"LlamaConfig.from_json: malformed JSON ({e})") from None
        if not isinstance(obj, dict):
            raise ValueError("LlamaConfig.from_json: top-level JSON value must be an object")
        cfg = LlamaConfig()
        names = {f.name for f in fields(LlamaConfig)}
        for k, v in obj.items():
            if k == "torch_dtype" and isinstance(v, str) and v in _DTYPES:
                cfg.dtype = _DTYPES[v]
            elif k == "num_local_experts" and isinstance(v, int):
                cfg.num_experts = v
            elif k == "eos_token_id" and isinstance(v, list) and v:
                cfg.eos_token_id = int(v[0])
            elif k in names and k != "dtype" and isinstance(v, (int, float, bool)):
                cur = getattr(cfg, k)
                setattr(cfg, k, type(cur)(v))
        return cfg

    @staticmethod
    def from_json_file(path: str) -> "LlamaConfig":
        try:
            with open(path, "r", encoding="utf-8") as f:
                return LlamaConfig.from_json(f.read())
        except OSError as e:
            raise ValueError(f"LlamaConfig.from_json_file: cannot read {path}: {e}") from None


def llama_local_to_hf_name(name: str) -> str:
    """Local parameter name -> Hugging Face key (src/models/Llama.cpp:205-226)."""
    if name == "lm_head.weight":
        return name
    out = "model." + name
    return (out.replace(".attn.", ".self_attn.").replace(".ffn.", ".mlp.")
            .replace(".norm_1.", ".input_layernorm.").replace(".norm_2.", ".post_attention_layernorm."))


class _FusedLMHeadCE(torch.autograd.Function):
    """loss = mean CE(h @ W^T, targets) without ever holding the full [T, V] logits.

    Runs over chunks of rows: logits chunk (GEMM) -> per-row stats -> loss and, in place, the logits
    gradient -> dh chunk (GEMM) and dW += (GEMM). The gradient with respect to ``h`` is kept for the
    backward pass; dW goes straight into ``wgrad_buf``. ``loss_scale`` multiplies the gradients (1 /
    number of micro-batches under gradient accumulation).
    """

    @staticmethod
    def forward(ctx, h, weight, targets, wgrad_buf, chunk_rows, loss_scale, total_rows):
        T, D = h.shape
        V = weight.shape[0]
        n_total = total_rows if total_rows else T
        dh = torch.empty_like(h)
        loss_sum = torch.zeros((), device=h.device, dtype=torch.float32)
        need_grad = wgrad_buf is not None or weight.requires_grad or h.requires_grad
        dw_local = None
        if need_grad and wgrad_buf is None:
            dw_local = torch.zeros_like(weight, dtype=torch.float32)
        native = h.is_cuda and h.dtype == torch.bfloat16
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            hc, tc = h[r0:r1], targets[r0:r1]
            logits = gemm_bf16(hc, weight) if native else (hc @ weight.t())
            stats = ops.ce_stats(logits, tc)
            loss_rows = ops.ce_loss_and_grad_(logits, tc, stats, loss_scale / n_total, write_grad=need_grad)
            loss_sum += loss_rows.sum()
            if need_grad:
                if native:
                    gemm_bf16(logits, weight, b_mn=True, out=dh[r0:r1])
                    tgt = wgrad_buf if wgrad_buf is not None else dw_local
                    gemm_bf16(logits, hc, a_mn=True, b_mn=True, out=tgt, accumulate=True)
                else:
                    dh[r0:r1] = (logits @ weight).to(dh.dtype)
                    upd = logits.t().float() @ hc.float()
                    if wgrad_buf is not None:
                        wgrad_buf.add_(upd.to(wgrad_buf.dtype))
                    else:
                        dw_local.add_(upd)
            del logits
        ctx.save_for_backward(dh)
        ctx.dw_local = dw_local
        ctx.wdtype = weight.dtype
        return loss_sum / n_total

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        dw = ctx.dw_local.to(ctx.wdtype) * g if ctx.dw_local is not None else None
        # The gradients were formed for an upstream gradient of 1 (times loss_scale).
        return dh * g.to(dh.dtype), dw, None, None, None, None, None


@dataclass
class GenerateConfig:
    """include/tesseract/models/Llama.hpp `GenerateConfig`."""

    max_new_tokens: int = 32
    eos_token_id: int = -1
    do_sample: bool = False
    sampling: "SamplingParams" = None
    seed: int = 0
    kv_int8: bool = False

    def __post_init__(self):
        if self.sampling is None:
            from .sampler import SamplingParams
            self.sampling = SamplingParams()


def pick_next_token(logits_row: torch.Tensor, sampler, history) -> int:
    """Greedy argmax (lowest index on ties) or a draw from ``sampler`` on the host copy of one logits row."""
    if sampler is None:
        return int(torch.argmax(logits_row.float()).item())
    return sampler.sample(logits_row.float().cpu().numpy(), history)


class LlamaModel(Module):
    def __init__(self, config: LlamaConfig, device=None, init_std: Optional[float] = None, seed: int = 0):
        super().__init__()
        c = config
        if c.hidden_size % c.num_attention_heads:
            raise ValueError("LlamaConfig: hidden_size must be divisible by num_attention_heads")
        if c.num_attention_heads % c.kv_heads():
            raise ValueError("LlamaConfig: num_key_value_heads must divide num_attention_heads")
        self.config = c
        dt = c.dtype
        self.rope = RotaryEmbedding(c.head_dim, c.max_position_embeddings, c.rope_theta, device)
        self.embed_tokens = Embedding(c.vocab_size, c.hidden_size, dtype=dt, device=device)
        blocks = []
        for _ in range(c.num_hidden_layers):
            ffn = None
            if c.num_experts > 0:
                from ..nn.moe import MoEFeedForward
                ffn = MoEFeedForward(c.hidden_size, c.intermediate_size, c.num_experts, c.num_experts_per_tok,
                                     dtype=dt, device=device)
            blocks.append(TransformerBlock(c.hidden_size, c.num_attention_heads, c.intermediate_size, c.kv_heads(),
                                           c.max_position_embeddings, c.rope_theta, c.rms_norm_eps, dt, device,
                                           rope=self.rope, ffn=ffn))
        self.layers = ModuleList(blocks)
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, dt, device)
        self.lm_head = Linear(c.hidden_size, c.vocab_size, bias=False, dtype=dt, device=device)
        if init_std is not None:
            self.init_weights(init_std, seed)
        if c.tie_word_embeddings:
            with torch.no_grad():
                self.lm_head.weight.copy_(self.embed_tokens.weight)

    # the shared rotary table is a child (buffers move with .to()) but owns no parameters
    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        """N(0, std) for every matrix from a fixed seed; norm weights stay 1."""
        dev = self.embed_tokens.weight.device
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, std, generator=gen)

    def num_layers(self) -> int:
        return len(self.layers)

    def hidden_states(self, tokens: torch.Tensor) -> torch.Tensor:
        """Token ids [B, S] (int64) -> final-norm hidden states [B, S, D]."""
        if tokens.dim() != 2:
            raise ValueError("LlamaModel: tokens must be [batch, seq]")
        if tokens.shape[1] > self.config.max_position_embeddings:
            raise ValueError("LlamaModel: sequence longer than max_position_embeddings")
        x = self.embed_tokens(tokens)
        res = None
        red = getattr(self, "grad_reducer", None)
        for li, blk in enumerate(self.layers):
            if red is not None:
                # fires (in backward) once this block's weight gradients are complete
                x = red.mark(x, red.block_bucket0 + li)
                if res is not None:
                    res = red.mark(res, red.block_bucket0 + li)
            x, res = blk.forward_fused(x, res)
        if red is not None:
            tail = red.tail_buckets(len(self.layers))
            if tail:
                x = red.mark(x, tail)
        if res is None:
            return self.norm(x)
        h, _ = self.norm(x, res)
        return h

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """Logits [B, S, V]."""
        return self.lm_head(self.hidden_states(tokens))

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, chunk_rows: int = 4096, loss_scale: float = 1.0,
             total_rows: int = 0) -> torch.Tensor:
        """Mean next-token cross-entropy of ``targets`` [B, S] given ``tokens`` [B, S], through the fused
        lm_head + cross-entropy path (no [B*S, V] logits tensor is kept)."""
        h = self.hidden_states(tokens)
        h2 = h.reshape(-1, h.shape[-1])
        w = self.lm_head.weight
        return _FusedLMHeadCE.apply(h2, w, targets.reshape(-1), _main_grad(w), chunk_rows, float(loss_scale),
                                    int(total_rows))

    # ------------------------------------------------------------------ incremental decode
    def _device(self):
        return self.embed_tokens.weight.device

    @torch.no_grad()
    def forward_step(self, tokens: torch.Tensor, caches: list) -> torch.Tensor:
        """tokens [B, S_new] (int64) through one cache per layer -> logits [B, S_new, V]. Inference only
        (src/models/Llama.cpp:352-375)."""
        if len(caches) != len(self.layers):
            raise ValueError(f"forward_step needs {len(self.layers)} caches, got {len(caches)}")
        x = self.embed_tokens(tokens)
        for blk, cache in zip(self.layers, caches):
            x = blk.forward_step(x, cache)
        return self.lm_head(self.norm(x))

    @torch.no_grad()
    def forward_step_batched(self, tokens: torch.Tensor, caches: list) -> torch.Tensor:
        """tokens [A, S_new]; ``caches[sequence][layer]`` -- A independent sequences, each with its own
        per-layer (batch 1) caches at its own length (src/models/Llama.cpp:377-415)."""
        A = tokens.shape[0]
        if len(caches) != A or any(len(c) != len(self.layers) for c in caches):
            raise ValueError("forward_step_batched: caches must be indexed [sequence][layer]")
        x = self.embed_tokens(tokens)
        for li, blk in enumerate(self.layers):
            x = blk.forward_step_batched(x, [caches[a][li] for a in range(A)])
        return self.lm_head(self.norm(x))

    # cache factories (src/models/Llama.cpp:417-475)
    def make_kv_caches(self, batch: int, max_len: int) -> list:
        from ..nn.kv_cache import KVCache
        c = self.config
        return [KVCache(batch, c.kv_heads(), max_len, c.head_dim, c.dtype, self._device()) for _ in self.layers]

    def make_quantized_kv_caches(self, batch: int, max_len: int) -> list:
        from ..nn.kv_cache import QuantizedKVCache
        c = self.config
        return [QuantizedKVCache(batch, c.kv_heads(), max_len, c.head_dim, c.dtype, self._device()) for _ in self.layers]

    def make_layer_pools(self, num_blocks: int, block_size: int) -> list:
        from ..nn.kv_cache import PagedKVPool
        c = self.config
        return [PagedKVPool(num_blocks, c.kv_heads(), block_size, c.head_dim, c.dtype, self._device()) for _ in self.layers]

    def make_paged_kv_caches(self, pools: list, max_len: int) -> list:
        from ..nn.kv_cache import PagedKVCache
        return [PagedKVCache(p, max_len) for p in pools]

    def make_quantized_layer_pools(self, num_blocks: int, block_size: int) -> list:
        from ..nn.kv_cache import QuantizedPagedKVPool
        c = self.config
        return [QuantizedPagedKVPool(num_blocks, c.kv_heads(), block_size, c.head_dim, c.dtype, self._device())
                for _ in self.layers]

    def make_quantized_paged_kv_caches(self, pools: list, max_len: int) -> list:
        from ..nn.kv_cache import QuantizedPagedKVCache
        return [QuantizedPagedKVCache(p, max_len) for p in pools]

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompt_ids, cfg: Optional["GenerateConfig"] = None) -> list:
        """Prefill ``prompt_ids`` then decode token by token until ``max_new_tokens`` or EOS (appended, then
        stop). Returns prompt + generated ids (src/models/Llama.cpp:513-575)."""
        from .sampler import Sampler
        cfg = cfg or GenerateConfig()
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("generate: empty prompt")
        V = self.config.vocab_size
        if any(t < 0 or t >= V for t in prompt):
            raise ValueError("generate: prompt id outside [0, vocab_size)")
        if cfg.max_new_tokens < 0:
            raise ValueError("generate: max_new_tokens must be >= 0")
        total = len(prompt) + cfg.max_new_tokens
        if total > self.config.max_position_embeddings:
            raise ValueError("generate: prompt + max_new_tokens exceeds max_position_embeddings")
        caches = (self.make_quantized_kv_caches(1, total) if cfg.kv_int8 else self.make_kv_caches(1, total))
        sampler = Sampler(cfg.sampling, cfg.seed) if cfg.do_sample else None
        out = list(prompt)
        if cfg.max_new_tokens == 0:
            return out
        dev = self._device()
        logits = self.forward_step(torch.tensor([prompt], dtype=torch.int64, device=dev), caches)
        for step in range(cfg.max_new_tokens):
            nxt = pick_next_token(logits[0, -1], sampler, out)
            out.append(nxt)
            if cfg.eos_token_id >= 0 and nxt == cfg.eos_token_id:
                break
            if step + 1 < cfg.max_new_tokens:
                logits = self.forward_step(torch.tensor([[nxt]], dtype=torch.int64, device=dev), caches)
        return out

    def quantize_(self, scheme) -> None:
        """Weight-only quantisation of every attention / FFN projection and of lm_head; embedding and norm
        weights stay in floating point (include/tesseract/models/Llama.hpp `quantize_`)."""
        from ..quant import quantize_linear
        for blk in self.layers:
            blk.attn.quantize_(scheme)
            if hasattr(blk.ffn, "quantize_"):
                blk.ffn.quantize_(scheme)
        self.replace_module("lm_head", quantize_linear(self.lm_head, scheme))

    def load_safetensors(self, path: str) -> list:
        """Load a Hugging Face-format safetensors file in place; returns the unmatched keys."""
        from ..io.safetensors import SafeTensors
        st = SafeTensors.open(path)
        return self.load_hf_state_dict({k: st.load(k) for k in st.keys()})

    @staticmethod
    def from_pretrained(path: str, config: LlamaConfig, device=None) -> "LlamaModel":
        m = LlamaModel(config, device=device)
        m.load_safetensors(path)
        return m

    def save_safetensors(self, path: str, metadata: Optional[dict] = None) -> None:
        from ..io.safetensors import save_file
        save_file({k: v.cpu() for k, v in self.hf_state_dict().items()}, path, metadata or {"format": "pt"})

    # ------------------------------------------------------------------ weights by HF name
    def hf_state_dict(self) -> dict:
        out = {}
        for name, p in self.named_parameters():
            if name == "lm_head.weight" and self.config.tie_word_embeddings:
                continue
            out[llama_local_to_hf_name(name)] = p.detach()
        return out

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> list:
        """Copy tensors by Hugging Face key into the existing parameters (float <-> float casts allowed).
        Returns the keys of ``sd`` that matched nothing (src/models/Llama.cpp:638-692)."""
        used = set()
        with torch.no_grad():
            for name, p in self.named_parameters():
                key = llama_local_to_hf_name(name)
                if name == "lm_head.weight" and self.config.tie_word_embeddings:
                    key = "model.embed_tokens.weight"
                if key not in sd:
                    if strict:
                        raise KeyError(f"load: required tensor {key!r} is missing")
                    continue
                t = sd[key]
                if tuple(t.shape) != tuple(p.shape):
                    raise ValueError(f"load: shape of {key!r} is {tuple(t.shape)}, expected {tuple(p.shape)}")
                if not t.is_floating_point():
                    raise TypeError(f"load: {key!r} is not a floating-point tensor")
                p.copy_(t.to(device=p.device, dtype=p.dtype))
                used.add(key)
        return [k for k in sd.keys() if k not in used]
