"""Mamba language model: embed -> N x (RMSNorm -> Mamba -> residual) -> norm -> lm_head
(src/models/MambaModel.cpp:60-173). ``generate`` feeds the prompt through the recurrent step token by token, as the
reference does, and then decodes with O(1) state; ``forward`` (training, scoring) uses the chunked full-sequence
scan kernel."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..nn.mamba import Mamba
from ..nn.modules import Embedding, Linear, Module, ModuleList, RMSNorm
from .llama import pick_next_token
from .sampler import Sampler, SamplingParams


@dataclass
class MambaConfig:
    vocab_size: int = 32000
    hidden_size: int = 256
    num_hidden_layers: int = 4
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    dt_rank: int = 0
    rms_norm_eps: float = 1e-5
    dtype: torch.dtype = torch.float32


@dataclass
class MambaGenerateConfig:
    max_new_tokens: int = 32
    eos_token_id: int = -1
    do_sample: bool = False
    sampling: SamplingParams = None
    seed: int = 0

    def __post_init__(self):
        if self.sampling is None:
            self.sampling = SamplingParams()


class _MambaLayer(Module):
    def __init__(self, c: MambaConfig, device=None):
        super().__init__()
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, c.dtype, device)
        self.mixer = Mamba(c.hidden_size, c.d_state, c.d_conv, c.expand, c.dt_rank, c.dtype, device)


class MambaModel(Module):
    def __init__(self, config: MambaConfig, device=None):
        super().__init__()
        self.config = c = config
        self.embed_tokens = Embedding(c.vocab_size, c.hidden_size, dtype=c.dtype, device=device)
        self.layers = ModuleList([_MambaLayer(c, device) for _ in range(c.num_hidden_layers)])
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, c.dtype, device)
        self.lm_head = Linear(c.hidden_size, c.vocab_size, bias=False, dtype=c.dtype, device=device)

    def num_layers(self) -> int:
        return len(self.layers)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        x = self.embed_tokens(tokens)
        for l in self.layers:
            x = x + l.mixer(l.norm(x))
        return self.lm_head(self.norm(x))

    @torch.no_grad()
    def forward_step(self, tokens: torch.Tensor, caches: list) -> torch.Tensor:
        x = self.embed_tokens(tokens)
        for l, c in zip(self.layers, caches):
            x = x + l.mixer.forward_step(l.norm(x), c)
        return self.lm_head(self.norm(x))

    def make_state_caches(self, batch: int) -> list:
        return [l.mixer.make_state_cache(batch) for l in self.layers]

    @torch.no_grad()
    def generate(self, prompt_ids, cfg: Optional[MambaGenerateConfig] = None) -> list:
        cfg = cfg or MambaGenerateConfig()
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("generate: empty prompt")
        if any(t < 0 or t >= self.config.vocab_size for t in prompt):
            raise ValueError("generate: prompt id outside [0, vocab_size)")
        dev = self.embed_tokens.weight.device
        caches = self.make_state_caches(1)
        sampler = Sampler(cfg.sampling, cfg.seed) if cfg.do_sample else None
        out = list(prompt)
        logits = None
        for t in prompt:  # recurrent prefill
            logits = self.forward_step(torch.tensor([[t]], dtype=torch.int64, device=dev), caches)
        for step in range(cfg.max_new_tokens):
            nxt = pick_next_token(logits[0, -1], sampler, out)
            out.append(nxt)
            if cfg.eos_token_id >= 0 and nxt == cfg.eos_token_id:
                break
            if step + 1 < cfg.max_new_tokens:
                logits = self.forward_step(torch.tensor([[nxt]], dtype=torch.int64, device=dev), caches)
        return out
