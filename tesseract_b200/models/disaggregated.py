"""Prefill / decode disaggregation in one process: the prefill role runs the prompt and exports every
layer's K/V prefix (``KvTransfer``); the decode role imports it into fresh caches and continues. The result
equals monolithic greedy generation (src/models/Disaggregated.cpp:40-126)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .llama import LlamaModel


@dataclass
class KvTransfer:
    keys: List[torch.Tensor]      # per layer [1, Hkv, P, D]
    values: List[torch.Tensor]
    prompt_len: int
    first_token: int

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.keys + self.values)


class DisaggregatedEngine:
    def __init__(self, prefill_model: LlamaModel, decode_model: LlamaModel):
        if prefill_model.config.vocab_size != decode_model.config.vocab_size:
            raise ValueError("DisaggregatedEngine: models disagree on the vocabulary")
        self.prefill_model, self.decode_model = prefill_model, decode_model

    @torch.no_grad()
    def prefill(self, prompt_ids) -> KvTransfer:
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("prefill: empty prompt")
        m = self.prefill_model
        caches = m.make_kv_caches(1, len(prompt))
        logits = m.forward_step(torch.tensor([prompt], dtype=torch.int64, device=m._device()), caches)
        first = int(torch.argmax(logits[0, -1].float()).item())
        return KvTransfer([c.keys_view().clone() for c in caches], [c.values_view().clone() for c in caches],
                          len(prompt), first)

    @torch.no_grad()
    def decode(self, prompt_ids, kv: KvTransfer, max_new_tokens: int, eos_token_id: int = -1) -> List[int]:
        m = self.decode_model
        dev = m._device()
        out = [int(t) for t in prompt_ids]
        if max_new_tokens <= 0:
            return out
        caches = m.make_kv_caches(1, kv.prompt_len + max_new_tokens)
        for c, k, v in zip(caches, kv.keys, kv.values):
            c.append(k.to(dev), v.to(dev))
        nxt = kv.first_token
        for step in range(max_new_tokens):
            out.append(nxt)
            if eos_token_id >= 0 and nxt == eos_token_id:
                break
            if step + 1 < max_new_tokens:
                logits = m.forward_step(torch.tensor([[nxt]], dtype=torch.int64, device=dev), caches)
                nxt = int(torch.argmax(logits[0, -1].float()).item())
        return out

    def generate(self, prompt_ids, max_new_tokens: int, eos_token_id: int = -1) -> List[int]:
        return self.decode(prompt_ids, self.prefill(prompt_ids), max_new_tokens, eos_token_id)
