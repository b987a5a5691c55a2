"""Greedy speculative decoding: a draft model proposes ``gamma`` tokens, the target verifies them in one
forward pass, caches are rewound with ``set_current_len`` and the first disagreement is replaced by the
target's own token. The output is exactly the target's greedy continuation for any draft model
(src/models/Speculative.cpp:35-155); ``Result`` carries the acceptance statistics."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import torch

from .llama import LlamaModel


@dataclass
class SpeculativeResult:
    tokens: List[int] = field(default_factory=list)
    proposed: int = 0
    accepted: int = 0
    rounds: int = 0
    target_forwards: int = 0


class SpeculativeDecoder:
    def __init__(self, target: LlamaModel, draft: LlamaModel, gamma: int = 4):
        if target is None or draft is None:
            raise ValueError("SpeculativeDecoder: null model")
        if gamma < 1:
            raise ValueError("SpeculativeDecoder: gamma must be >= 1")
        if target.config.vocab_size != draft.config.vocab_size:
            raise ValueError("SpeculativeDecoder: target and draft vocabularies differ")
        self.target, self.draft, self.gamma = target, draft, gamma

    @torch.no_grad()
    def generate(self, prompt_ids, max_new_tokens: int, eos_token_id: int = -1) -> SpeculativeResult:
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("SpeculativeDecoder: empty prompt")
        dev = self.target._device()
        cap = len(prompt) + max_new_tokens + self.gamma + 2
        tc = self.target.make_kv_caches(1, cap)
        dc = self.draft.make_kv_caches(1, cap)

        def feed(model, caches, ids):
            return model.forward_step(torch.tensor([ids], dtype=torch.int64, device=dev), caches)[0].float()

        def top(row):
            return int(torch.argmax(row).item())

        res = SpeculativeResult(tokens=list(prompt))
        t_next = top(feed(self.target, tc, prompt)[-1])
        d_next = top(feed(self.draft, dc, prompt)[-1])
        res.target_forwards += 1
        produced = 0
        while produced < max_new_tokens:
            base = len(res.tokens)
            # draft proposes gamma tokens (the first is already known from its last logits)
            proposal = [d_next]
            while len(proposal) < self.gamma:
                proposal.append(top(feed(self.draft, dc, [proposal[-1]])[-1]))
            res.proposed += self.gamma
            verify = feed(self.target, tc, proposal)       # row i predicts the token after proposal[i]
            res.target_forwards += 1
            res.rounds += 1
            expected = [t_next] + [top(verify[i]) for i in range(self.gamma - 1)]
            n_ok = 0
            while n_ok < self.gamma and proposal[n_ok] == expected[n_ok]:
                n_ok += 1
            correction = t_next if n_ok == 0 else top(verify[n_ok - 1])
            res.accepted += n_ok
            done = False
            for tok in proposal[:n_ok]:
                if produced >= max_new_tokens or done:
                    break
                res.tokens.append(tok)
                produced += 1
                done = eos_token_id >= 0 and tok == eos_token_id
            committed = False
            if not done and produced < max_new_tokens:
                res.tokens.append(correction)
                produced += 1
                committed = True
                done = eos_token_id >= 0 and correction == eos_token_id
            if done or produced >= max_new_tokens:
                break
            for c in tc + dc:                               # drop everything after the accepted prefix
                c.set_current_len(base + n_ok)
            if committed:
                t_next = top(feed(self.target, tc, [correction])[-1])
                d_next = top(feed(self.draft, dc, [correction])[-1])
                res.target_forwards += 1
        return res
