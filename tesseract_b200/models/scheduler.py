"""Continuous-batching scheduler over paged KV pools.

Contract of the reference (include/tesseract/models/Scheduler.hpp:48-147, src/models/Scheduler.cpp:51-232):
FIFO admission while there is batch room and ``free_blocks >= ceil(prompt / block_size)`` (head-of-line
blocking when the head does not fit; an error when nothing is running that could free blocks);
``prompt + max_new_tokens <= max_seq_len``; every request owns a sampler seeded with its ``seed``;
one ``step()`` = admit -> emit one token per running request -> retire on EOS / length (blocks go back to
the pool) -> one batched forward over the survivors; finished results are retained. On CPU the output of a
request is identical to a standalone ``generate`` with the same config (greedy, seeded sampling, INT8 KV).

What differs from the reference: requests admitted in the same step are prefilled together when their
prompts have equal length, and decode uses one ragged paged-attention launch per layer for the whole batch.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

import torch

from .llama import GenerateConfig, LlamaModel, pick_next_token
from .sampler import Sampler


@dataclass
class EngineConfig:
    block_size: int = 16
    num_blocks: int = 2048      # blocks in EACH per-layer pool
    max_seq_len: int = 2048
    max_batch_size: int = 16
    kv_int8: bool = False


@dataclass
class _Request:
    id: int
    gen: GenerateConfig
    tokens: List[int]
    prompt_len: int
    generated: int = 0
    finished: bool = False
    caches: Optional[list] = None
    sampler: Optional[Sampler] = None
    last_logits: Optional[torch.Tensor] = None
    t_submit: float = 0.0
    t_first: float = 0.0


class ContinuousBatchingScheduler:
    def __init__(self, model: LlamaModel, cfg: Optional[EngineConfig] = None):
        self.model, self.cfg = model, cfg or EngineConfig()
        c = self.cfg
        if c.block_size <= 0 or c.num_blocks <= 0 or c.max_batch_size <= 0:
            raise ValueError("EngineConfig: block_size, num_blocks and max_batch_size must be positive")
        self.pools = (model.make_quantized_layer_pools(c.num_blocks, c.block_size) if c.kv_int8
                      else model.make_layer_pools(c.num_blocks, c.block_size))
        self.waiting: Deque[_Request] = deque()
        self.running: List[int] = []
        self.requests: Dict[int, _Request] = {}
        self._next_id = 0
        self.steps = 0

    # ---- occupancy -------------------------------------------------------------------------------
    def has_pending(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def num_waiting(self) -> int:
        return len(self.waiting)

    def num_running(self) -> int:
        return len(self.running)

    def allocated_blocks(self) -> int:
        return self.pools[0].allocator.num_used()

    def free_blocks(self) -> int:
        return self.pools[0].allocator.num_free()

    def is_finished(self, rid: int) -> bool:
        r = self.requests.get(rid)
        return bool(r and r.finished)

    def result(self, rid: int) -> List[int]:
        r = self.requests.get(rid)
        if r is None or not r.finished:
            raise KeyError(f"request {rid} is unknown or not finished")
        return list(r.tokens)

    # ---- request lifecycle -----------------------------------------------------------------------
    def add_request(self, prompt_ids, gen: Optional[GenerateConfig] = None) -> int:
        gen = gen or GenerateConfig()
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("add_request: empty prompt")
        V = self.model.config.vocab_size
        if any(t < 0 or t >= V for t in prompt):
            raise ValueError("add_request: prompt id outside [0, vocab_size)")
        if gen.max_new_tokens < 0:
            raise ValueError("add_request: max_new_tokens must be >= 0")
        if len(prompt) + gen.max_new_tokens > self.cfg.max_seq_len:
            raise ValueError("add_request: prompt + max_new_tokens exceeds max_seq_len")
        if self._blocks_for(len(prompt) + gen.max_new_tokens) > self.cfg.num_blocks:
            raise ValueError("add_request: the request can never fit in the KV pool")
        rid = self._next_id
        self._next_id += 1
        r = _Request(rid, gen, prompt, len(prompt))
        if gen.do_sample:
            r.sampler = Sampler(gen.sampling, gen.seed)
        self.waiting.append(r)
        return rid

    def _blocks_for(self, n: int) -> int:
        return (n + self.cfg.block_size - 1) // self.cfg.block_size

    def _make_caches(self):
        m, c = self.model, self.cfg
        return (m.make_quantized_paged_kv_caches(self.pools, c.max_seq_len) if c.kv_int8
                else m.make_paged_kv_caches(self.pools, c.max_seq_len))

    def _admit(self) -> None:
        admitted: List[_Request] = []
        reserved = 0
        while self.waiting and len(self.running) + len(admitted) < self.cfg.max_batch_size:
            head = self.waiting[0]
            need = self._blocks_for(head.prompt_len)
            if self.free_blocks() - reserved < need:
                if not self.running and not admitted:
                    raise RuntimeError("scheduler: the head request does not fit and nothing is running to reclaim from")
                break
            reserved += need
            admitted.append(self.waiting.popleft())
        dev = self.model._device()
        # prefill: group equal-length prompts into one batched call
        by_len: Dict[int, List[_Request]] = {}
        for r in admitted:
            by_len.setdefault(r.prompt_len, []).append(r)
        for plen, group in by_len.items():
            for r in group:
                r.caches = self._make_caches()
            toks = torch.tensor([r.tokens for r in group], dtype=torch.int64, device=dev)
            if len(group) == 1:
                logits = self.model.forward_step(toks, group[0].caches)
            else:
                logits = self.model.forward_step_batched(toks, [r.caches for r in group])
            for i, r in enumerate(group):
                r.last_logits = logits[i, -1]
        for r in admitted:  # keep FIFO order in the running list
            self.requests[r.id] = r
            self.running.append(r.id)

    def _retire(self, r: _Request) -> None:
        for c in r.caches or []:
            c.reset()
        r.caches = None
        r.last_logits = None
        r.finished = True

    def step(self) -> bool:
        """One scheduling tick. Returns ``has_pending()`` afterwards."""
        self._admit()
        survivors: List[_Request] = []
        for rid in self.running:
            r = self.requests[rid]
            if r.generated >= r.gen.max_new_tokens:
                self._retire(r)
                continue
            nxt = pick_next_token(r.last_logits, r.sampler, r.tokens)
            r.tokens.append(nxt)
            r.generated += 1
            if (r.gen.eos_token_id >= 0 and nxt == r.gen.eos_token_id) or r.generated >= r.gen.max_new_tokens:
                self._retire(r)
            else:
                survivors.append(r)
        self.running = [r.id for r in survivors]
        if survivors:
            dev = self.model._device()
            toks = torch.tensor([[r.tokens[-1]] for r in survivors], dtype=torch.int64, device=dev)
            logits = self.model.forward_step_batched(toks, [r.caches for r in survivors])
            for i, r in enumerate(survivors):
                r.last_logits = logits[i, -1]
        self.steps += 1
        return self.has_pending()

    def run(self) -> None:
        while self.has_pending():
            self.step()
