#!/usr/bin/env python
"""Continuous-batching serving demo (the reference's examples/llama_serve.cpp:54-171, same flags): several prompts
are queued on one engine, decoded together step by step over a paged KV cache, and printed as they finish.

    python examples/llama_serve.py --synthetic --prompts "alpha|beta|gamma" --max-new-tokens 16 --max-batch 4
    python examples/llama_serve.py --device cuda --model small --sample --temperature 0.8 --seed 7
"""
from __future__ import annotations

import argparse
import sys
import time

from _common import load_tokenizer, pick_device, preset, torch


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--prompts", default="alpha|beta|gamma|delta")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--max-batch", type=int, default=4)
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--synthetic", action="store_true", help="random weights (the default, as in the reference)")
    ap.add_argument("--model", default="small")
    ap.add_argument("--kv-int8", action="store_true")
    ap.add_argument("--engine", default="auto", help="auto | scheduler (reference semantics) | batched (device-resident engine)")
    a = ap.parse_args()

    from tesseract_b200.models import GenerateConfig, LlamaModel
    from tesseract_b200.models.sampler import SamplingParams
    from tesseract_b200.models.scheduler import ContinuousBatchingScheduler, EngineConfig
    dev = pick_device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = preset(a.model, dtype, 2048)
    model = LlamaModel(cfg, device=dev, init_std=0.02, seed=a.seed)
    model.eval()
    tok = load_tokenizer(a.tokenizer)
    ecfg = EngineConfig(block_size=16, num_blocks=1024, max_seq_len=2048, max_batch_size=a.max_batch, kv_int8=a.kv_int8)
    use_batched = a.engine == "batched" or (a.engine == "auto" and dev.type == "cuda")
    if use_batched:
        from tesseract_b200.serving.engine import ServingEngine
        from tesseract_b200.parallel.launch import job_metrics
        engine = ServingEngine(model, ecfg).instrument(metrics=job_metrics())    # TESSERACT_METRICS_FILE / TESSERACT_NVTX
    else:
        engine = ContinuousBatchingScheduler(model, ecfg)
    prompts = [p for p in a.prompts.split("|") if p]
    rids = []
    for i, p in enumerate(prompts):
        ids = [t % cfg.vocab_size for t in tok.encode(p)]
        gen = GenerateConfig(max_new_tokens=a.max_new_tokens, eos_token_id=cfg.eos_token_id, do_sample=a.sample,
                             seed=a.seed + i, sampling=SamplingParams(temperature=a.temperature))
        rids.append((engine.add_request(ids, gen), p, len(ids)))
    t0, steps, done = time.time(), 0, set()
    with torch.no_grad():
        while engine.has_pending():
            engine.step()
            steps += 1
            for rid, p, n in rids:
                if rid not in done and engine.is_finished(rid):
                    done.add(rid)
                    out = engine.result(rid)
                    print(f"[req {rid} done at step {steps}] {p!r} -> {tok.decode(out[n:])!r}")
    dt = time.time() - t0
    total = sum(len(engine.result(r)) - n for r, _, n in rids)
    print(f"{len(rids)} requests, {total} tokens, {steps} engine steps, {dt:.2f} s ({total / max(dt, 1e-9):.1f} tok/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
