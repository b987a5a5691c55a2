#!/usr/bin/env python
"""One decode step of the serving engine in isolation: B resident requests with the same context length, a few steps
through the captured CUDA graph, device time per step. Meant for per-kernel launch lists:

    python benchmarks/bench_decode_step.py --batch 32 --context 1300 --layers 8 && \
    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv \
        --log-file launches.csv python benchmarks/bench_decode_step.py --batch 32 --context 1300 --layers 8

(the profiled region -- two steps -- is bracketed by cudaProfilerStart / Stop, so the prompt pass is not captured).
Llama-3-8B layer shape with ``--layers`` layers (8 by default: a capture stays small), random-init weights, random
prompt tokens, paged KV with 16-token blocks. Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.scheduler import EngineConfig
    from tesseract_b200.serving import ServingEngine

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--context", type=int, default=1300)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--weights", default="fp8", choices=["fp8", "bf16"])
    ap.add_argument("--kv-int8", type=int, default=0)
    ap.add_argument("--steps", type=int, default=2, help="steps inside the profiled region")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = LlamaConfig.llama_3_8b(dtype=torch.bfloat16, max_position_embeddings=a.context + 64)
    cfg.num_hidden_layers = a.layers
    model = LlamaModel(cfg, device=dev, init_std=0.02, seed=1)
    ecfg = EngineConfig(block_size=16, num_blocks=a.batch * (a.context + 64) // 16 + 64, max_seq_len=a.context + 64,
                        max_batch_size=a.batch, kv_int8=bool(a.kv_int8))
    eng = ServingEngine(model, ecfg, use_cuda_graph=True, weights=a.weights, max_prefill_tokens=65536)
    rng = random.Random(0)
    for _ in range(a.batch):
        eng.add_request([rng.randrange(cfg.vocab_size) for _ in range(a.context)],
                        GenerateConfig(max_new_tokens=a.steps + 16))
    while eng.waiting:
        eng.step()
    for _ in range(4):                      # graph capture and warm-up of the decode bucket
        eng.step()
    eng.stats["decode_gpu_s"], eng.stats["decode_steps"] = 0.0, 0
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(a.steps):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    m = eng.metrics()
    print(json.dumps({"bench": "decode_step", "batch": a.batch, "context": a.context, "layers": a.layers,
                      "weights": a.weights, "kv": "int8" if a.kv_int8 else "bf16",
                      "decode_gpu_ms_per_step": round(m["decode_gpu_ms_per_step"], 4),
                      "per_layer_us": round(1e3 * m["decode_gpu_ms_per_step"] / a.layers, 1),
                      "running": len(eng.running)}))


if __name__ == "__main__":
    main()
