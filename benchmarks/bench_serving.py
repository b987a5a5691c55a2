#!/usr/bin/env python
"""Serving benchmark: continuous batching of N requests on the device-resident engine.

Workload of the headline serving configuration: Llama-3-8B shape, random-init weights, 256 requests with prompt
lengths uniform in [128, 2048] and output lengths uniform in [64, 512] (random token ids), paged KV with 16-token
blocks (bf16 or INT8), greedy or top-p 0.9 sampling. Reports prefill tokens/s, decode tokens/s and p50 TTFT as one
JSON line. Timing is wall clock around the engine loop with a device synchronise on both sides; the per-phase
numbers come from the engine's own accounting (each phase ends with the device-to-host read of the new tokens).

    python benchmarks/bench_serving.py --requests 256 --kv-int8 0 --top-p 1.0
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
        benchmarks/bench_serving.py --requests 256          # tensor parallel over the 8 ranks

With more than one rank every rank runs the same engine on the same requests (tensor-parallel layers, replicated
sampling); the reported times are the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_serving_bench(requests=256, layers=32, kv_int8=False, top_p=1.0, temperature=0.0, max_batch=256,
                      prompt_range=(128, 2048), out_range=(64, 512), seed=0, cuda_graph=True, device=None, model=None,
                      tp_group=None, rank=0, world=1, max_prefill_tokens=16384, fp8_prefill=False, weights="fp8",
                      engine=None, tp=None):
    """One pass of the workload. ``engine`` (with ``tp``) may be a ``ServingEngine`` from an earlier pass with the same
    weights and KV format: its sampling settings are replaced and its pools reused (no second copy of the model)."""
    import torch

    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.scheduler import EngineConfig
    from tesseract_b200.serving import ServingEngine

    dev = device or torch.device("cuda", 0)
    max_seq = prompt_range[1] + out_range[1]
    if engine is not None:
        model = engine.model
    if model is None:
        cfg = LlamaConfig.llama_3_8b(dtype=torch.bfloat16, max_position_embeddings=max_seq)
        cfg.num_hidden_layers = layers
        model = LlamaModel(cfg, device=dev, init_std=0.02, seed=1)
    cfg = model.config
    rng = random.Random(seed)
    reqs = []
    for _ in range(requests):
        p, o = rng.randint(*prompt_range), rng.randint(*out_range)
        reqs.append(([rng.randrange(cfg.vocab_size) for _ in range(p)], o))
    total_tokens = sum(len(p) + o for p, o in reqs)
    block = 16
    num_blocks = total_tokens // block + requests + 64       # every request can be resident at once
    ecfg = EngineConfig(block_size=block, num_blocks=num_blocks, max_seq_len=max_seq, max_batch_size=max_batch,
                        kv_int8=kv_int8)
    if engine is None:
        if world > 1:
            from tesseract_b200.serving.engine import TPServe
            tp = TPServe(tp_group, rank, world, dev, cfg.hidden_size, max_batch=max(512, max_batch))
        eng = ServingEngine(model, ecfg, use_cuda_graph=cuda_graph, temperature=temperature, top_p=top_p, seed=seed, tp=tp,
                            max_prefill_tokens=max_prefill_tokens, fp8_prefill=fp8_prefill, weights=weights)
    else:
        eng = engine
        if eng.running or eng.waiting:
            raise RuntimeError("run_serving_bench: the engine passed in still has requests")
        new_greedy = temperature <= 1e-6
        if new_greedy != eng.greedy:
            eng._graphs.clear()                 # the captured step ends in the other token-selection kernel
        eng.temperature, eng.top_p, eng.seed, eng.greedy = temperature, top_p, seed, new_greedy
        eng.requests.clear()
    # warm-up: one short request end to end (kernel attributes, allocator pools, first graph bucket)
    eng.add_request(reqs[0][0][:64], GenerateConfig(max_new_tokens=4))
    eng.run()
    eng.stats = {k: 0 if isinstance(v, int) else 0.0 for k, v in eng.stats.items()}
    eng.steps = 0
    for p, o in reqs:
        eng.add_request(p, GenerateConfig(max_new_tokens=o))
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    eng.run()
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    m = eng.metrics()
    gen_tokens = sum(o for _, o in reqs)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([eng.stats["prefill_s"], eng.stats["decode_s"], wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=tp_group)
        pre_s, dec_s, wall = t.tolist()
        m["prefill_tok_s"] = eng.stats["prefill_tokens"] / pre_s if pre_s > 0 else 0.0
        m["decode_tok_s"] = eng.stats["decode_tokens"] / dec_s if dec_s > 0 else 0.0
        digest = torch.tensor([sum(sum(r.tokens[r.prompt_len:]) for r in eng.requests.values()) % (1 << 40)],
                              device=dev, dtype=torch.int64)
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=tp_group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=tp_group)
        if int(lo) != int(hi):
            raise RuntimeError("tensor-parallel ranks generated different tokens")
    from tesseract_b200 import _native
    return {
        "tp": world, "kernel_status": _native.read_status(torch.cuda.current_stream(dev).cuda_stream),
        "requests": requests, "kv": "int8" if kv_int8 else "bf16", "fp8_prefill": bool(fp8_prefill), "sampling": "greedy" if temperature <= 0 else f"top_p={top_p}",
        "prefill_tok_s": m["prefill_tok_s"], "decode_tok_s": m["decode_tok_s"], "ttft_p50_ms": m["ttft_p50_ms"],
        "end_to_end_s": wall, "generated_tokens": gen_tokens, "total_tok_s": (total_tokens) / wall,
        "steps": m["steps"], "decode_ms_per_step": m["decode_ms_per_step"],
        "decode_gpu_ms_per_step": m["decode_gpu_ms_per_step"], "max_batch": max_batch, "block_size": block, "cuda_graph": cuda_graph,
        "weights": "fp8-e4m3-block128 (bf16 activations on the decode path, 1x128 fp8 on the prompt path)"
                   if eng.weights == "fp8" else "bf16",
        "weight_bytes_per_rank": eng.weight_bytes(), "layers": len(model.layers),
        "max_prefill_tokens": max_prefill_tokens, "_engine": eng, "_tp": tp,
    }


def run_serving_variants(requests=256, layers=32, device=None, tp_group=None, rank=0, world=1, weights="fp8",
                         variants=(("bf16", "greedy"), ("bf16", "top_p"), ("int8", "greedy"), ("int8", "top_p"))):
    """The four variants of the named serving configuration (KV bf16 / INT8 x greedy / top-p 0.9), one engine per KV
    format. Returns {"<kv>_<sampling>": result}; the first variant is the headline."""
    import gc

    import torch
    out, eng, tp, cur_kv = {}, None, None, None
    for kv, samp in variants:
        if kv != cur_kv and eng is not None:
            del eng
            eng, cur_kv = None, None
            gc.collect()
            torch.cuda.empty_cache()
        r = run_serving_bench(requests=requests, layers=layers, kv_int8=(kv == "int8"),
                              temperature=0.0 if samp == "greedy" else 1.0, top_p=1.0 if samp == "greedy" else 0.9,
                              device=device, tp_group=tp_group, rank=rank, world=world, weights=weights,
                              engine=eng, tp=tp)
        eng, tp, cur_kv = r.pop("_engine"), r.pop("_tp"), kv
        out[f"{kv}_{samp}"] = r
    del eng
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--kv-int8", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--max-batch", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--fp8-prefill", type=int, default=0, help="1: prefill GEMMs on per-tensor-scaled E4M3 weight copies")
    ap.add_argument("--max-prefill-tokens", type=int, default=16384, help="prompt tokens admitted per engine step (0 = all)")
    ap.add_argument("--weights", default="fp8", choices=["fp8", "bf16"])
    a = ap.parse_args()
    import torch
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    group = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    out = run_serving_bench(a.requests, a.layers, bool(a.kv_int8), a.top_p, a.temperature, a.max_batch,
                            cuda_graph=not a.no_graph, device=dev, tp_group=group, rank=rank, world=world,
                            max_prefill_tokens=a.max_prefill_tokens, fp8_prefill=bool(a.fp8_prefill), weights=a.weights)
    out.pop("_engine", None)
    out.pop("_tp", None)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
