#!/usr/bin/env python
"""Serving benchmark: continuous batching of N requests on the device-resident engine.

Workload of the headline serving configuration: Llama-3-8B shape, random-init weights, 256 requests with prompt
lengths uniform in [128, 2048] and output lengths uniform in [64, 512] (random token ids), paged KV with 16-token
blocks (bf16 or INT8), fp8 E4M3 block-scaled weights (or bf16), greedy or top-p 0.9 sampling. Reports prefill
tokens/s, decode tokens/s and p50 TTFT as one JSON line. Timing is wall clock around the engine loop with a device
synchronise on both sides; the per-phase numbers come from the engine's own accounting (each phase ends with the
device-to-host read of the new tokens).

    python benchmarks/bench_serving.py --requests 256 --kv-int8 0 --top-p 1.0
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
        benchmarks/bench_serving.py --requests 256 [--tp 8]

With more than one rank the ranks form ``world / tp`` replicas of ``tp`` tensor-parallel ranks (``--tp``; default:
``serving.default_tp``). Every replica serves its round-robin share of the requests with its own engine; inside a
replica every rank runs the same engine on the same requests (tensor-parallel layers, replicated sampling, digest
check). Reported rates are the sum over replicas of each replica's tokens divided by the slowest replica's time of that
phase; TTFT is the median over all requests of all replicas.
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
                      rank=0, world=1, tp_size=0, max_prefill_tokens=16384, fp8_prefill=False, weights="fp8",
                      state=None):
    """One pass of the workload. ``state`` is the dict a previous pass returned under "_state" (engine, replica plan):
    with the same weights and KV format its engine is reused with new sampling settings (no second model copy)."""
    import torch

    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.scheduler import EngineConfig
    from tesseract_b200.serving import ServingEngine, default_tp, make_replica_plan, split_requests

    dev = device or torch.device("cuda", 0)
    max_seq = prompt_range[1] + out_range[1]
    if state is None:
        tp_size = tp_size or default_tp(world)
        plan = make_replica_plan(world, rank, tp_size)
        state = {"plan": plan, "engine": None, "tp": None}
    plan = state["plan"]
    eng = state["engine"]
    if eng is not None:
        model = eng.model
    if model is None:
        cfg = LlamaConfig.llama_3_8b(dtype=torch.bfloat16, max_position_embeddings=max_seq)
        cfg.num_hidden_layers = layers
        model = LlamaModel(cfg, device=dev, init_std=0.02, seed=1)
    cfg = model.config
    rng = random.Random(seed)
    all_reqs = []
    for _ in range(requests):
        p, o = rng.randint(*prompt_range), rng.randint(*out_range)
        all_reqs.append(([rng.randrange(cfg.vocab_size) for _ in range(p)], o))
    reqs = split_requests(all_reqs, plan)
    total_tokens_all = sum(len(p) + o for p, o in all_reqs)
    my_tokens = sum(len(p) + o for p, o in reqs)
    block = 16
    num_blocks = my_tokens // block + len(reqs) + 64          # every request of the replica can be resident at once
    rep_batch = max(1, (max_batch + plan.replicas - 1) // plan.replicas)
    ecfg = EngineConfig(block_size=block, num_blocks=num_blocks, max_seq_len=max_seq, max_batch_size=rep_batch,
                        kv_int8=kv_int8)
    if eng is None:
        tp = None
        if plan.tp > 1:
            from tesseract_b200.serving.engine import TPServe
            tp = TPServe(plan.group, plan.tp_rank, plan.tp, dev, cfg.hidden_size, max_batch=max(512, rep_batch))
        eng = ServingEngine(model, ecfg, use_cuda_graph=cuda_graph, temperature=temperature, top_p=top_p, seed=seed, tp=tp,
                            max_prefill_tokens=max_prefill_tokens, fp8_prefill=fp8_prefill, weights=weights)
        state["engine"], state["tp"] = eng, tp
    else:
        if eng.running or eng.waiting:
            raise RuntimeError("run_serving_bench: the engine passed in still has requests")
        new_greedy = temperature <= 1e-6
        if new_greedy != eng.greedy:
            eng._graphs.clear()                 # the captured step ends in the other token-selection kernel
        eng.temperature, eng.top_p, eng.seed, eng.greedy = temperature, top_p, seed, new_greedy
        eng.requests.clear()
    # warm-up: one short request end to end (kernel attributes, allocator pools, first graph bucket)
    eng.add_request(all_reqs[0][0][:64], GenerateConfig(max_new_tokens=4))
    eng.run()
    eng.warm_graphs()                           # every decode bucket captured before the clock starts
    eng.requests.clear()
    eng.stats = {k: 0 if isinstance(v, int) else 0.0 for k, v in eng.stats.items()}
    eng.steps = 0
    for p, o in reqs:
        eng.add_request(p, GenerateConfig(max_new_tokens=o))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()                          # the replicas start together
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    eng.run()
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    m = eng.metrics()
    s = eng.stats
    gen_tokens = sum(o for _, o in all_reqs)
    pre_tok, dec_tok, pre_s, dec_s = s["prefill_tokens"], s["decode_tokens"], s["prefill_s"], s["decode_s"]
    ttfts = sorted((r.t_first - r.t_submit) * 1e3 for r in eng.requests.values() if r.finished and r.t_first > 0)
    if world > 1:
        import torch.distributed as dist
        if plan.tp > 1:                          # every rank of a replica must have produced the same tokens
            digest = torch.tensor([sum(sum(r.tokens[r.prompt_len:]) for r in eng.requests.values()) % (1 << 40)],
                                  device=dev, dtype=torch.int64)
            lo, hi = digest.clone(), digest.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=plan.group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=plan.group)
            if int(lo) != int(hi):
                raise RuntimeError("tensor-parallel ranks generated different tokens")
        lead = 1.0 if plan.is_leader else 0.0
        sums = torch.tensor([pre_tok * lead, dec_tok * lead], device=dev, dtype=torch.float64)
        maxs = torch.tensor([pre_s, dec_s, wall, m["decode_ms_per_step"], m["decode_gpu_ms_per_step"]], device=dev,
                            dtype=torch.float64)
        dist.all_reduce(sums)
        dist.all_reduce(maxs, op=dist.ReduceOp.MAX)
        pre_tok, dec_tok = sums.tolist()
        pre_s, dec_s, wall, m["decode_ms_per_step"], m["decode_gpu_ms_per_step"] = maxs.tolist()
        gathered = [None] * world
        dist.all_gather_object(gathered, ttfts if plan.is_leader else [])
        ttfts = sorted(t for part in gathered for t in part)
    from tesseract_b200 import _native
    return {
        "n_gpus": world, "tp": plan.tp, "replicas": plan.replicas,
        "parallelism": (f"tp{plan.tp}" if plan.tp > 1 else "single") + (f" x {plan.replicas} replicas" if plan.replicas > 1 else ""),
        "kernel_status": _native.read_status(torch.cuda.current_stream(dev).cuda_stream),
        "requests": requests, "kv": "int8" if kv_int8 else "bf16", "fp8_prefill": bool(fp8_prefill),
        "sampling": "greedy" if temperature <= 0 else f"top_p={top_p}",
        "prefill_tok_s": pre_tok / pre_s if pre_s > 0 else 0.0, "decode_tok_s": dec_tok / dec_s if dec_s > 0 else 0.0,
        "ttft_p50_ms": ttfts[len(ttfts) // 2] if ttfts else 0.0,
        "end_to_end_s": wall, "generated_tokens": gen_tokens, "total_tok_s": total_tokens_all / wall,
        "steps": m["steps"], "decode_ms_per_step": m["decode_ms_per_step"],
        "decode_gpu_ms_per_step": m["decode_gpu_ms_per_step"], "max_batch": max_batch, "max_batch_per_replica": rep_batch,
        "block_size": block, "cuda_graph": cuda_graph,
        "weights": "fp8-e4m3-block128, power-of-two scales (decode: E4M3 activations with 1x32 power-of-two scales on mxf8f6f4; prefill: 1x128 fp8)"
                   if eng.weights == "fp8" else "bf16",
        "weight_bytes_per_rank": eng.weight_bytes(), "layers": len(model.layers),
        "max_prefill_tokens": max_prefill_tokens, "_state": state,
    }


def run_serving_variants(requests=256, layers=32, device=None, rank=0, world=1, tp_size=0, weights="fp8",
                         variants=(("bf16", "greedy"), ("bf16", "top_p"), ("int8", "greedy"), ("int8", "top_p"))):
    """The four variants of the named serving configuration (KV bf16 / INT8 x greedy / top-p 0.9), one engine per KV
    format. Returns {"<kv>_<sampling>": result}; the first variant is the headline."""
    import gc

    import torch
    out, state, cur_kv = {}, None, None
    for kv, samp in variants:
        if kv != cur_kv and state is not None:
            state["engine"] = None              # another KV format: new pools (the replica plan and groups stay)
            state["tp"] = None
            gc.collect()
            torch.cuda.empty_cache()
        r = run_serving_bench(requests=requests, layers=layers, kv_int8=(kv == "int8"),
                              temperature=0.0 if samp == "greedy" else 1.0, top_p=1.0 if samp == "greedy" else 0.9,
                              device=device, rank=rank, world=world, tp_size=tp_size, weights=weights, state=state)
        state, cur_kv = r.pop("_state"), kv
        out[f"{kv}_{samp}"] = r
    state["engine"] = None
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
    ap.add_argument("--fp8-prefill", type=int, default=0, help="1: prefill GEMMs on per-tensor-scaled E4M3 weight copies (bf16 weights)")
    ap.add_argument("--max-prefill-tokens", type=int, default=16384, help="prompt tokens admitted per engine step (0 = all)")
    ap.add_argument("--weights", default="fp8", choices=["fp8", "bf16"])
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel ranks per replica (0 = serving.default_tp)")
    a = ap.parse_args()
    import torch
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    out = run_serving_bench(a.requests, a.layers, bool(a.kv_int8), a.top_p, a.temperature, a.max_batch,
                            cuda_graph=not a.no_graph, device=dev, rank=rank, world=world, tp_size=a.tp,
                            max_prefill_tokens=a.max_prefill_tokens, fp8_prefill=bool(a.fp8_prefill), weights=a.weights)
    out.pop("_state", None)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
