#!/usr/bin/env python
"""Mixture-of-experts Llama, expert-parallel over all ranks: one training pass (forward + backward + gradient
reduction) over the global batch, and one decode step.

    python benchmarks/bench_moe_model.py                                    # EP = 1: all experts on one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29660 \
        benchmarks/bench_moe_model.py                                       # EP = 8: one expert of every layer per rank

Model of the MoE north-star configuration: 32 layers, d_model 4096, 32 / 8 GQA heads, 8 experts per layer with a top-2
softmax router, expert FFN 14336 (SwiGLU), vocabulary 32000, bf16, random-init N(0, 0.02) weights (so the routing is
near-uniform with natural skew). Input: 16 sequences of 4096 random tokens, split evenly over the ranks; each rank
runs its sequences one at a time (one MoE exchange per layer and sequence, all ranks in step). The training number
has no optimizer step (the configuration names forward + backward). The decode step feeds one new token per sequence
through key/value caches that already hold 4095 positions (zeros: the cost does not depend on the values).

``--layers 0`` (default) keeps all 32 layers when the experts, their gradients and the activations of one sequence
fit the device, and halves the depth otherwise (EP = 1 holds every expert: 32 layers are 90 GB of weights plus 90 GB of
gradients); the JSON line says how many layers ran. Timing: CUDA events around the whole pass, max over ranks; every
pass streams far more weight bytes than L2 holds.

The reference's counterpart is an fp32 single-GPU inference chain (benchmarks/bench_cuda_moe.cpp,
src/cuda/MoeForward.cu:188-298); it has neither a backward pass through that chain nor expert parallelism.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=0, help="0 = 32 if they fit the device, else 16, 8, ...")
    ap.add_argument("--batch", type=int, default=16, help="sequences in the global batch")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--decode-iters", type=int, default=8)
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if a.batch % world or a.experts % world:
        raise SystemExit("the batch and the experts must divide over the ranks")
    from tesseract_b200 import _native
    from tesseract_b200.models import LlamaConfig
    from tesseract_b200.parallel.ep_model import EPMoELlama

    heads = max(1, a.d_model // 128)
    el, b_local = a.experts // world, a.batch // world
    free_b, _total = torch.cuda.mem_get_info(dev)
    expert_layer = el * 3 * a.d_model * a.d_ff * 2                                # bf16 weights of one layer's local experts
    rows = min(2 * a.seq * a.top_k, world * a.seq * a.top_k) + el * 127            # rows a rank may receive in one call
    act_layer = rows * (a.d_model + 3 * a.d_ff) * 2 + a.seq * a.d_model * 2 * 14   # xs, h (2F), a (F); attention + norms
    layers = a.layers
    if layers <= 0:
        layers = 32
        while layers > 1:
            # weights + gradients + one transient weight-gradient buffer, activations of one sequence, replicated part
            need = expert_layer * (2 * layers + 1) + act_layer * layers + 8e9
            if need < 0.85 * free_b:
                break
            layers //= 2
    cfg = LlamaConfig(vocab_size=a.vocab, hidden_size=a.d_model, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=max(1, heads // 4), intermediate_size=a.d_ff,
                      max_position_embeddings=a.seq + 64, rope_theta=500000.0, num_experts=a.experts,
                      num_experts_per_tok=a.top_k, dtype=torch.bfloat16)
    ep = EPMoELlama(cfg, dist.group.WORLD if world > 1 else None, rank, world, dev, max_tokens=a.seq, exchange=a.exchange)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    tokens = torch.randint(0, a.vocab, (b_local, a.seq), device=dev, generator=g)
    targets = torch.randint(0, a.vocab, (b_local, a.seq), device=dev, generator=g)

    def reduce_max(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def train_pass():
        ep.zero_grad()
        loss = None
        for i in range(b_local):
            loss = ep.forward_backward(tokens[i:i + 1], targets[i:i + 1], scale=1.0 / a.batch)
        ep.reduce_replicated_grads()
        return loss

    for _ in range(a.warmup):
        train_pass()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        loss = train_pass()
    e1.record()
    torch.cuda.synchronize()
    train_ms = reduce_max(e0.elapsed_time(e1) / a.iters)
    loss = float(loss)
    peak_gb = reduce_max(torch.cuda.max_memory_allocated(dev) / 1e9)

    # ---- decode: one token per sequence against 4095 cached positions
    ep.zero_grad()
    torch.cuda.empty_cache()
    caches = ep.make_kv_caches(b_local, a.seq + 64)
    for c in caches:
        c.set_current_len(a.seq - 1)              # zero keys / values: the cost of a step does not depend on them
    nxt = torch.randint(0, a.vocab, (b_local, 1), device=dev, generator=g)
    for _ in range(3):
        ep.decode_step(nxt, caches)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.decode_iters):
        logits = ep.decode_step(nxt, caches)
    e1.record()
    torch.cuda.synchronize()
    decode_ms = reduce_max(e0.elapsed_time(e1) / a.decode_iters)
    finite = bool(torch.isfinite(logits.float()).all())
    status = int(reduce_max(_native.read_status(torch.cuda.current_stream().cuda_stream)))

    active = layers * (a.d_model * (a.d_model + 2 * (a.d_model // 4)) + a.d_model * a.d_model
                       + a.top_k * 3 * a.d_model * a.d_ff) + a.vocab * a.d_model
    tok = a.batch * a.seq
    if rank == 0:
        print(json.dumps({
            "bench": "moe_model", "ep": world, "layers": layers, "named_layers": 32, "experts": a.experts, "top_k": a.top_k,
            "d_model": a.d_model, "d_ff": a.d_ff, "vocab": a.vocab, "global_batch": a.batch, "seq_len": a.seq,
            "exchange": ep.exchange, "dtype": "bf16", "expert_gemm": "bf16 grouped tcgen05",
            "train_fwd_bwd_ms": round(train_ms, 2), "train_tok_s": round(tok / train_ms * 1e3, 1),
            "train_model_tflops_per_gpu": round(6.0 * active * tok / (train_ms * 1e-3) / world / 1e12, 1),
            "decode_step_ms": round(decode_ms, 3), "decode_tok_s": round(a.batch / decode_ms * 1e3, 1),
            "decode_context": a.seq - 1, "loss": round(loss, 4), "logits_finite": finite,
            "peak_mem_gb": round(peak_gb, 1), "param_bytes": ep.param_bytes(), "kernel_status": status,
            "optimizer": "none (forward + backward + replicated-gradient all-reduce)"}), flush=True)
    if world > 1:
        dist.barrier()
    ep.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
