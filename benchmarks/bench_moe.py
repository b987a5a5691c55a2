#!/usr/bin/env python
"""Mixture-of-experts layer benchmark: grouped-GEMM experts on one GPU, expert-parallel over N ranks.

    python benchmarks/bench_moe.py                         # one GPU: all 8 experts local
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29650 \
        benchmarks/bench_moe.py                            # EP = 8: one expert per rank, all-to-all dispatch / combine

Layer of the MoE north-star configuration: 8 experts, top-2 softmax router, d_model 4096, expert FFN 14336 (SwiGLU),
bf16; tokens = batch x seq per rank (random activations, router logits from random weights). Times forward and
forward + backward with CUDA events (max over ranks, L2 flushed between iterations) and reports the expert-GEMM
FLOP rate. The reference's counterpart is an fp32 single-GPU inference kernel chain with a host synchronisation
in the middle (benchmarks/bench_cuda_moe.cpp, src/cuda/MoeForward.cu:188-298).
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
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per rank")
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="expert-parallel token exchange: device-side pushes over peer memory, or NCCL all-to-all")
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from tesseract_b200 import _native
    from tesseract_b200.nn.moe import MoEFeedForward
    from tesseract_b200.parallel.expert import ExpertParallel

    torch.manual_seed(5)
    el = a.experts // world
    # build only this rank's experts (the router is replicated): a full 8-expert layer is 2.8 GB in bf16
    layer = MoEFeedForward(a.d_model, a.d_ff, num_experts=el, num_experts_per_tok=min(a.top_k, el), dtype=torch.bfloat16,
                           device=dev)
    if world > 1:
        from tesseract_b200.nn.modules import Linear
        layer.gate = Linear(a.d_model, a.experts, bias=False, dtype=torch.bfloat16, device=dev)
        layer.num_experts, layer.top_k = a.experts, a.top_k
        for p in layer.gate.parameters():
            dist.broadcast(p.data, src=0)
        if a.exchange == "fused":
            from tesseract_b200.parallel.expert import FusedExpertParallel
            FusedExpertParallel(dist.group.WORLD, rank, world, dev, a.d_model, a.experts, a.top_k,
                                max_tokens=a.tokens).shard_(layer)
        else:
            ExpertParallel(dist.group.WORLD, rank, world).shard_(layer)
    for p in layer.parameters():
        p.data.mul_(0.5)
    x = torch.randn(a.tokens, a.d_model, device=dev).bfloat16().requires_grad_(True)
    dout = torch.randn(a.tokens, a.d_model, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(2):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        t = torch.tensor([tot / a.iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def fwd():
        with torch.no_grad():
            return layer(x)

    def fwd_bwd():
        x.grad = None
        for p in layer.parameters():
            p.grad = None
        layer(x).backward(dout)

    ms_f, ms_fb = timed(fwd), timed(fwd_bwd)
    flops_f = 2.0 * a.tokens * a.top_k * 3 * a.d_model * a.d_ff          # per rank's tokens, expert GEMMs only
    status = _native.read_status(torch.cuda.current_stream().cuda_stream)
    if rank == 0:
        print(json.dumps({"bench": "moe_layer", "ep": world, "tokens_per_rank": a.tokens, "experts": a.experts,
                          "top_k": a.top_k, "exchange": a.exchange if world > 1 else "local", "d_model": a.d_model, "d_ff": a.d_ff, "fwd_ms": round(ms_f, 3),
                          "fwd_bwd_ms": round(ms_fb, 3), "fwd_tflops_per_gpu": round(flops_f / ms_f / 1e9, 1),
                          "fwd_bwd_tflops_per_gpu": round(3 * flops_f / ms_fb / 1e9, 1), "kernel_status": status}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
