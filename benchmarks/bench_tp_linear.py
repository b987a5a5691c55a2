#!/usr/bin/env python
"""Tensor-parallel Linear microbenchmark: fused GEMM+collective kernels against NCCL + GEMM back to back.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        benchmarks/bench_tp_linear.py --tokens 1024 4096 16384

For every token count M and the Llama-8B layer shapes it times, on every rank with CUDA events (max over ranks):
  * row-parallel  GEMM -> reduce-scatter   (o_proj: K = 4096 / tp, N = 4096; down_proj: K = 14336 / tp, N = 4096)
  * column-parallel all-gather -> GEMM     (qkv: N = 6144 / tp; gate_up: N = 28672 / tp; K = 4096)
in two implementations: ``fused`` (one kernel moves the tiles over NVLink peer memory while it multiplies) and
``nccl`` (torch.distributed collective + the same tcgen05 GEMM). It prints one JSON line per (op, shape) with both
times, the roofline time max(FLOPs / measured bf16 peak, NVLink bytes / 770 GB/s) and the achieved fractions.
The reference's counterpart is an fp32 MLP + one all-reduce (benchmarks/bench_cuda_nccl_tp.cpp:88-222).
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
    ap.add_argument("--tokens", dest="m", type=int, nargs="+", default=[1024, 4096, 16384, 32768])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--comm-ctas", type=int, default=16)
    ap.add_argument("--peak-tflops", type=float, default=0.0)
    ap.add_argument("--trace", action="store_true", help="print per-phase timestamps (min, max over CTAs) of one gather call")
    ap.add_argument("--only", default="", help="gemm_rs or ag_gemm: time only that op")
    ap.add_argument("--parts", action="store_true", help="also time the halves of the gather kernel separately")
    a = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    from tesseract_b200 import _native
    from tesseract_b200.parallel.fused_tp import FusedTP
    from tesseract_b200.parallel.tp_layers import TPContext, _mm, ag_matmul, matmul_rs

    peak = a.peak_tflops
    if peak <= 0:
        try:
            peak = json.load(open(os.environ["TESSERACT_PEAKS_FILE"]))["bf16_tflops"]
        except Exception:
            peak = 1590.0
    link_gbs = 770.0
    fused = FusedTP(dist.group.WORLD, rank, world, dev, comm_ctas=a.comm_ctas)
    ctx_f = TPContext(dist.group.WORLD, rank, world, impl="fused", fused=fused)
    ctx_n = TPContext(dist.group.WORLD, rank, world, impl="nccl")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(a.iters):
            flush.zero_()                                   # evict L2 between timed iterations
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    d, ff, qkv = 4096, 14336, 6144
    t_bar = timed(fused.barrier)
    if rank == 0:
        print(json.dumps({"op": "symm_barrier", "tp": world, "ms": round(t_bar, 4)}), flush=True)
    for M in a.m:
        if M % (128 * world):
            continue
        cases = [("gemm_rs", "o_proj", d // world, d), ("gemm_rs", "down_proj", ff // world, d),
                 ("ag_gemm", "qkv", d, qkv // world), ("ag_gemm", "gate_up", d, 2 * ff // world)]
        for op, name, K, N in cases:
            if a.only and op != a.only:
                continue
            extra = {}
            g = torch.Generator(device=dev).manual_seed(rank + M)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
            if op == "gemm_rs":
                x = torch.randn(M, K, device=dev, generator=g).bfloat16()
                tf = timed(lambda: matmul_rs(ctx_f, x, w))
                tn = timed(lambda: matmul_rs(ctx_n, x, w))
                tg = timed(lambda: _mm(x, w))
                err = (matmul_rs(ctx_f, x, w).float() - matmul_rs(ctx_n, x, w).float()).abs().max().item()
            else:
                x = torch.randn(M // world, K, device=dev, generator=g).bfloat16()
                tf = timed(lambda: ag_matmul(ctx_f, x, w))
                tn = timed(lambda: ag_matmul(ctx_n, x, w))
                xf = ctx_n.all_gather_rows(x)
                tg = timed(lambda: _mm(xf, w))
                err = (ag_matmul(ctx_f, x, w)[0].float() - ag_matmul(ctx_n, x, w)[0].float()).abs().max().item()
                if a.trace:
                    sms = torch.cuda.get_device_properties(dev).multi_processor_count
                    fused.trace = torch.zeros(sms, 8, dtype=torch.int64, device=dev)
                    dist.barrier()
                    torch.cuda.synchronize()
                    fused.ag_gemm(x, w, keep=True)
                    torch.cuda.synchronize()
                    tr = fused.trace.cpu().double()
                    fused.trace = None
                    t0 = tr[:, 0].min()
                    names = ["start", "remote_pushed", "all_pushed", "wait_begin", "wait_end", "loads_issued",
                             "epilogue_done", "kept"]
                    extra["trace_us"] = {n: [round(float((tr[:, i][tr[:, i] > 0].min() - t0) / 1e3), 1),
                                             round(float((tr[:, i].max() - t0) / 1e3), 1)]
                                         for i, n in enumerate(names) if (tr[:, i] > 0).any()}
                if a.parts:
                    extra.update({"fused_nokeep_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False)), 4),
                             "push_only_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False, phase_mask=1)), 4),
                             "mult_only_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False, phase_mask=2)), 4),
                             "mult_keep_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=True, phase_mask=2)), 4)})
            flops = 2.0 * M * N * K
            link_bytes = (world - 1) / world * M * d * 2      # bf16 activations crossing NVLink per GPU
            roof_ms = max(flops / (peak * 1e12), link_bytes / (link_gbs * 1e9)) * 1e3
            status = _native.read_status(torch.cuda.current_stream().cuda_stream)
            if rank == 0:
                print(json.dumps({"op": op, "layer": name, "tp": world, "M": M, "N": N, "K": K,
                                  "fused_ms": round(tf, 4), "nccl_ms": round(tn, 4), "gemm_only_ms": round(tg, 4), "speedup": round(tn / tf, 3),
                                  "roofline_ms": round(roof_ms, 4), "fused_frac_of_roofline": round(roof_ms / tf, 3),
                                  "nccl_frac_of_roofline": round(roof_ms / tn, 3), "max_abs_diff": err,
                                  "bound": "compute" if flops / (peak * 1e12) > link_bytes / (link_gbs * 1e9) else "link",
                                  "kernel_status": status, **extra}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
