#!/usr/bin/env python
"""Tensor-parallel Linear microbenchmark: fused GEMM+collective kernels against NCCL + a library GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        benchmarks/bench_tp_linear.py                          # the sweep below
    ... benchmarks/bench_tp_linear.py --tokens 32768 --shapes llama --parts --trace     # one size, with phase detail

Default sweep: tokens M in {128, 512, 2048, 8192, 16384}; shapes "square" (hidden K = N = 4096, row- and
column-parallel) and "mlp" (4096 -> 14336 column-parallel, 14336 -> 4096 row-parallel); ``--shapes llama`` adds the
Llama-8B attention projections (qkv 4096 -> 6144, gate_up 4096 -> 28672). For every case, on every rank with CUDA
events (L2 flushed between launches, max over ranks):

  * ``fused``        one kernel that multiplies while it moves tiles over NVLink peer memory
                     (row-parallel: GEMM -> reduce-scatter; column-parallel: all-gather -> GEMM); needs whole 128-row
                     tiles per rank, so sizes below 128 x TP rows have none;
  * ``nccl_cublas``  torch.distributed collective + ``torch.matmul`` (cuBLASLt): the unfused library baseline;
  * ``nccl_tcgen05`` the same collective + this repository's tcgen05 GEMM;
  * ``nccl_fp8``     the same collective + this repository's block-scaled fp8 GEMM (E4M3, 1 x 128 activation /
                     128 x 128 weight scales; the activation quantiser runs inside the timed region). There is no fused
                     fp8 kernel; the column is the unfused fp8 composition.

One JSON line per case with the times, the roofline time max(FLOPs / bf16 peak, NVLink bytes / link bandwidth) and
the achieved fractions; ``choice`` is what ``parallel.tp_layers`` runs at that size (fused only where it wins).
The reference's counterpart is an fp32 MLP + one all-reduce (benchmarks/bench_cuda_nccl_tp.cpp:88-222).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
# the benchmark compares the two implementations at every size: no size-based fallback inside the fused context
os.environ["TESSERACT_TP_FUSED_MIN_AG"] = "0"
os.environ["TESSERACT_TP_FUSED_MIN_RS"] = "0"


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", dest="m", type=int, nargs="+", default=[128, 512, 2048, 8192, 16384])
    ap.add_argument("--shapes", nargs="+", default=["square", "mlp"], choices=["square", "mlp", "llama"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--comm-ctas", type=int, default=16)
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured library bf16 GEMM rate (TFLOP/s)")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="NVLink bandwidth per direction per GPU (GB/s)")
    ap.add_argument("--no-fp8", action="store_true")
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
    from tesseract_b200.ops import fp8
    from tesseract_b200.parallel import tp_layers
    from tesseract_b200.parallel.fused_tp import FusedTP
    from tesseract_b200.parallel.tp_layers import TPContext, _mm, ag_matmul, matmul_rs

    peak = a.peak_tflops
    if peak <= 0:
        try:
            peak = json.load(open(os.environ["TESSERACT_PEAKS_FILE"]))["bf16_tflops"]
        except Exception:
            peak = 1590.0
    link_gbs = a.link_gbs
    fused = FusedTP(dist.group.WORLD, rank, world, dev, comm_ctas=a.comm_ctas)
    ctx_f = TPContext(dist.group.WORLD, rank, world, impl="fused", fused=fused)
    ctx_n = TPContext(dist.group.WORLD, rank, world, impl="nccl")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    prod_min = {"ag": 8192, "rs": 1024}          # the thresholds parallel.tp_layers uses outside this benchmark

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
    cases = []
    if "square" in a.shapes:
        cases += [("gemm_rs", "square_row", d // world, d), ("ag_gemm", "square_col", d, d // world)]
    if "mlp" in a.shapes:
        cases += [("ag_gemm", "mlp_up", d, ff // world), ("gemm_rs", "mlp_down", ff // world, d)]
    if "llama" in a.shapes:
        cases += [("gemm_rs", "o_proj", d // world, d), ("gemm_rs", "down_proj", ff // world, d),
                  ("ag_gemm", "qkv", d, qkv // world), ("ag_gemm", "gate_up", d, 2 * ff // world)]
    for M in a.m:
        if M % world:
            continue
        fused_ok = M % (128 * world) == 0
        for op, name, K, N in cases:
            if a.only and op != a.only:
                continue
            extra = {}
            g = torch.Generator(device=dev).manual_seed(rank + M)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
            wq = fp8.quantize_weight(w) if (not a.no_fp8 and K % 128 == 0) else None
            tf = err = None
            if op == "gemm_rs":
                x = torch.randn(M, K, device=dev, generator=g).bfloat16()
                if fused_ok:
                    tf = timed(lambda: matmul_rs(ctx_f, x, w))
                    err = (matmul_rs(ctx_f, x, w).float() - matmul_rs(ctx_n, x, w).float()).abs().max().item()
                tn = timed(lambda: matmul_rs(ctx_n, x, w))
                tc = timed(lambda: ctx_n.reduce_scatter_rows(torch.matmul(x, w.t())))
                tg = timed(lambda: _mm(x, w))
                t8 = None
                if wq is not None:
                    def rs_fp8():
                        qa, sa = fp8.quantize_act(x)
                        return ctx_n.reduce_scatter_rows(fp8.fp8_gemm(qa, sa, wq[0], wq[1]))
                    t8 = timed(rs_fp8)
            else:
                x = torch.randn(M // world, K, device=dev, generator=g).bfloat16()
                if fused_ok:
                    tf = timed(lambda: ag_matmul(ctx_f, x, w))
                    err = (ag_matmul(ctx_f, x, w)[0].float() - ag_matmul(ctx_n, x, w)[0].float()).abs().max().item()
                tn = timed(lambda: ag_matmul(ctx_n, x, w))
                tc = timed(lambda: torch.matmul(ctx_n.all_gather_rows(x), w.t()))
                xf = ctx_n.all_gather_rows(x)
                tg = timed(lambda: _mm(xf, w))
                t8 = None
                if wq is not None:
                    def ag_fp8():
                        qa, sa = fp8.quantize_act(ctx_n.all_gather_rows(x))
                        return fp8.fp8_gemm(qa, sa, wq[0], wq[1])
                    t8 = timed(ag_fp8)
                if a.trace and fused_ok:
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
                if a.parts and fused_ok:
                    extra.update({"fused_nokeep_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False)), 4),
                                  "push_only_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False, phase_mask=1)), 4),
                                  "mult_only_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=False, phase_mask=2)), 4),
                                  "mult_keep_ms": round(timed(lambda: fused.ag_gemm(x, w, keep=True, phase_mask=2)), 4)})
            flops = 2.0 * M * N * K
            link_bytes = (world - 1) / world * M * d * 2      # bf16 activations crossing NVLink per GPU
            roof_ms = max(flops / (peak * 1e12), link_bytes / (link_gbs * 1e9)) * 1e3
            status = _native.read_status(torch.cuda.current_stream().cuda_stream)
            kind = "rs" if op == "gemm_rs" else "ag"
            choice = "fused" if (fused_ok and M >= prod_min[kind]) else "nccl"
            if kind == "ag" and N < 1024 and M < 32768:
                choice = "nccl"                    # the rule of parallel.tp_layers for gathers with few columns per rank
            if rank == 0:
                r4 = lambda v: None if v is None else round(v, 4)   # noqa: E731
                best_unfused = min(tn, tc)
                print(json.dumps({
                    "op": op, "layer": name, "tp": world, "M": M, "N": N, "K": K, "fused_ms": r4(tf),
                    "nccl_cublas_ms": r4(tc), "nccl_tcgen05_ms": r4(tn), "nccl_fp8_ms": r4(t8), "gemm_only_ms": r4(tg),
                    "speedup_vs_nccl_cublas": None if tf is None else round(tc / tf, 3),
                    "roofline_ms": round(roof_ms, 4), "link_gbs": link_gbs,
                    "fused_frac_of_roofline": None if tf is None else round(roof_ms / tf, 3),
                    "nccl_cublas_frac_of_roofline": round(roof_ms / tc, 3), "max_abs_diff": err,
                    "bound": "compute" if flops / (peak * 1e12) > link_bytes / (link_gbs * 1e9) else "link",
                    "choice": choice, "choice_ms": r4(tf if choice == "fused" else tn),
                    "choice_is_fastest_bf16": (tf if choice == "fused" else tn) <= 1.03 * min(best_unfused, tf or 1e9),
                    "kernel_status": status, **extra}), flush=True)
            del w, x, wq
    dist.barrier()
    fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
