#!/usr/bin/env python
"""CPU decode GEMV: INT8 weights x INT8 activations (AVX-512-VNNI where the CPU has it) against the fp32 product,
on the projection shapes of one 7B-class block (the reference's benchmarks/bench_cpu_decode_vnni.cpp).

    python benchmarks/bench_cpu_decode_vnni.py [--gen 24] [--threads 0]

Prints one JSON line per shape with the time per call, the weight bandwidth and the speed-up over fp32; informational
(no bar), as in the reference.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tesseract_b200.ops import cpu_gemv  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gen", type=int, default=24, help="decode steps timed per shape")
    ap.add_argument("--threads", type=int, default=0, help="0: up to 16 hardware threads")
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=11008)
    a = ap.parse_args()
    g = torch.Generator().manual_seed(0)
    print(json.dumps({"vnni": cpu_gemv.gemv_vnni_supported(), "torch_threads": torch.get_num_threads()}))
    for name, (N, K) in (("qkv", (3 * a.d_model, a.d_model)), ("o_proj", (a.d_model, a.d_model)),
                         ("gate_up", (2 * a.d_ff, a.d_model)), ("down", (a.d_model, a.d_ff))):
        Wf = torch.randn(N, K, generator=g) * 0.02
        wscale = Wf.abs().amax(1) / 127.0
        W = torch.round(Wf / wscale[:, None]).to(torch.int8)
        rowsum = cpu_gemv.compute_row_sums(W)
        x = torch.randn(K, generator=g)
        for _ in range(2):
            xq, xs = cpu_gemv.quantize_row_int8(x)
            y8 = cpu_gemv.gemv_w8a8(W, wscale, rowsum, xq, xs, threads=a.threads)
            y32 = Wf @ x
        t0 = time.perf_counter()
        for _ in range(a.gen):
            xq, xs = cpu_gemv.quantize_row_int8(x)
            cpu_gemv.gemv_w8a8(W, wscale, rowsum, xq, xs, threads=a.threads)
        t8 = (time.perf_counter() - t0) / a.gen
        t0 = time.perf_counter()
        for _ in range(a.gen):
            Wf @ x
        t32 = (time.perf_counter() - t0) / a.gen
        rel = float((y8 - y32).norm() / y32.norm())
        print(json.dumps({"shape": name, "N": N, "K": K, "int8_us": round(t8 * 1e6, 1), "fp32_us": round(t32 * 1e6, 1),
                          "int8_gbs": round(N * K / t8 / 1e9, 1), "speedup_vs_fp32": round(t32 / t8, 2),
                          "rel_err_vs_fp32": round(rel, 4)}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
