#!/usr/bin/env python
"""One hot kernel at a time, on one GPU, at a size that is larger than L2 but small enough to profile.

    python benchmarks/kernel_cases.py --case gemm            # one case
    python benchmarks/kernel_cases.py --case all             # every case, one JSON line each
    ncu --set full --clock-control none -k regex:gemm_bf16_kernel -s 3 -c 1 -o prof \
        python benchmarks/kernel_cases.py --case gemm --iters 1

Every case warms up, then times ``--iters`` launches with CUDA events (an L2 flush between launches) and prints
the achieved rate next to the measured peak it is bounded by (copy bandwidth / cuBLAS bf16 rate of this machine,
given with --hbm-gbs / --bf16-tflops or a JSON file named by --peaks-file / $TESSERACT_PEAKS_FILE). The fused tensor-parallel kernels run here as
an emulation of two ranks on one GPU: all buffers local, the gather kernel split into its push half and its
multiply half so that no launch waits for a later one.
Shapes follow the reference's microbenchmarks where it has one (benchmarks/bench_cuda_matmul.cpp,
bench_cuda_fused_attention.cpp, bench_cuda_moe.cpp, bench_cuda_mamba_scaling.cpp, bench_cuda_fp8_gemm.cpp).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "default"}


def set_peaks(hbm_gbs=None, bf16_tflops=None, peaks_file=None):
    """The denominators of the reported fractions: --hbm-gbs / --bf16-tflops, or a JSON file with the keys
    ``hbm_gbs`` and ``bf16_tflops`` (--peaks-file or $TESSERACT_PEAKS_FILE), else 6650 GB/s and 1590 TFLOP/s."""
    path = peaks_file or os.environ.get("TESSERACT_PEAKS_FILE", "")
    if path:
        d = json.load(open(path))
        _PEAKS.update(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]), src="measured")
    if hbm_gbs:
        _PEAKS.update(hbm_gbs=float(hbm_gbs), src="given")
    if bf16_tflops:
        _PEAKS.update(bf16_tflops=float(bf16_tflops), src="given")


def peaks():
    return _PEAKS["hbm_gbs"], _PEAKS["bf16_tflops"], _PEAKS["src"]


class Bench:
    def __init__(self, iters: int):
        self.dev = torch.device("cuda", 0)
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        self.gen = torch.Generator(device=self.dev).manual_seed(0)

    def randn(self, *shape, scale=1.0):
        return (torch.randn(*shape, device=self.dev, generator=self.gen) * scale).bfloat16()

    def time(self, fn, warmup=2):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / self.iters


def report(name, ms, flops=None, bytes_=None, **extra):
    hbm, tf, src = peaks()
    out = {"case": name, "ms": round(ms, 4)}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out["frac_of_hbm_peak"] = round(bytes_ / ms / 1e6 / hbm, 3)
    out["peaks"] = src
    out.update(extra)
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------- cases
def case_gemm(b: Bench):
    from tesseract_b200.ops import gemm_bf16
    M = N = K = 8192
    a, w = b.randn(M, K), b.randn(N, K, scale=0.02)
    out = torch.empty(M, N, device=b.dev, dtype=torch.bfloat16)
    ms = b.time(lambda: gemm_bf16(a, w, out=out))
    report("gemm", ms, flops=2.0 * M * N * K, shape=[M, N, K])


def case_gemm_wgrad(b: Bench):
    from tesseract_b200.ops import gemm_bf16
    T, N, K = 16384, 4096, 4096
    dy, x = b.randn(T, N), b.randn(T, K)
    dw = torch.zeros(N, K, device=b.dev, dtype=torch.float32)
    ms = b.time(lambda: gemm_bf16(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True))
    report("gemm_wgrad", ms, flops=2.0 * T * N * K, shape=[N, K, T])


def case_gemm_fp8(b: Bench):
    from tesseract_b200.ops import fp8
    M = N = K = 8192
    qa, sa = fp8.quantize_act(b.randn(M, K))
    qb, sb = fp8.quantize_weight(b.randn(N, K, scale=0.02))
    ms = b.time(lambda: fp8.fp8_gemm(qa, sa, qb, sb))
    report("gemm_fp8", ms, flops=2.0 * M * N * K, shape=[M, N, K], note="fractions are of the bf16 peak")


def case_gemm_fp8_pertensor(b: Bench):
    """The reference's FP8 benchmark shape family (square, one scale per operand); its bar is FP8 >= 1.3 x FP16
    (benchmarks/bench_cuda_fp8_gemm.cpp:156-159): the 16-bit product of the same shape is timed next to it."""
    from tesseract_b200.ops import fp8, gemm_bf16
    for n in (4096, 8192):
        x, w = b.randn(n, n), b.randn(n, n, scale=0.02)
        qa, sa = fp8.quantize_tensor(x)
        qb, sb = fp8.quantize_tensor(w)
        ms8 = b.time(lambda: fp8.fp8_gemm_pertensor(qa, sa, qb, sb))
        out = torch.empty(n, n, device=b.dev, dtype=torch.bfloat16)
        ms16 = b.time(lambda: gemm_bf16(x, w, out=out))
        report(f"gemm_fp8_pertensor_{n}", ms8, flops=2.0 * n ** 3, shape=[n, n, n], bf16_ms=round(ms16, 4),
               fp8_over_bf16=round(ms16 / ms8, 3), note="fractions are of the bf16 peak")


def case_decode_gemm(b: Bench):
    """Weight-streaming GEMMs of one decode step (Llama-8B layer shapes) at 64 and 256 rows."""
    from tesseract_b200 import ops
    for M in (64, 256):
        tot_ms, tot_bytes = 0.0, 0
        for name, N, K in (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
            x, w = b.randn(M, K), b.randn(N, K, scale=0.02)
            ms = b.time(lambda: ops.decode_linear(x, w))
            tot_ms += ms
            tot_bytes += N * K * 2
            report(f"decode_gemm_{name}_M{M}", ms, bytes_=N * K * 2, shape=[M, N, K])
        report(f"decode_gemm_layer_M{M}", tot_ms, bytes_=tot_bytes)


def case_stream_linear(b: Bench):
    """The weight-streaming decode GEMM (bf16 and block-scaled fp8 weights) on the layer shapes of one decode step,
    next to the cluster split-K kernel it replaces; bytes = the weight matrix once."""
    from tesseract_b200 import ops
    from tesseract_b200.ops import fp8
    for M in (16, 64, 141, 256):
        tot = {"bf16": [0.0, 0], "fp8": [0.0, 0], "old": [0.0, 0]}
        for name, N, K in (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
            x, w = b.randn(M, K), b.randn(N, K, scale=0.02)
            q, sc = fp8.quantize_weight(w)
            ms_old = b.time(lambda: ops.decode_linear(x, w))
            ms_bf = b.time(lambda: ops.stream_linear(x, w))
            ms_f8 = b.time(lambda: ops.stream_linear(x, q, sc))
            for key, ms, nbytes in (("old", ms_old, N * K * 2), ("bf16", ms_bf, N * K * 2), ("fp8", ms_f8, N * K)):
                tot[key][0] += ms
                tot[key][1] += nbytes
            report(f"stream_linear_bf16_{name}_M{M}", ms_bf, bytes_=N * K * 2, shape=[M, N, K], cluster_splitk_ms=round(ms_old, 4))
            report(f"stream_linear_fp8_{name}_M{M}", ms_f8, bytes_=N * K, shape=[M, N, K])
        for key in ("old", "bf16", "fp8"):
            report(f"stream_linear_layer_{key}_M{M}", tot[key][0], bytes_=tot[key][1])


def case_gemm_mx(b: Bench):
    """Block-scaled fp8 GEMM on the tensor core's own block scaling (E4M3 x E4M3, power-of-two scales, persistent
    128 x 192 tiles), next to the bf16 GEMM of the same shape; the activation quantiser is timed separately."""
    import os

    from tesseract_b200.ops import fp8, gemm_bf16
    shapes = ((8192, 8192, 8192), (16384, 4096, 4096), (16384, 28672, 4096), (16384, 4096, 14336))
    if os.environ.get("TESSERACT_KERNEL_CASES_SMALL", "0") == "1":
        shapes = shapes[:1]                                   # one shape for a profiler capture
    for M, N, K in shapes:
        a, w = b.randn(M, K), b.randn(N, K, scale=0.02)
        wq, ws = fp8.quantize_weight(w, pow2=True)
        q, sf = fp8.quantize_act_mx(a, atoms=True)
        wa = fp8.weight_scale_atoms(ws)
        out = torch.empty(M, N, device=b.dev, dtype=torch.bfloat16)
        ms = b.time(lambda: fp8.mx_linear(q, sf, wq, ws, out=out, w_atoms=wa))
        ms_bf = b.time(lambda: gemm_bf16(a, w, out=out))
        ms_q = b.time(lambda: fp8.quantize_act_mx(a, out=(q, sf), atoms=True))
        report(f"gemm_mx_{M}x{N}x{K}", ms, flops=2.0 * M * N * K, shape=[M, N, K], bf16_gemm_ms=round(ms_bf, 4),
               speedup_over_bf16=round(ms_bf / ms, 3), quantiser_ms=round(ms_q, 4))


def case_mx_linear(b: Bench):
    """The block-scaled fp8 decode GEMM on tcgen05.mma kind::mxf8f6f4 (E4M3 activations and weights, power-of-two
    scales applied by the tensor core) on the layer shapes of one decode step; bytes = the fp8 weight matrix once.
    ``with_quant`` adds the stand-alone activation quantiser in front (the serving engine fuses it into RMSNorm /
    SwiGLU instead); ``TESSERACT_KERNEL_CASES_SMALL=1`` runs one shape only (a profiler capture)."""
    import os

    from tesseract_b200.ops import fp8
    small = os.environ.get("TESSERACT_KERNEL_CASES_SMALL", "0") == "1"
    shapes = (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336))
    for M in ((32,) if small else (16, 32, 64, 128, 256)):
        tot = [0.0, 0.0, 0]
        for name, N, K in (shapes[2:3] if small else shapes):
            x, w = b.randn(M, K), b.randn(N, K, scale=0.02)
            wq, ws = fp8.quantize_weight(w, pow2=True)
            q, sf = fp8.quantize_act_mx(x)
            ms = b.time(lambda: fp8.mx_linear(q, sf, wq, ws))
            # (not in the small profiler case: it launches with the programmatic-serialisation attribute)
            ms_q = ms if small else b.time(lambda: fp8.mx_linear(*fp8.quantize_act_mx(x, out=(q, sf)), wq, ws, pdl=True))
            tot[0] += ms
            tot[1] += ms_q
            tot[2] += N * K
            bn, split, stages, _ = fp8.mx_linear_plan(M, N, K)
            report(f"mx_linear_{name}_M{M}", ms, bytes_=N * K, shape=[M, N, K], with_quant_ms=round(ms_q, 4),
                   tile=bn, k_split=split, stages=stages)
        report(f"mx_linear_layer_M{M}", tot[0], bytes_=tot[2], with_quant_ms=round(tot[1], 4))


def case_grouped_gemm(b: Bench):
    from tesseract_b200.ops import moe
    E, N, K, per = 8, 4096, 4096, 2048
    offsets = torch.arange(E + 1, device=b.dev, dtype=torch.int32) * per
    a, w = b.randn(E * per, K), b.randn(E, N, K, scale=0.02)
    ms = b.time(lambda: moe.grouped_gemm_rows(a, w[0], N * K, offsets, E))
    report("grouped_gemm", ms, flops=2.0 * E * per * N * K, shape=[E, per, N, K])


def _qkv(b: Bench, B, S, H, Hkv, D):
    return b.randn(B, S, H + 2 * Hkv, D)


def case_flash_fwd(b: Bench):
    from tesseract_b200.ops import flash_attention_packed
    B, S, H, Hkv, D = 2, 4096, 32, 8, 128
    qkv = _qkv(b, B, S, H, Hkv, D)
    with torch.no_grad():
        ms = b.time(lambda: flash_attention_packed(qkv, H, Hkv, causal=True))
    report("flash_fwd", ms, flops=4.0 * B * H * S * S * D / 2, shape=[B, S, H, Hkv, D])


def case_flash_bwd(b: Bench):
    from tesseract_b200.ops import flash_attention_packed
    B, S, H, Hkv, D = 2, 4096, 32, 8, 128
    qkv = _qkv(b, B, S, H, Hkv, D).requires_grad_(True)
    o = flash_attention_packed(qkv, H, Hkv, causal=True)
    do = torch.randn_like(o)

    def run():
        qkv.grad = None
        o.backward(do, retain_graph=True)
    ms = b.time(run)
    report("flash_bwd", ms, flops=10.0 * B * H * S * S * D / 2, shape=[B, S, H, Hkv, D])


def _paged(b: Bench, A, L, int8):
    H, Hkv, D, bs = 32, 8, 128, 16
    mb = (L + bs - 1) // bs
    nb = A * mb + 1
    if int8:
        k = torch.randint(-127, 127, (nb, Hkv, bs, D), device=b.dev, dtype=torch.int8)
        v = torch.randint(-127, 127, (nb, Hkv, bs, D), device=b.dev, dtype=torch.int8)
        ks, vs = torch.rand(nb, Hkv, bs, device=b.dev), torch.rand(nb, Hkv, bs, device=b.dev)
    else:
        k, v, ks, vs = b.randn(nb, Hkv, bs, D), b.randn(nb, Hkv, bs, D), None, None
    tables = torch.randperm(nb - 1, device=b.dev)[:A * mb].view(A, mb).int()
    lens = torch.full((A,), L, device=b.dev, dtype=torch.int32)
    q = b.randn(A, H, D)
    return q, k, v, tables, lens, ks, vs, A * L * Hkv * D * 2 * (1 if int8 else 2)


def case_decode(b: Bench):
    from tesseract_b200 import ops
    q, k, v, tables, lens, ks, vs, nbytes = _paged(b, 256, 1400, False)
    ms = b.time(lambda: ops.paged_decode_attention(q, k, v, tables, lens, None, ks, vs, max_len_hint=2560))
    report("decode", ms, bytes_=nbytes, shape=[256, 1400])


def case_decode_int8(b: Bench):
    from tesseract_b200 import ops
    q, k, v, tables, lens, ks, vs, nbytes = _paged(b, 256, 1400, True)
    ms = b.time(lambda: ops.paged_decode_attention(q, k, v, tables, lens, None, ks, vs, max_len_hint=2560))
    report("decode_int8", ms, bytes_=nbytes, shape=[256, 1400])


def case_rmsnorm(b: Bench):
    from tesseract_b200 import ops
    x, w = b.randn(32768, 4096), torch.ones(4096, device=b.dev, dtype=torch.bfloat16)
    with torch.no_grad():
        ms = b.time(lambda: ops.rms_norm(x, w, 1e-5))
    report("rmsnorm", ms, bytes_=2 * x.numel() * 2, shape=list(x.shape))


def case_swiglu(b: Bench):
    from tesseract_b200 import ops
    x = b.randn(16384, 2 * 14336)
    with torch.no_grad():
        ms = b.time(lambda: ops.swiglu(x))
    report("swiglu", ms, bytes_=x.numel() * 2 * 1.5, shape=list(x.shape))


def case_swiglu_bwd(b: Bench):
    from tesseract_b200.ops import fused
    x = b.randn(16384, 2 * 14336)
    d = b.randn(16384, 14336)
    ms = b.time(lambda: fused.swiglu_backward(x, d))
    report("swiglu_bwd", ms, bytes_=d.numel() * 2 * 5, shape=list(x.shape))


def case_adam(b: Bench):
    from tesseract_b200 import _native
    from tesseract_b200.optim import optimizers  # noqa: F401  (registers the signatures of loss_optim.cu)
    n = 256 << 20
    p = torch.zeros(n, device=b.dev, dtype=torch.bfloat16)
    g = torch.zeros(n, device=b.dev, dtype=torch.bfloat16)
    m = torch.zeros(n, device=b.dev, dtype=torch.float32)
    v = torch.zeros(n, device=b.dev, dtype=torch.float32)
    s = torch.cuda.current_stream().cuda_stream
    lib = _native.lib()
    ms = b.time(lambda: _native.check(lib.tsb_adam_flat(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), None, n,
                                                        1e-4, 0.9, 0.999, 1e-8, 0.1, 0.001, 0.0, None, 1, 1, s),
                                      "tsb_adam_flat"))
    report("adam", ms, bytes_=n * (2 + 2 + 4 + 4 + 2 + 4 + 4), shape=[n])


def case_ce(b: Bench):
    from tesseract_b200 import ops
    T, V = 4096, 128256
    logits = b.randn(T, V)
    tgt = torch.randint(0, V, (T,), device=b.dev)
    ms = b.time(lambda: ops.ce_stats(logits, tgt))
    report("ce_stats", ms, bytes_=T * V * 2, shape=[T, V])


def case_scan(b: Bench):
    from tesseract_b200.ops import ssm
    B, L, D, N = 4, 4096, 4096, 16
    u = torch.randn(B, L, D, device=b.dev, generator=b.gen)
    delta = torch.rand(B, L, D, device=b.dev, generator=b.gen) * 0.1
    A = -torch.rand(D, N, device=b.dev, generator=b.gen)
    Bm = torch.randn(B, L, N, device=b.dev, generator=b.gen)
    C = torch.randn(B, L, N, device=b.dev, generator=b.gen)
    Dv = torch.ones(D, device=b.dev)
    with torch.no_grad():
        ms = b.time(lambda: ssm.selective_scan(u, delta, A, Bm, C, Dv))
    report("selective_scan", ms, bytes_=3 * B * L * D * 4, shape=[B, L, D, N])


def case_gemv(b: Bench):
    from tesseract_b200 import quant
    N, K = 14336, 4096
    w = torch.randn(N, K, device=b.dev, generator=b.gen)
    q8, s8 = (t.to(b.dev) for t in quant.pack_int8_symmetric(w))     # the packer works on the host
    x = b.randn(1, K)
    ms = b.time(lambda: quant.dequantize_matmul_int8(x, q8, s8))
    report("gemv_w8", ms, bytes_=N * K, shape=[1, N, K])


def _ptrs(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def case_gemm_rs_emul(b: Bench):
    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401
    lib = _native.lib()
    world, rpr, N, K = 2, 4096, 4096, 2048
    M = world * rpr
    x, w = b.randn(M, K), b.randn(N, K, scale=0.02)
    staging = [torch.empty(world, rpr, N, device=b.dev, dtype=torch.bfloat16) for _ in range(world)]
    pa = _ptrs(staging)
    s = torch.cuda.current_stream().cuda_stream
    ms = b.time(lambda: _native.check(lib.tsb_gemm_rs(x.data_ptr(), w.data_ptr(), pa, M, N, K, x.stride(0), w.stride(0),
                                                      0, rpr, 0, world, s), "tsb_gemm_rs"))
    report("gemm_rs_emul", ms, flops=2.0 * M * N * K, shape=[M, N, K], note="rank 0 of 2, peers on the same GPU")


def case_ag_gemm_emul(b: Bench):
    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401
    lib = _native.lib()
    world, rpr, N, K = 2, 4096, 3072, 4096
    M = world * rpr
    shards = [b.randn(rpr, K) for _ in range(world)]
    w = b.randn(N, K, scale=0.02)
    lands = [torch.empty(M, K, device=b.dev, dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=b.dev) for _ in range(world)]
    y = torch.empty(M, N, device=b.dev, dtype=torch.bfloat16)
    pl, pf = _ptrs(lands), _ptrs(flags)
    s = torch.cuda.current_stream().cuda_stream
    calls = [0]

    def call(rank, mask):
        _native.check(lib.tsb_gemm_ag(shards[rank].data_ptr(), pl, pf, None, w.data_ptr(), y.data_ptr(), calls[0], 1,
                                      mask, M, N, K, w.stride(0), y.stride(0), 0, rpr, rank, world, None, s),
                      "tsb_gemm_ag")

    def push_all():
        calls[0] += 1
        for r in range(world):
            call(r, 1)
    push_all()
    ms_mult = b.time(lambda: call(0, 2))
    ms_push = b.time(push_all) / world
    report("ag_gemm_emul", ms_mult, flops=2.0 * M * N * K, shape=[M, N, K], push_ms=round(ms_push, 4),
           note="multiply half of rank 0 of 2 after both ranks' push halves; push_ms = one rank's push half alone")


CASES = {"gemm": case_gemm, "gemm_fp8": case_gemm_fp8, "gemm_fp8_pertensor": case_gemm_fp8_pertensor, "decode_gemm": case_decode_gemm, "gemm_wgrad": case_gemm_wgrad, "grouped_gemm": case_grouped_gemm,
         "flash_fwd": case_flash_fwd, "flash_bwd": case_flash_bwd, "decode": case_decode,
         "decode_int8": case_decode_int8, "rmsnorm": case_rmsnorm, "swiglu": case_swiglu, "swiglu_bwd": case_swiglu_bwd, "adam": case_adam,
         "ce_stats": case_ce, "selective_scan": case_scan, "gemv_w8": case_gemv, "gemm_rs_emul": case_gemm_rs_emul,
         "ag_gemm_emul": case_ag_gemm_emul, "stream_linear": case_stream_linear, "mx_linear": case_mx_linear, "gemm_mx": case_gemm_mx}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all"] + sorted(CASES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--hbm-gbs", type=float, default=0.0, help="measured copy bandwidth of this GPU (GB/s)")
    ap.add_argument("--bf16-tflops", type=float, default=0.0, help="measured library bf16 GEMM rate of this GPU")
    ap.add_argument("--peaks-file", default="", help="JSON file with hbm_gbs and bf16_tflops")
    a = ap.parse_args()
    set_peaks(a.hbm_gbs, a.bf16_tflops, a.peaks_file)
    from tesseract_b200 import _native
    names = sorted(CASES) if a.case == "all" else [a.case]
    for n in names:
        CASES[n](Bench(a.iters))
        torch.cuda.synchronize()
    status = _native.read_status(torch.cuda.current_stream().cuda_stream)
    if status:
        print(json.dumps({"kernel_status": status}))
        sys.exit(1)


if __name__ == "__main__":
    main()
