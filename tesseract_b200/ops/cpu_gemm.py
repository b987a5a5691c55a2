"""Native CPU FP32 GEMM (``csrc/host/gemm_f32.cpp``: a 14 x 32 AVX-512 or 6 x 16 AVX2 register tile chosen at run
time, unpacked up to 512^3 and packed panels above, OpenMP with a work-proportional thread count capped by
``TESSERACT_GEMM_MAX_THREADS``).

The reference's CPU ``ops::matmul`` runs an AVX2 4 x 8 FMA microkernel with an adaptive thread cap
(src/ops/cpu/GemmAvx2.cpp:25-150); this is the host-runtime counterpart. torch CPU tensors normally go through
torch's own matmul (a vendor BLAS); with ``TESSERACT_CPU_GEMM=native`` the frontend's ``ops.matmul`` sends 2-D fp32
CPU products (forward and both backward products) here through ``matmul``. ``benchmarks/bench_cpu.py --case matmul``
times it beside the vendor BLAS.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .. import _native


def _host():
    if os.environ.get("TESSERACT_HOST", "") == "python":
        return None
    return _native.host()


def gemm_avx2_supported() -> bool:
    h = _host()
    return bool(h.gemm_avx2_supported()) if h is not None else False


def gemm_num_threads(M: int, N: int, K: int, requested: int = 0) -> int:
    """Threads the native GEMM uses for this problem (about half a MFLOP per thread, at most one per 6-row strip, capped by
    ``TESSERACT_GEMM_MAX_THREADS`` and ``requested``)."""
    h = _host()
    if h is None:
        return 1
    return int(h.gemm_num_threads(M, N, K, requested))


def matmul_f32(a: torch.Tensor, b: torch.Tensor, b_is_nk: bool = False, threads: int = 0) -> torch.Tensor:
    """a [M, K] @ b [K, N] (or b^T with ``b_is_nk``: b stored [N, K], the layout of a Linear weight), fp32 on the CPU."""
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("matmul_f32: matrices expected")
    if (b.shape[1] if b_is_nk else b.shape[0]) != a.shape[1]:
        raise ValueError("matmul_f32: inner dimensions differ")
    h = _host()
    if h is None or a.is_cuda or b.is_cuda:
        return a.float() @ (b.float().t() if b_is_nk else b.float())
    an = np.ascontiguousarray(a.detach().float().numpy())
    bn = np.ascontiguousarray(b.detach().float().numpy())
    return torch.from_numpy(np.asarray(h.gemm_f32(an, bn, bool(b_is_nk), int(threads))))


def native_selected() -> bool:
    """``TESSERACT_CPU_GEMM=native`` and the host runtime is there."""
    return os.environ.get("TESSERACT_CPU_GEMM", "torch") == "native" and _host() is not None


class _NativeMatmul(torch.autograd.Function):
    """a [M, K] @ b [K, N] with the native GEMM in the forward pass and in both backward products."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return matmul_f32(a, b)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = g.contiguous()
        ga = matmul_f32(g, b, b_is_nk=True) if ctx.needs_input_grad[0] else None          # g @ b^T: b is [K, N] = [out, inner]
        gb = matmul_f32(a.t().contiguous(), g) if ctx.needs_input_grad[1] else None       # a^T @ g
        return ga, gb


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Differentiable 2-D fp32 CPU product on the native GEMM."""
    return _NativeMatmul.apply(a, b)
