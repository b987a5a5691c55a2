"""Native CPU FP32 GEMM (``csrc/host/gemm_f32.cpp``: AVX2 / FMA 6 x 16 register tile, packed panels, OpenMP over row
blocks with a work-proportional thread count capped by ``TESSERACT_GEMM_MAX_THREADS``).

The reference's CPU ``ops::matmul`` runs an AVX2 4 x 8 FMA microkernel with an adaptive thread cap
(src/ops/cpu/GemmAvx2.cpp:25-150); this is the host-runtime counterpart. torch CPU tensors normally go through
torch's own matmul (a vendor BLAS); ``TESSERACT_CPU_GEMM=native`` routes 2-D fp32 products of ``matmul_f32`` here,
which is also what the CPU benchmark (``benchmarks/reference_bars.py --case cpu_gemm``) times.
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
    """Threads the native GEMM uses for this problem (about 2 MFLOP per thread, at most one per 6-row strip, capped by
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
