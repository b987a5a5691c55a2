"""CPU decode GEMV with INT8 weights and INT8 activations (W8A8): ``quantize_row_int8``, ``compute_row_sums``,
``gemv_w8a8``, ``gemv_w8a8_range``, ``gemv_vnni_supported`` -- the reference's CPU-only INT8 decode ops
(src/ops/cpu/GemvVnni.cpp:33-107). The native path (``csrc/host/gemv_int8.cpp``) uses AVX-512-VNNI ``vpdpbusd`` with
the +128 activation bias taken out through the row sums, and a scalar loop elsewhere; ``TESSERACT_HOST=python``
or a missing host module selects the torch restatement below, which produces the same integers.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native


def _host():
    if os.environ.get("TESSERACT_HOST", "") == "python":
        return None
    h = _native.host()
    return h if h is not None and hasattr(h, "gemv_w8a8") else None


def _threads(threads: int) -> int:
    """0 lets the native code pick (up to 16 hardware threads) unless TESSERACT_GEMM_MAX_THREADS caps it."""
    cap = int(os.environ.get("TESSERACT_GEMM_MAX_THREADS", "0") or 0)
    if cap > 0:
        return min(threads, cap) if threads > 0 else cap
    return threads


def gemv_vnni_supported() -> bool:
    h = _host()
    return bool(h.gemv_vnni_supported()) if h is not None else False


def quantize_row_int8(x: torch.Tensor) -> Tuple[torch.Tensor, float]:
    """x [K] fp32 -> (int8 [K], scale): scale = absmax / 127 (0 for a zero vector), round to nearest even, clip +-127."""
    x = x.detach().reshape(-1).float().cpu()
    h = _host()
    if h is not None:
        q, scale = h.quantize_row_int8(x.numpy())
        return torch.from_numpy(np.asarray(q)), float(scale)
    amax = float(x.abs().max()) if x.numel() else 0.0
    if amax <= 0:
        return torch.zeros_like(x, dtype=torch.int8), 0.0
    scale = float(np.float32(amax) / np.float32(127.0))
    inv = np.float32(1.0) / np.float32(scale)
    q = torch.clamp(torch.round(x * float(inv)), -127, 127).to(torch.int8)
    return q, scale


def compute_row_sums(W: torch.Tensor) -> torch.Tensor:
    """W [N, K] int8 -> int32 [N] row sums (the correction term of the unsigned-bias trick)."""
    if W.dim() != 2 or W.dtype != torch.int8:
        raise ValueError("compute_row_sums: W must be an int8 [N, K] tensor")
    h = _host()
    if h is not None:
        return torch.from_numpy(np.asarray(h.compute_row_sums(W.contiguous().numpy())))
    return W.to(torch.int32).sum(dim=1, dtype=torch.int32)


def gemv_w8a8_range(W: torch.Tensor, wscale: torch.Tensor, rowsum: Optional[torch.Tensor], xq: torch.Tensor, xscale: float,
                    n_begin: int = 0, n_end: int = -1, threads: int = 0) -> torch.Tensor:
    """y [N] fp32 with rows [n_begin, n_end) filled: y[n] = xscale * wscale[n] * sum_k xq[k] * W[n, k]; other rows 0."""
    if W.dim() != 2 or W.dtype != torch.int8 or xq.dtype != torch.int8:
        raise ValueError("gemv_w8a8: W [N, K] and xq [K] must be int8")
    N, K = W.shape
    if wscale.numel() != N or xq.numel() != K:
        raise ValueError(f"gemv_w8a8: wscale must have {N} entries and xq {K}")
    n_end = N if n_end < 0 else n_end
    if not (0 <= n_begin <= n_end <= N):
        raise ValueError("gemv_w8a8: bad row range")
    h = _host()
    if h is not None:
        rs = None if rowsum is None else rowsum.to(torch.int32).contiguous().numpy()
        y = h.gemv_w8a8(W.contiguous().numpy(), wscale.float().contiguous().numpy(), rs, xq.contiguous().numpy(),
                        float(xscale), int(n_begin), int(n_end), _threads(int(threads)))
        return torch.from_numpy(np.asarray(y))
    y = torch.zeros(N, dtype=torch.float32)
    acc = (W[n_begin:n_end].to(torch.int32) * xq.to(torch.int32)[None, :]).sum(dim=1, dtype=torch.int32)
    y[n_begin:n_end] = (np.float32(xscale) * wscale[n_begin:n_end].float()) * acc.float()
    return y


def gemv_w8a8(W: torch.Tensor, wscale: torch.Tensor, rowsum: Optional[torch.Tensor], xq: torch.Tensor, xscale: float,
              threads: int = 0) -> torch.Tensor:
    return gemv_w8a8_range(W, wscale, rowsum, xq, xscale, 0, -1, threads)


__all__ = ["gemv_vnni_supported", "quantize_row_int8", "compute_row_sums", "gemv_w8a8", "gemv_w8a8_range"]
