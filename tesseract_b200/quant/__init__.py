"""Weight-only quantisation: packers, schemes and the quantised Linear layers.

Numerical contract of the reference (include/tesseract/quant/Pack.hpp:40-103, src/quant/Pack.cpp,
include/tesseract/quant/Scheme.hpp:33-79, src/nn/QuantizedLinear.cpp:15-148):
  * INT8: one symmetric scale per output row = absmax / 127 (1.0 for an all-zero row), values in [-127, 127];
  * INT4: one scale per group of ``group_size`` (even, dividing in_features) input columns = absmax / 7,
    values in [-7, 7] as two's-complement nibbles, low nibble = even k, high nibble = odd k;
  * quantised layers expose ``q_weight`` / ``weight_scale`` as buffers and ``bias`` as a parameter.
Decode-shaped calls (few rows) on CUDA go to the GEMV kernels of ``csrc/quant_gemv.cu``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from .. import _native
from .._native import check, lib, stream_ptr
from ..nn.kv_cache import dequantize_kv_per_token, quantize_kv_per_token  # noqa: F401 (re-export)

P, I, L, F = _native.P, _native.I, _native.L, _native.F
_native.register_signatures({
    "tsb_gemv_w8": [P, P, P, P, P, I, I, I, I, P],
    "tsb_gemv_w4g": [P, P, P, P, P, I, I, I, I, I, P],
    "tsb_dequant_w8_bf16": [P, P, P, L, I, P],
    "tsb_dequant_w4g_bf16": [P, P, P, L, I, I, P],
})


def pack_int8_symmetric(w: torch.Tensor):
    """w [out, in] -> (int8 [out, in], fp32 scale [out])."""
    wf = w.detach().float().cpu()
    absmax = wf.abs().amax(dim=1)
    scale = torch.where(absmax > 0, absmax / 127.0, torch.ones_like(absmax))
    q = torch.clamp(torch.round(wf / scale[:, None]), -127, 127).to(torch.int8)
    return q, scale


def pack_int4_group(w: torch.Tensor, group_size: int = 128):
    """w [out, in] -> (uint8 [out, in/2] packed nibbles, fp32 scale [out, in/group])."""
    out_f, in_f = w.shape
    if group_size <= 0 or group_size % 2 or in_f % group_size:
        raise ValueError("pack_int4_group: group_size must be even and divide in_features")
    wf = w.detach().float().cpu().view(out_f, in_f // group_size, group_size)
    absmax = wf.abs().amax(dim=2)
    scale = torch.where(absmax > 0, absmax / 7.0, torch.ones_like(absmax))
    q = torch.clamp(torch.round(wf / scale[:, :, None]), -7, 7).to(torch.int16).view(out_f, in_f)
    lo = (q[:, 0::2] & 0xF).to(torch.uint8)
    hi = (q[:, 1::2] & 0xF).to(torch.uint8)
    return (lo | (hi << 4)).contiguous(), scale


def unpack_int4_group(packed: torch.Tensor, scale: torch.Tensor, group_size: int) -> torch.Tensor:
    lo = (packed & 0xF).to(torch.int16)
    hi = (packed >> 4).to(torch.int16)
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    q = torch.stack((lo, hi), dim=-1).flatten(-2).float()
    out_f, in_f = q.shape
    return (q.view(out_f, in_f // group_size, group_size) * scale[:, :, None].float()).view(out_f, in_f)


@dataclass(frozen=True)
class Scheme:
    kind: str               # "int8" | "int4g"
    group_size: int = 0

    @staticmethod
    def Int8Symmetric() -> "Scheme":
        return Scheme("int8")

    @staticmethod
    def Int4GroupSymmetric(group_size: int = 128) -> "Scheme":
        return Scheme("int4g", group_size)


def _small_m(x2: torch.Tensor) -> bool:
    return x2.is_cuda and x2.shape[0] <= 16 and x2.dtype in (torch.bfloat16, torch.float16, torch.float32)


def _large_m_native(x2: torch.Tensor, N: int, K: int) -> bool:
    """More rows than the GEMV kernels take, bf16 on the GPU, shapes the tcgen05 GEMM accepts (16-byte rows)."""
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[0] > 16 and N % 8 == 0 and K % 8 == 0
            and not (torch.is_grad_enabled() and x2.requires_grad) and _native.available())


def dequantize_matmul_int8(x: torch.Tensor, q_weight: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
    """x [..., in] @ dequant(q_weight [out, in])^T (src/ops/cpu/DequantMatMul.cpp)."""
    x2 = x.reshape(-1, x.shape[-1])
    N, K = q_weight.shape
    if q_weight.device != x.device or weight_scale.device != x.device:
        raise ValueError("dequantize_matmul_int8: activations, packed weights and scales must be on one device")
    if _small_m(x2) and K % 16 == 0 and hasattr(lib(), "tsb_gemv_w8"):
        xc = x2.contiguous()
        y = torch.empty((x2.shape[0], N), device=x.device, dtype=x.dtype)
        check(lib().tsb_gemv_w8(xc.data_ptr(), q_weight.data_ptr(), weight_scale.data_ptr(), None, y.data_ptr(),
                                x2.shape[0], N, K, _native.dtype_code(x.dtype), stream_ptr(x.device)), "tsb_gemv_w8")
        return y.view(*x.shape[:-1], N)
    if _large_m_native(x2, N, K) and K % 16 == 0 and hasattr(lib(), "tsb_dequant_w8_bf16"):
        # widen once to bf16 with the native kernel, multiply on the tcgen05 GEMM
        w = torch.empty((N, K), device=x.device, dtype=torch.bfloat16)
        check(lib().tsb_dequant_w8_bf16(q_weight.data_ptr(), weight_scale.data_ptr(), w.data_ptr(), N, K,
                                        stream_ptr(x.device)), "tsb_dequant_w8_bf16")
        from ..ops.gemm import gemm_bf16
        return gemm_bf16(x2.contiguous(), w).view(*x.shape[:-1], N)
    w = (q_weight.float() * weight_scale[:, None].float()).to(x.dtype)
    return torch.nn.functional.linear(x, w)


def dequantize_matmul_int4_group(x: torch.Tensor, q_weight: torch.Tensor, weight_scale: torch.Tensor,
                                 group_size: int) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    N, K2 = q_weight.shape
    K = K2 * 2
    if q_weight.device != x.device or weight_scale.device != x.device:
        raise ValueError("dequantize_matmul_int4_group: activations, packed weights and scales must be on one device")
    if _small_m(x2) and K % 32 == 0 and group_size % 32 == 0 and hasattr(lib(), "tsb_gemv_w4g"):
        xc = x2.contiguous()
        y = torch.empty((x2.shape[0], N), device=x.device, dtype=x.dtype)
        check(lib().tsb_gemv_w4g(xc.data_ptr(), q_weight.data_ptr(), weight_scale.data_ptr(), None, y.data_ptr(),
                                 x2.shape[0], N, K, group_size, _native.dtype_code(x.dtype), stream_ptr(x.device)),
              "tsb_gemv_w4g")
        return y.view(*x.shape[:-1], N)
    if (_large_m_native(x2, N, K) and K % 32 == 0 and group_size % 32 == 0 and K % group_size == 0
            and hasattr(lib(), "tsb_dequant_w4g_bf16")):
        w = torch.empty((N, K), device=x.device, dtype=torch.bfloat16)
        check(lib().tsb_dequant_w4g_bf16(q_weight.data_ptr(), weight_scale.data_ptr(), w.data_ptr(), N, K, group_size,
                                         stream_ptr(x.device)), "tsb_dequant_w4g_bf16")
        from ..ops.gemm import gemm_bf16
        return gemm_bf16(x2.contiguous(), w).view(*x.shape[:-1], N)
    w = unpack_int4_group(q_weight, weight_scale, group_size).to(x.dtype)
    return torch.nn.functional.linear(x, w)


class QuantizedLinear(nn.Module):
    """INT8 weight-only Linear (src/nn/QuantizedLinear.cpp:15-148)."""

    def __init__(self, q_weight: torch.Tensor, weight_scale: torch.Tensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.out_features, self.in_features = q_weight.shape
        self.register_buffer("q_weight", q_weight)
        self.register_buffer("weight_scale", weight_scale)
        self.bias = nn.Parameter(bias) if bias is not None else None

    @classmethod
    def from_linear(cls, lin) -> "QuantizedLinear":
        q, s = pack_int8_symmetric(lin.weight)
        dev = lin.weight.device
        bias = lin.bias.detach().clone() if lin.bias is not None else None
        return cls(q.to(dev), s.to(dev), bias)

    def forward(self, x):
        y = dequantize_matmul_int8(x, self.q_weight, self.weight_scale)
        return y + self.bias if self.bias is not None else y

    def weight_bytes(self) -> int:
        return self.q_weight.numel() + self.weight_scale.numel() * 4


class QuantizedLinearInt4G(nn.Module):
    """INT4 group-quantised weight-only Linear (src/nn/QuantizedLinearInt4G.cpp)."""

    def __init__(self, q_weight: torch.Tensor, weight_scale: torch.Tensor, group_size: int,
                 bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.out_features, self.in_features = q_weight.shape[0], q_weight.shape[1] * 2
        self.group_size = group_size
        self.register_buffer("q_weight", q_weight)
        self.register_buffer("weight_scale", weight_scale)
        self.bias = nn.Parameter(bias) if bias is not None else None

    @classmethod
    def from_linear(cls, lin, group_size: int = 128) -> "QuantizedLinearInt4G":
        q, s = pack_int4_group(lin.weight, group_size)
        dev = lin.weight.device
        bias = lin.bias.detach().clone() if lin.bias is not None else None
        return cls(q.to(dev), s.to(dev), group_size, bias)

    def forward(self, x):
        y = dequantize_matmul_int4_group(x, self.q_weight, self.weight_scale, self.group_size)
        return y + self.bias if self.bias is not None else y

    def weight_bytes(self) -> int:
        return self.q_weight.numel() + self.weight_scale.numel() * 4


def quantize_linear(lin, scheme: Scheme):
    """Factory used by ``quantize_``: returns the quantised twin of ``lin`` (idempotent on quantised layers)."""
    if isinstance(lin, (QuantizedLinear, QuantizedLinearInt4G)):
        return lin
    if scheme.kind == "int8":
        return QuantizedLinear.from_linear(lin)
    if scheme.kind == "int4g":
        return QuantizedLinearInt4G.from_linear(lin, scheme.group_size)
    raise ValueError(f"unknown quantisation scheme {scheme.kind!r}")


__all__ = ["pack_int8_symmetric", "pack_int4_group", "unpack_int4_group", "Scheme", "QuantizedLinear",
           "QuantizedLinearInt4G", "quantize_linear", "dequantize_matmul_int8", "dequantize_matmul_int4_group",
           "quantize_kv_per_token", "dequantize_kv_per_token"]
