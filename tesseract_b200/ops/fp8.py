"""Block-scaled FP8 (E4M3) GEMM path: quantisers, the tcgen05 GEMM and their torch restatement.

Scaling follows the 1 x 128 (activations: one scale per row and 128-wide K block) / 128 x 128 (weights) scheme:
``scale = absmax / 448`` (1 for an all-zero block), ``q = e4m3(x / scale)``, and the GEMM applies
``sa[m, kb] * sb[n // 128, kb]`` to every 128-deep partial product before adding it in fp32
(``csrc/gemm_fp8.cu``). Activation scales are stored K-block-major, ``[K / 128, M]``.
The reference's FP8 path is a per-tensor-scale cuBLASLt GEMM reachable only from a microbenchmark
(src/cuda/Fp8MatMul.cu:93-157, benchmarks/bench_cuda_fp8_gemm.cpp); this one is usable as a layer (``Fp8Linear``).
"""
from __future__ import annotations

import torch

from .. import _native
from .._native import check, lib, stream_ptr

P, I, L = _native.P, _native.I, _native.L
_native.register_signatures({
    "tsb_gemm_fp8_blockscaled": [P, P, P, P, P, I, I, I, L, P],
    "tsb_quant_act_1x128": [P, P, P, I, I, L, I, P],
    "tsb_quant_weight_128x128": [P, P, P, I, I, L, I, P],
    "tsb_gemm_fp8_pertensor": [P, P, P, P, P, I, I, I, L, P],
    "tsb_quant_tensor_e4m3": [P, P, P, L, I, P],
})

E4M3_MAX = 448.0


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and _native.available()


# ----------------------------------------------------------------------------------------- torch restatement
def quantize_act_ref(x: torch.Tensor):
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    amax = xb.abs().amax(dim=2)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xb / scale[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(M, K)
    return q.view(torch.uint8), scale.t().contiguous()


def quantize_weight_ref(w: torch.Tensor):
    N, K = w.shape
    nb = (N + 127) // 128
    wp = torch.zeros(nb * 128, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    blk = wp.view(nb, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blk / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(nb * 128, K)[:N]
    return q.contiguous().view(torch.uint8), scale.contiguous()


def dequantize_act(q: torch.Tensor, sa: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.view(torch.float8_e4m3fn).float().view(M, K // 128, 128) * sa.t()[:, :, None]).view(M, K)


def dequantize_weight(q: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    rows = torch.arange(N, device=q.device) // 128
    return (q.view(torch.float8_e4m3fn).float().view(N, K // 128, 128) * sb[rows][:, :, None]).view(N, K)


def fp8_gemm_ref(qa, sa, qb, sb) -> torch.Tensor:
    return (dequantize_act(qa, sa) @ dequantize_weight(qb, sb).t()).to(torch.bfloat16)


# ----------------------------------------------------------------------------------------- device ops
def quantize_act(x: torch.Tensor):
    """x [M, K] (K % 128 == 0) -> (e4m3 bytes uint8 [M, K], scales fp32 [K / 128, M])."""
    M, K = x.shape
    if K % 128:
        raise ValueError("quantize_act: K must be a multiple of 128")
    if not _native_ok(x) or x.stride(1) != 1:
        return quantize_act_ref(x)
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    sa = torch.empty((K // 128, M), dtype=torch.float32, device=x.device)
    check(lib().tsb_quant_act_1x128(x.data_ptr(), q.data_ptr(), sa.data_ptr(), M, K, x.stride(0),
                                    _native.dtype_code(x.dtype), stream_ptr(x.device)), "tsb_quant_act_1x128")
    return q, sa


def quantize_weight(w: torch.Tensor):
    """w [N, K] (K % 128 == 0) -> (e4m3 bytes uint8 [N, K], scales fp32 [ceil(N / 128), K / 128])."""
    N, K = w.shape
    if K % 128:
        raise ValueError("quantize_weight: K must be a multiple of 128")
    if not _native_ok(w) or w.stride(1) != 1:
        return quantize_weight_ref(w)
    q = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    sb = torch.empty(((N + 127) // 128, K // 128), dtype=torch.float32, device=w.device)
    check(lib().tsb_quant_weight_128x128(w.data_ptr(), q.data_ptr(), sb.data_ptr(), N, K, w.stride(0),
                                         _native.dtype_code(w.dtype), stream_ptr(w.device)), "tsb_quant_weight_128x128")
    return q, sb


def fp8_gemm(qa: torch.Tensor, sa: torch.Tensor, qb: torch.Tensor, sb: torch.Tensor,
             out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [M, N] = block-scaled qa [M, K] @ qb [N, K]^T on the tensor cores (fp32 accumulation); ``out`` (bf16,
    unit stride in the last dimension) receives the result when given."""
    M, K = qa.shape
    N = qb.shape[0]
    if not _native_ok(qa):
        r = fp8_gemm_ref(qa, sa, qb, sb)
        return r if out is None else out.copy_(r)
    if not (qa.is_contiguous() and qb.is_contiguous() and sa.is_contiguous() and sb.is_contiguous()):
        raise ValueError("fp8_gemm: operands must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=qa.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("fp8_gemm: out must be a bf16 [M, N] tensor with contiguous rows")
    check(lib().tsb_gemm_fp8_blockscaled(qa.data_ptr(), qb.data_ptr(), out.data_ptr(), sa.data_ptr(), sb.data_ptr(), M, N,
                                         K, out.stride(0), stream_ptr(qa.device)), "tsb_gemm_fp8_blockscaled")
    return out


class Fp8Linear(torch.nn.Module):
    """Inference Linear with E4M3 weights (128 x 128 scales); activations are quantised 1 x 128 per call."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor = None):
        super().__init__()
        q, sb = quantize_weight(weight.detach())
        self.register_buffer("q_weight", q)
        self.register_buffer("weight_scale", sb)
        self.bias = None if bias is None else torch.nn.Parameter(bias.detach().clone(), requires_grad=False)
        self.out_features, self.in_features = weight.shape

    @classmethod
    def from_linear(cls, lin) -> "Fp8Linear":
        return cls(lin.weight, getattr(lin, "bias", None))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        qa, sa = quantize_act(x2.contiguous())
        y = fp8_gemm(qa, sa, self.q_weight, self.weight_scale).to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.view(*x.shape[:-1], self.out_features)


# ----------------------------------------------------------------------------------------- per-tensor scaling
def quantize_tensor(x: torch.Tensor):
    """x -> (e4m3 bytes uint8 of the same shape, fp32 scale [1] on x's device): scale = absmax / 448 (1 for an all-zero
    tensor). The reference's FP8 contract (one device scale per operand, src/cuda/Fp8MatMul.cu:34-41,93-157)."""
    amax = x.detach().abs().amax().float().reshape(1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    xc = x.contiguous()
    if not _native_ok(xc):
        q = (xc.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
        return q, scale
    q = torch.empty(xc.shape, dtype=torch.uint8, device=xc.device)
    check(lib().tsb_quant_tensor_e4m3(xc.data_ptr(), q.data_ptr(), scale.data_ptr(), xc.numel(),
                                      _native.dtype_code(xc.dtype), stream_ptr(xc.device)), "tsb_quant_tensor_e4m3")
    return q, scale


def fp8_gemm_pertensor(qa: torch.Tensor, sa: torch.Tensor, qb: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """bf16 [M, N] = (sa * sb) * qa [M, K] @ qb [N, K]^T with one scale per operand; the whole K range accumulates
    in tensor memory (tcgen05 kind::f8f6f4, 128 x 256 tiles)."""
    M, K = qa.shape
    N = qb.shape[0]
    if not _native_ok(qa):
        a = qa.view(torch.float8_e4m3fn).float() * sa.float()
        b = qb.view(torch.float8_e4m3fn).float() * sb.float()
        return (a @ b.t()).to(torch.bfloat16)
    if K % 128 or not (qa.is_contiguous() and qb.is_contiguous()):
        raise ValueError("fp8_gemm_pertensor: K must be a multiple of 128 and the operands contiguous")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=qa.device)
    check(lib().tsb_gemm_fp8_pertensor(qa.data_ptr(), qb.data_ptr(), out.data_ptr(), sa.data_ptr(), sb.data_ptr(), M, N, K,
                                       out.stride(0), stream_ptr(qa.device)), "tsb_gemm_fp8_pertensor")
    return out
