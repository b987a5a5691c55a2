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
    "tsb_quant_act_mx": [P, L, P, P, I, I, P],
    "tsb_gemm_decode_mx": [P, P, P, P, P, I, I, I, L, L, I, I, I, P],
    "tsb_rmsnorm_quant_mx": [P, P, P, P, P, P, I, I, _native.F, P],
    "tsb_swiglu_quant_mx": [P, P, P, I, I, P],
    "tsb_gemm_decode_mx_plan": [I, I, I, P, P, P, P],
    "tsb_gemm_mx": [P, P, P, P, P, I, I, I, L, L, P],
    "tsb_quant_act_mx_layout": [P, L, P, P, I, I, I, P],
    "tsb_mx_weight_scale_atoms": [P, P, I, I, P],
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


def quantize_weight_ref(w: torch.Tensor, pow2: bool = False):
    N, K = w.shape
    nb = (N + 127) // 128
    wp = torch.zeros(nb * 128, K, dtype=torch.float32, device=w.device)
    wp[:N] = w.float()
    blk = wp.view(nb, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
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


def quantize_weight(w: torch.Tensor, pow2: bool = False):
    """w [N, K] (K % 128 == 0) -> (e4m3 bytes uint8 [N, K], scales fp32 [ceil(N / 128), K / 128]).
    ``pow2=True`` rounds every block scale up to a power of two (the block then uses at most one binade less of the
    E4M3 range; the relative precision of a floating-point payload does not depend on the scale). Such weights can be
    multiplied by ``mx_linear``, where the tensor core applies the scales itself."""
    N, K = w.shape
    if K % 128:
        raise ValueError("quantize_weight: K must be a multiple of 128")
    if pow2:
        return quantize_weight_ref(w, pow2=True)
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


class MxLinear(torch.nn.Module):
    """Inference Linear with E4M3 weights whose 128 x 128 block scales are powers of two; activations are quantised per
    call to E4M3 with one power-of-two scale per row and 32 columns, and the tensor core applies both scale sets
    (``mx_linear``: the weight-streaming kernel up to 256 rows, the persistent tiled kernel above). bf16 in, bf16 out."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor = None):
        super().__init__()
        q, sb = quantize_weight(weight.detach(), pow2=True)
        self.register_buffer("q_weight", q)
        self.register_buffer("weight_scale", sb)
        self.register_buffer("weight_scale_atoms", weight_scale_atoms(sb))
        self.bias = None if bias is None else torch.nn.Parameter(bias.detach().clone(), requires_grad=False)
        self.out_features, self.in_features = weight.shape

    @classmethod
    def from_linear(cls, lin) -> "MxLinear":
        return cls(lin.weight, getattr(lin, "bias", None))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        big = x2.shape[0] > 256
        q, sf = quantize_act_mx(x2, atoms=big)
        y = mx_linear(q, sf, self.q_weight, self.weight_scale, w_atoms=self.weight_scale_atoms if big else None).to(x.dtype)
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


# ----------------------------------------------------------------------------------------- MX path (decode-sized M)
def _mx_m_pad(M: int) -> int:
    return (M + 127) // 128 * 128


def scales_are_pow2(scale: torch.Tensor) -> bool:
    """True when every fp32 scale is a positive power of two (mantissa bits zero)."""
    bits = scale.contiguous().view(torch.int32)
    return bool(((bits & 0x7FFFFF) == 0).all() and (bits > 0).all())


def _words_to_atoms(sf: torch.Tensor) -> torch.Tensor:
    """[K / 128, m_pad] scale words -> 512-byte atoms [m_pad / 128, K / 128, 128]: word (r % 32) * 4 + (r % 128) / 32."""
    kb, m_pad = sf.shape
    a = sf.t().reshape(m_pad // 128, 4, 32, kb)                # [mb, r / 32, r % 32, kb]
    return a.permute(0, 3, 2, 1).reshape(m_pad // 128, kb, 128).contiguous()


def _atoms_to_words(atoms: torch.Tensor) -> torch.Tensor:
    mb, kb, _ = atoms.shape
    return atoms.view(mb, kb, 32, 4).permute(1, 0, 3, 2).reshape(kb, mb * 128).contiguous()


def weight_scale_atoms(w_scale: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two block scales [N / 128, K / 128] -> scale atoms int32 [N / 128, K / 128, 128] for ``mx_linear``
    above 256 rows (every word = the scale's exponent byte four times)."""
    rows, cols = w_scale.shape
    if _native_ok(w_scale):
        out = torch.empty((rows, cols, 128), dtype=torch.int32, device=w_scale.device)
        check(lib().tsb_mx_weight_scale_atoms(w_scale.contiguous().data_ptr(), out.data_ptr(), rows, cols,
                                              stream_ptr(w_scale.device)), "tsb_mx_weight_scale_atoms")
        return out
    e = ((w_scale.contiguous().view(torch.int32).to(torch.int64) >> 23) & 0xFF) * 0x01010101
    e = torch.where(e >= 2 ** 31, e - 2 ** 32, e).to(torch.int32)
    return e[:, :, None].expand(rows, cols, 128).contiguous()


def quantize_act_mx_ref(x: torch.Tensor, atoms: bool = False):
    if atoms:
        q, sf = quantize_act_mx_ref(x)
        return q, _words_to_atoms(sf)
    M, K = x.shape
    xb = x.float().view(M, K // 32, 32)
    amax = xb.abs().amax(dim=2)
    e = torch.ceil(torch.log2(torch.where(amax > 0, amax, torch.ones_like(amax)) / E4M3_MAX)) + 127
    e = torch.where(amax > 0, e, torch.full_like(e, 127)).clamp(1, 254)
    q = (xb * torch.exp2(127 - e)[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(M, K)
    eb = e.to(torch.int64).view(M, K // 128, 4)
    words = eb[:, :, 0] | (eb[:, :, 1] << 8) | (eb[:, :, 2] << 16) | (eb[:, :, 3] << 24)          # [M, K / 128]
    sf = torch.full((K // 128, _mx_m_pad(M)), 0x7F7F7F7F, dtype=torch.int64, device=x.device)
    sf[:, :M] = words.t()
    sf = torch.where(sf >= 2 ** 31, sf - 2 ** 32, sf).to(torch.int32)
    return q.view(torch.uint8), sf


def quantize_act_mx(x: torch.Tensor, out=None, atoms: bool = False):
    """x [M, K] bf16 (K % 128 == 0) -> (E4M3 bytes uint8 [M, K], scale words int32 [K / 128, ceil(M / 128) * 128]):
    one power-of-two scale per row and 32 columns, ``q = x * 2^(127 - e)`` with the smallest exponent byte ``e`` that
    keeps the block within +-448; byte j of word [k / 128, m] is the exponent of columns 128 (k / 128) + 32 j .. + 31.
    ``atoms=True`` lays the same words out as 512-byte atoms int32 [ceil(M / 128), K / 128, 128] (word
    (m % 32) * 4 + (m % 128) / 32): the form the persistent GEMM behind ``mx_linear`` copies into tensor memory.
    ``out`` = (q, sf) buffers of those shapes to write into."""
    M, K = x.shape
    if K % 128:
        raise ValueError("quantize_act_mx: K must be a multiple of 128")
    if not (_native_ok(x) and x.dtype == torch.bfloat16):
        q, sf = quantize_act_mx_ref(x, atoms)
        if out is not None:
            out[0].copy_(q)
            out[1].copy_(sf)
            return out
        return q, sf
    if x.stride(1) != 1:
        raise ValueError("quantize_act_mx: rows must be contiguous")
    if out is None:
        q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
        sf = torch.empty((_mx_m_pad(M) // 128, K // 128, 128) if atoms else (K // 128, _mx_m_pad(M)), dtype=torch.int32,
                         device=x.device)
    else:
        q, sf = out
    check(lib().tsb_quant_act_mx_layout(x.data_ptr(), x.stride(0), q.data_ptr(), sf.data_ptr(), M, K, int(atoms),
                                        stream_ptr(x.device)), "tsb_quant_act_mx_layout")
    return q, sf


def _mx_buffers(M: int, K: int, device):
    return (torch.empty((M, K), dtype=torch.uint8, device=device),
            torch.empty((K // 128, _mx_m_pad(M)), dtype=torch.int32, device=device))


def rms_norm_quant_mx(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """RMSNorm whose result exists only as the MX-quantised operand of the next GEMM (one kernel):
    returns ``(q, sf, h)`` with ``h = x + residual`` (``x`` itself without a residual) and ``(q, sf)`` =
    ``quantize_act_mx(rmsnorm(h) * weight)``. x [M, D] bf16, D % 128 == 0."""
    M, D = x.shape
    fused = _native_ok(x) and x.dtype == torch.bfloat16 and D % 128 == 0 and D <= 8192 and x.is_contiguous() \
        and (residual is None or residual.is_contiguous())
    if not fused:
        from . import fused as F_
        if residual is None:
            y, h = F_.rms_norm(x, weight, eps), x
        else:
            y, h = F_.rms_norm(x, weight, eps, residual=residual)
        q, sf = quantize_act_mx(y)
        return q, sf, h
    q, sf = _mx_buffers(M, D, x.device)
    h = torch.empty_like(x) if residual is not None else x
    check(lib().tsb_rmsnorm_quant_mx(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                     weight.data_ptr(), h.data_ptr() if residual is not None else None, q.data_ptr(),
                                     sf.data_ptr(), M, D, float(eps), stream_ptr(x.device)), "tsb_rmsnorm_quant_mx")
    return q, sf, h


def swiglu_quant_mx(gate_up: torch.Tensor):
    """``quantize_act_mx(swiglu(gate_up))`` in one kernel: gate_up [M, 2F] bf16 (gate first), F % 128 == 0."""
    M, F2 = gate_up.shape
    F = F2 // 2
    if not (_native_ok(gate_up) and gate_up.dtype == torch.bfloat16 and F % 128 == 0 and gate_up.is_contiguous()
            and M <= 65535):
        from . import fused as F_
        return quantize_act_mx(F_.swiglu(gate_up))
    q, sf = _mx_buffers(M, F, gate_up.device)
    check(lib().tsb_swiglu_quant_mx(gate_up.data_ptr(), q.data_ptr(), sf.data_ptr(), M, F, stream_ptr(gate_up.device)),
          "tsb_swiglu_quant_mx")
    return q, sf


def dequantize_act_mx(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    if sf.dim() == 3:
        sf = _atoms_to_words(sf)
    M, K = q.shape
    words = sf[:, :M].t().to(torch.int64) & 0xFFFFFFFF                                            # [M, K / 128]
    e = torch.stack([(words >> (8 * j)) & 0xFF for j in range(4)], dim=2).view(M, K // 32).float()
    return (q.view(torch.float8_e4m3fn).float().view(M, K // 32, 32) * torch.exp2(e - 127)[:, :, None]).view(M, K)


def mx_linear(q: torch.Tensor, sf: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, out=None, pdl: bool = False,
              bn: int = 0, split: int = 0, w_atoms: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [M, N] = dequant(q, sf) @ dequant(wq, w_scale)^T with the scales applied by the tensor core
    (tcgen05.mma kind::mxf8f6f4.block_scale). ``q, sf`` from ``quantize_act_mx``; ``wq, w_scale`` from
    ``quantize_weight(w, pow2=True)`` (the scales must be powers of two: only their exponent reaches the hardware).
    ``sf`` as scale words (2-D) selects the weight-streaming kernel ``csrc/gemm_decode_mx.cu`` (meant for up to 256
    rows); ``sf`` as scale atoms (3-D, ``quantize_act_mx(..., atoms=True)``) selects the persistent 128 x 192-tile
    kernel ``csrc/gemm_mx.cu`` (prompt-sized M), which also wants the weight scales as atoms (``w_atoms`` =
    ``weight_scale_atoms(w_scale)``; made on the fly when not given)."""
    M, K = q.shape
    N = wq.shape[0]
    if not _native_ok(q):
        r = (dequantize_act_mx(q, sf) @ dequantize_weight(wq, w_scale).t()).to(torch.bfloat16)
        return r if out is None else out.copy_(r)
    if not (q.is_contiguous() and wq.stride(1) == 1 and w_scale.is_contiguous() and sf.is_contiguous()):
        raise ValueError("mx_linear: operands must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=q.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("mx_linear: out must be a bf16 [M, N] tensor with contiguous rows")
    if sf.dim() == 3:
        if w_atoms is None:
            w_atoms = weight_scale_atoms(w_scale)
        check(lib().tsb_gemm_mx(q.data_ptr(), sf.data_ptr(), wq.data_ptr(), w_atoms.data_ptr(), out.data_ptr(), M, N, K,
                                wq.stride(0), out.stride(0), stream_ptr(q.device)), "tsb_gemm_mx")
        return out
    check(lib().tsb_gemm_decode_mx(q.data_ptr(), sf.data_ptr(), wq.data_ptr(), w_scale.data_ptr(), out.data_ptr(), M, N,
                                   K, wq.stride(0), out.stride(0), bn, split, int(pdl), stream_ptr(q.device)),
          "tsb_gemm_decode_mx")
    return out


def mx_linear_plan(M: int, N: int, K: int, bn: int = 0):
    """(tile width, K split, ring depth [negative: two row blocks per CTA], resident CTAs) on the current device."""
    import ctypes
    b, s_, st, res = ctypes.c_int(bn), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    check(lib().tsb_gemm_decode_mx_plan(M, N, K, ctypes.byref(b), ctypes.byref(s_), ctypes.byref(st), ctypes.byref(res)),
          "tsb_gemm_decode_mx_plan")
    return b.value, s_.value, st.value, res.value
