"""Dense GEMM entry points: the tcgen05 bf16 kernel for CUDA bf16 tensors, torch elsewhere.

``linear`` is the autograd-aware op every projection of the model goes through. Its backward issues
the two transposed GEMMs directly on the row-major operands (M/N-major UMMA descriptors), and can
accumulate the weight gradient straight into a caller-owned ``main_grad`` buffer.

Reference counterpart: ``ops::matmul`` -> cuBLASLt (src/ops/cpu/MatMul.cpp:424-435,
src/cuda/MatMul.cpp:422-490) and ``MatMulBackward`` (src/ops/cpu/MatMul.cpp:400-420).
"""
from __future__ import annotations

import os

import torch

from .. import _native


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and os.environ.get("TESSERACT_GEMM", "tcgen05") != "cublas"


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
              out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, accumulate: bool = False,
              block_n: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """C[M,N] (+)= op(A) @ op(B)^T on the tcgen05 kernel.

    ``a`` is [M,K] (``a_mn=False``) or [K,M] (``a_mn=True``); ``b`` is [N,K] or [K,N] (``b_mn=True``).
    Rows must be contiguous (stride 1 in the last dimension), row strides multiples of 8 elements.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1, "gemm_bf16 needs unit stride in the last dimension"
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm_bf16: inner dimensions differ ({K} vs {Kb})")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or torch.bfloat16)
        if accumulate:
            raise ValueError("accumulate=True needs an existing `out`")
    else:
        assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    rc = _native.lib().tsb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), block_n, max_ctas,
        _native.stream_ptr(a.device))
    _native.check(rc, "tsb_gemm_bf16")
    return out


_native.register_signatures({
    "tsb_gemm_cluster_splitk": [_native.P, _native.P, _native.P, _native.I, _native.I, _native.I, _native.L, _native.L,
                                _native.L, _native.I, _native.P],
    "tsb_gemm_bf16_splitk": [_native.P, _native.P, _native.P, _native.I, _native.I, _native.I, _native.L, _native.L,
                             _native.L, _native.I, _native.I, _native.I, _native.P],
})


def plan_decode_gemm(M: int, N: int, K: int, sm_count: int = 148, mode: str = "cluster"):
    """How a decode-shaped product x [M, K] @ w [N, K]^T is run: ``("cluster", S)`` -- S K-slices per output tile,
    reduced through the shared memory of a thread-block cluster; ``("plain", 0)`` -- the persistent GEMM;
    ``("atomic", S)`` -- S K-slices added into a zeroed fp32 buffer with atomics, then one cast."""
    mt = (M + 127) // 128
    kb = (K + 63) // 64
    tiles = mt * ((N + 127) // 128)
    if mode == "cluster" and 2 * tiles <= sm_count:
        # only for problems whose CTAs fit in ONE wave: every CTA of the non-persistent cluster kernel pays a fixed
        # start-up cost, and clusters of a second wave have to wait for a whole group of SMs to drain (measured
        # 2-4x slower than the persistent kernel there)
        sp = 1
        while sp < 8 and tiles * sp * 2 <= sm_count and kb // (sp * 2) >= 8:
            sp *= 2
        return "cluster", sp
    if tiles >= sm_count:
        return "plain", 0
    split = max(1, min(kb // 4, (2 * sm_count + tiles - 1) // tiles, 16))
    return ("atomic", split) if split > 1 else ("plain", 128)


def decode_linear(x: torch.Tensor, w: torch.Tensor, sm_count: int = 148, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] @ w [N, K]^T for decode-shaped calls (few rows against a weight matrix that is streamed once): when
    the plain tiling would leave most SMs idle the K range is split across CTAs -- a thread-block cluster per output
    tile that sums its slices through distributed shared memory (``csrc/gemm_cluster_splitk.cu``), or, with
    ``TESSERACT_DECODE_GEMM=simple``, fp32 atomics into a zeroed buffer and one cast. ``out`` (bf16 [M, N])
    receives the result when given."""
    M, K = x.shape
    N = w.shape[0]
    if not (_use_native(x) and M <= 512 and hasattr(_native.lib(), "tsb_gemm_bf16_splitk")):
        r = matmul_nt(x, w)
        return r if out is None else out.copy_(r)
    mode = os.environ.get("TESSERACT_DECODE_GEMM", "cluster")
    if not (hasattr(_native.lib(), "tsb_gemm_cluster_splitk") and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1):
        mode = "simple"
    kind, arg = plan_decode_gemm(M, N, K, sm_count, mode)
    if kind == "cluster":
        res = out if out is not None else torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
        rc = _native.lib().tsb_gemm_cluster_splitk(x.data_ptr(), w.data_ptr(), res.data_ptr(), M, N, K, x.stride(0),
                                                   w.stride(0), res.stride(0), arg, _native.stream_ptr(x.device))
        _native.check(rc, "tsb_gemm_cluster_splitk")
        return res
    if kind == "plain":
        return gemm_bf16(x, w, block_n=arg, out=out)
    out32 = torch.zeros((M, N), device=x.device, dtype=torch.float32)
    rc = _native.lib().tsb_gemm_bf16_splitk(x.data_ptr(), w.data_ptr(), out32.data_ptr(), M, N, K, x.stride(0),
                                            w.stride(0), N, 0, arg, 128, _native.stream_ptr(x.device))
    _native.check(rc, "tsb_gemm_bf16_splitk")
    return out32.to(torch.bfloat16) if out is None else out.copy_(out32)


_native.register_signatures({
    "tsb_gemm_decode_wq": [_native.P, _native.P, _native.P, _native.P, _native.I, _native.I, _native.I, _native.L,
                           _native.L, _native.L, _native.I, _native.I, _native.I, _native.I, _native.P],
})


_native.register_signatures({
    "tsb_gemm_decode_wq_plan": [_native.I, _native.I, _native.I, _native.I, _native.P, _native.P, _native.P, _native.P],
})


def stream_linear_plan(M: int, N: int, K: int, fp8: bool, bn: int = 0):
    """(tile width, K split) the streaming kernel chooses on the current device (``bn`` > 0 fixes the width)."""
    import ctypes
    b, s_, st, res = ctypes.c_int(bn), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    _native.check(_native.lib().tsb_gemm_decode_wq_plan(M, N, K, int(fp8), ctypes.byref(b), ctypes.byref(s_),
                                                        ctypes.byref(st), ctypes.byref(res)), "tsb_gemm_decode_wq_plan")
    return b.value, s_.value


def pack_fp8_weight(q: torch.Tensor, bn: int) -> torch.Tensor:
    """E4M3 payload [N, K] -> tile-major [ceil(N / bn), K / 64, bn, 64] (rows past N zero): the layout in which every
    tile the streaming kernel loads is one contiguous run of HBM. K must be a multiple of 64."""
    N, K = q.shape
    if K % 64 or bn % 16 or not 32 <= bn <= 256:
        raise ValueError("pack_fp8_weight: K % 64 == 0 and bn a multiple of 16 in [32, 256]")
    tiles = (N + bn - 1) // bn
    qp = q.view(torch.uint8)
    if tiles * bn != N:
        qp = torch.cat([qp, torch.zeros(tiles * bn - N, K, dtype=torch.uint8, device=q.device)], dim=0)
    return qp.view(tiles, bn, K // 64, 64).permute(0, 2, 1, 3).contiguous()


def unpack_fp8_weight(packed: torch.Tensor, N: int) -> torch.Tensor:
    """Inverse of ``pack_fp8_weight``: uint8 [N, K]."""
    tiles, nkb, bn, _ = packed.shape
    return packed.permute(0, 2, 1, 3).reshape(tiles * bn, nkb * 64)[:N]


def stream_linear(x: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor | None = None,
                  out: torch.Tensor | None = None, pdl: bool = False, bn: int = 0, split: int = 0,
                  packed_n: int = 0) -> torch.Tensor:
    """x [M, K] (bf16) @ W^T for decode-sized M with the weight-streaming kernel (``csrc/gemm_decode_wq.cu``).

    ``w`` is bf16 [N, K], or -- with ``w_scale`` (fp32 [ceil(N/128), ceil(K/128)]) -- the E4M3 payload (uint8 /
    float8_e4m3fn [N, K]) of a 128 x 128 block-scaled weight as ``ops.fp8.quantize_weight`` produces it, or that
    payload packed tile-major by ``pack_fp8_weight`` (then ``packed_n`` = N and ``bn`` = the packing width).
    Activations are not quantised. ``pdl=True`` launches with programmatic stream serialisation: the kernel may begin
    (and prefetch weights) while the previous kernel of the stream is still running. CPU tensors / other dtypes run
    the torch restatement."""
    M, K = x.shape
    packed = packed_n > 0
    if packed:
        if w_scale is None or w.dim() != 4 or w.shape[3] != 64 or w.shape[1] * 64 != K or w.shape[2] != bn:
            raise ValueError("stream_linear: packed weights are [tiles, K / 64, bn, 64] with their block scales")
        N = packed_n
    else:
        N = w.shape[0]
    fp8 = w_scale is not None
    if not (x.is_cuda and x.dtype == torch.bfloat16 and _native.available()):
        wf = w.float() if not fp8 else _dequant_block128(unpack_fp8_weight(w, N) if packed else w, w_scale)
        r = (x.float() @ wf.t()).to(x.dtype)
        return r if out is None else out.copy_(r)
    if x.stride(1) != 1 or (not packed and w.stride(1) != 1) or (packed and not w.is_contiguous()):
        raise ValueError("stream_linear: rows must be contiguous")
    res = out if out is not None else torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    rc = _native.lib().tsb_gemm_decode_wq(x.data_ptr(), w.data_ptr(), w_scale.data_ptr() if fp8 else None,
                                          res.data_ptr(), M, N, K, x.stride(0), 64 if packed else w.stride(0),
                                          res.stride(0), 2 if packed else int(fp8), bn, split,
                                          int(pdl) if isinstance(pdl, bool) else pdl, _native.stream_ptr(x.device))
    _native.check(rc, "tsb_gemm_decode_wq")
    return res


def _dequant_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 [N, K] from an E4M3 payload and its [ceil(N/128), ceil(K/128)] block scales."""
    N, K = q.shape
    w = q.view(torch.float8_e4m3fn).float()
    s = scale.float().repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)[:, :K]
    return w * s


def matmul_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M,K] @ b[N,K]^T without autograd."""
    if _use_native(a):
        return gemm_bf16(a, b)
    return a @ b.t()


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, wgrad_buf, force_wgrad):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        # allocate the result in its final shape: a view made inside a Function may not be modified in
        # place downstream (RoPE rotates the packed QKV projection in place)
        y = torch.empty(*x.shape[:-1], w.shape[0], device=x.device, dtype=torch.bfloat16)
        gemm_bf16(x2, w, out=y.view(-1, w.shape[0]))
        ctx.save_for_backward(x2, w)
        ctx.wgrad_buf = wgrad_buf
        ctx.force_wgrad = force_wgrad
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.x_shape, device=dy.device, dtype=torch.bfloat16)
            gemm_bf16(dy2, w, b_mn=True, out=dx.view(-1, w.shape[1]))     # dX = dY @ W
        if ctx.needs_input_grad[1] or ctx.force_wgrad:
            buf = ctx.wgrad_buf
            if buf is not None:
                gemm_bf16(dy2, x2, a_mn=True, b_mn=True, out=buf, accumulate=True)   # dW += dY^T @ X
            else:
                dw = gemm_bf16(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           wgrad_buf: torch.Tensor | None = None, force_wgrad: bool = False) -> torch.Tensor:
    """y = x @ weight^T (+ bias). ``weight`` is [out, in].

    With ``wgrad_buf`` (same shape as ``weight``, bf16 or fp32) the backward pass adds the weight
    gradient into that buffer and reports no gradient for ``weight`` to autograd. ``force_wgrad``
    computes it even when ``weight`` itself is not an autograd leaf (a fused view over several
    parameters that share one arena).
    """
    # the tcgen05 path needs 16-byte aligned rows in all three GEMMs (forward, dX, dW): out and in multiples of 8
    aligned = weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0 and weight.stride(0) % 8 == 0
    if _use_native(x) and weight.dtype == torch.bfloat16 and weight.stride(-1) == 1 and aligned:
        y = _LinearFn.apply(x, weight, wgrad_buf, bool(force_wgrad and wgrad_buf is not None))
        if bias is not None:
            y = y + bias
        return y
    if wgrad_buf is not None and torch.is_grad_enabled() and (weight.requires_grad or force_wgrad):
        return _AccumLinearFn.apply(x, weight, bias, wgrad_buf)
    return torch.nn.functional.linear(x, weight, bias)


class _AccumLinearFn(torch.autograd.Function):
    """Library-GEMM twin of _LinearFn (CPU tensors, fp32 CUDA tensors) with the same main_grad contract."""

    @staticmethod
    def forward(ctx, x, w, bias, wgrad_buf):
        ctx.save_for_backward(x, w)
        ctx.wgrad_buf = wgrad_buf
        ctx.has_bias = bias is not None
        return torch.nn.functional.linear(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = (dy2 @ w).view(x.shape) if ctx.needs_input_grad[0] else None
        ctx.wgrad_buf.add_((dy2.t() @ x2).to(ctx.wgrad_buf.dtype))
        db = dy2.sum(0) if ctx.has_bias else None
        return dx, None, db, None
