"""MoE expert compute on CUDA: device-side routing bookkeeping and grouped tcgen05 GEMMs.

``moe_ffn_grouped`` sorts the (token, expert) assignments by expert entirely on the device (every expert's row
block padded to a multiple of 128 rows), gathers the token rows once, runs gate_up and down as ONE grouped
tcgen05 GEMM launch each (the kernel reads the per-expert offsets from device memory, so nothing is copied back
to the host), and combines the weighted expert outputs with a gather-sum kernel. The backward pass uses the same
grouped kernel for the input gradients and its reduction-grouped mode for all experts' weight gradients. The
routing math itself (softmax, top-k, renormalisation) stays in ``nn.moe.route_topk`` so that every path shares it.
Replaces the reference's host-synchronised count -> permute -> cublasGemmGroupedBatchedEx pipeline
(src/cuda/MoeForward.cu:139-298).
"""
from __future__ import annotations

import torch

from .. import _native
from .._native import check, lib, stream_ptr
from .gemm import gemm_bf16, linear
from .fused import swiglu

P, I, L = _native.P, _native.I, _native.L
_native.register_signatures({
    "tsb_moe_route": [P, P, P, P, P, I, I, I, I, P],
    "tsb_moe_sort": [P, P, P, P, P, P, I, I, I, P],
    "tsb_moe_sort_padded": [P, P, P, P, P, P, I, I, I, I, I, P],
    "tsb_moe_gather_rows": [P, P, P, P, I, I, I, P],
    "tsb_moe_combine": [P, P, P, P, I, I, I, P],
    "tsb_moe_gate_grad": [P, P, P, P, I, I, I, P],
    "tsb_gemm_grouped": [P, P, P, P, I, I, I, I, I, I, L, L, L, I, L, L, I, I, P],
    "tsb_gemm_grouped_scatter": [P, P, P, I, I, I, I, L, L, I, L, P, _native.ctypes.POINTER(_native.ctypes.c_void_p), I, L,
                                 L, P],
    "tsb_ep_publish_counts": [_native.ctypes.POINTER(_native.ctypes.c_void_p), P, I, I, I, P],
    "tsb_ep_plan": [P, P, P, P, I, I, I, I, P],
    "tsb_ep_fill_i32": [P, L, I, P],
    "tsb_ep_dispatch": [P, P, P, _native.ctypes.POINTER(_native.ctypes.c_void_p), _native.ctypes.POINTER(_native.ctypes.c_void_p),
                        P, P, P, L, I, I, I, I, I, I, L, P],
    "tsb_ep_return": [P, P, _native.ctypes.POINTER(_native.ctypes.c_void_p), L, P, I, L, I, P],
    "tsb_ep_clean_copy": [P, P, P, L, P, I, P],
})


def route_native(logits: torch.Tensor, k: int, want_probs: bool = True):
    """Device router (no autograd): returns (probs [T, E] fp32 or None, idx int64 [T, k], gates fp32 [T, k],
    counts int32 [E])."""
    T, E = logits.shape
    lg = logits.contiguous()
    idx = torch.empty((T, k), dtype=torch.int32, device=lg.device)
    gates = torch.empty((T, k), dtype=torch.float32, device=lg.device)
    probs = torch.empty((T, E), dtype=torch.float32, device=lg.device) if want_probs else None
    counts = torch.zeros(E, dtype=torch.int32, device=lg.device)
    check(lib().tsb_moe_route(lg.data_ptr(), idx.data_ptr(), gates.data_ptr(),
                              probs.data_ptr() if probs is not None else None, counts.data_ptr(), T, E, k,
                              _native.dtype_code(lg.dtype), stream_ptr(lg.device)), "tsb_moe_route")
    return probs, idx.long(), gates, counts


def sort_by_expert(idx: torch.Tensor, counts: torch.Tensor):
    """Expert-sorted permutation of the T * k assignments, computed on the device.
    Returns (offsets int32 [E + 1], sorted_pos int32 [T * k], sorted_token int32 [T * k])."""
    T, k = idx.shape
    E = counts.shape[0]
    idx32 = idx.to(torch.int32).contiguous()
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    cursor = torch.empty(E, dtype=torch.int32, device=idx.device)
    pos = torch.empty(T * k, dtype=torch.int32, device=idx.device)
    tok = torch.empty(T * k, dtype=torch.int32, device=idx.device)
    check(lib().tsb_moe_sort(idx32.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(), pos.data_ptr(),
                             tok.data_ptr(), T, E, k, stream_ptr(idx.device)), "tsb_moe_sort")
    _native.add_launches(1)
    return offsets, pos, tok


def sort_by_expert_padded(idx32: torch.Tensor, counts: torch.Tensor, pad: int = 128):
    """Expert-sorted order in which every expert's row block starts at a multiple of ``pad`` rows.
    Returns (offsets int32 [E + 1], pos int32 [T * k], assign int32 [rows_cap] with -1 on padding rows, rows_cap)."""
    T, k = idx32.shape
    E = counts.shape[0]
    rows_cap = (T * k + E * (pad - 1) + pad - 1) // pad * pad
    dev = idx32.device
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    cursor = torch.empty(E, dtype=torch.int32, device=dev)
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    assign = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    check(lib().tsb_moe_sort_padded(idx32.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(),
                                    pos.data_ptr(), assign.data_ptr(), T, E, k, pad, rows_cap, stream_ptr(dev)),
          "tsb_moe_sort_padded")
    _native.add_launches(2)
    return offsets, pos, assign, rows_cap


def gather_rows(src: torch.Tensor, assign: torch.Tensor, k: int, row_scale: torch.Tensor = None) -> torch.Tensor:
    """dst[r] = (row_scale[assign[r]] if given else 1) * src[assign[r] // k], zeros where assign[r] < 0."""
    rows, D = assign.shape[0], src.shape[1]
    dst = torch.empty((rows, D), dtype=torch.bfloat16, device=src.device)
    check(lib().tsb_moe_gather_rows(src.data_ptr(), assign.data_ptr(),
                                    row_scale.data_ptr() if row_scale is not None else None, dst.data_ptr(), rows, D, k,
                                    stream_ptr(src.device)), "tsb_moe_gather_rows")
    return dst


def combine_rows(ys: torch.Tensor, pos: torch.Tensor, T: int, k: int, gates: torch.Tensor = None) -> torch.Tensor:
    """out[t] = sum_r (gates[t, r] if given else 1) * ys[pos[t * k + r]]."""
    D = ys.shape[1]
    out = torch.empty((T, D), dtype=torch.bfloat16, device=ys.device)
    check(lib().tsb_moe_combine(ys.data_ptr(), pos.data_ptr(), gates.data_ptr() if gates is not None else None,
                                out.data_ptr(), T, D, k, stream_ptr(ys.device)), "tsb_moe_combine")
    return out


def grouped_gemm_rows(a: torch.Tensor, w0: torch.Tensor, group_stride: int, offsets: torch.Tensor, groups: int,
                      b_mn: bool = False) -> torch.Tensor:
    """Row-grouped GEMM: out[r] = a[r] @ op(W[g(r)]). ``w0`` is group 0's weight ([N, K], or used as [K, N] when
    ``b_mn``); group g's weight starts ``g * group_stride`` elements later in the same allocation."""
    rows_cap, K = a.shape
    N = w0.shape[1] if b_mn else w0.shape[0]
    out = torch.empty((rows_cap, N), dtype=torch.bfloat16, device=a.device)
    check(lib().tsb_gemm_grouped(a.data_ptr(), w0.data_ptr(), out.data_ptr(), offsets.data_ptr(), groups, 1, rows_cap,
                                 0, N, K, a.stride(0), w0.stride(0), out.stride(0), int(b_mn), group_stride, 0, 0, 0,
                                 stream_ptr(a.device)), "tsb_gemm_grouped")
    return out


def grouped_gemm_rows_scatter(a: torch.Tensor, w0: torch.Tensor, group_stride: int, offsets: torch.Tensor, groups: int,
                              tags: torch.Tensor, peer_out, world: int, peer_rows: int, b_mn: bool = False) -> None:
    """``grouped_gemm_rows`` whose result rows leave through the GEMM epilogue for peer-mapped buffers: row r is
    stored at ``peer_out[tags[r] >> 24] + (tags[r] & 0xFFFFFF) * N`` when ``tags[r] >= 0`` (``peer_out``: a ctypes
    array of ``world`` device pointers, each [peer_rows, N] bf16); rows with a negative tag are dropped and nothing
    is written locally. The expert-parallel return exchange as the epilogue of the down projection."""
    rows_cap, K = a.shape
    N = w0.shape[1] if b_mn else w0.shape[0]
    check(lib().tsb_gemm_grouped_scatter(a.data_ptr(), w0.data_ptr(), offsets.data_ptr(), groups, rows_cap, N, K,
                                         a.stride(0), w0.stride(0), int(b_mn), group_stride, tags.data_ptr(), peer_out,
                                         world, peer_rows, N, stream_ptr(a.device)), "tsb_gemm_grouped_scatter")


def grouped_gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, offsets: torch.Tensor, groups: int, out: torch.Tensor,
                       group_stride: int, ldc: int, accumulate: bool) -> None:
    """Reduction-grouped GEMM: out[g] (+)= dy[rows of g]^T @ x[rows of g]; out[g] is [M, N] with row stride ldc and
    starts ``g * group_stride`` elements after out[0] (fp32 or bf16)."""
    rows_cap, M = dy.shape
    N = x.shape[1]
    check(lib().tsb_gemm_grouped(dy.data_ptr(), x.data_ptr(), out.data_ptr(), offsets.data_ptr(), groups, 2, rows_cap,
                                 M, N, 0, dy.stride(0), x.stride(0), ldc, 1, 0, group_stride,
                                 int(out.dtype == torch.float32), int(accumulate), stream_ptr(dy.device)),
          "tsb_gemm_grouped")


def _strided_stack(ws):
    """Element stride between consecutive tensors of ``ws`` if they sit at equal distances in one allocation, else 0."""
    if len(ws) == 1:
        return ws[0].numel()
    step = ws[1].data_ptr() - ws[0].data_ptr()
    if step <= 0 or step % ws[0].element_size():
        return 0
    for i, w in enumerate(ws):
        if w.data_ptr() - ws[0].data_ptr() != i * step or w.shape != ws[0].shape or not w.is_contiguous():
            return 0
    return step // ws[0].element_size()


def fuse_expert_storage_(moe) -> None:
    """Re-home the expert weights of ``moe`` in one flat buffer, expert after expert as [gate | up | down], so that
    gate and up form one [2 F, D] matrix per expert and the experts sit at a constant stride (what the grouped GEMM
    needs). Parameter objects and names are unchanged; only their storage moves."""
    ex = moe.experts
    w0 = ex[0].gate_proj.weight
    per = sum(getattr(e, n).weight.numel() for e in ex[:1] for n in ("gate_proj", "up_proj", "down_proj"))
    flat = torch.empty(per * len(ex), dtype=w0.dtype, device=w0.device)
    o = 0
    with torch.no_grad():
        for e in ex:
            for n in ("gate_proj", "up_proj", "down_proj"):
                p = getattr(e, n).weight
                view = flat[o:o + p.numel()].view_as(p)
                view.copy_(p)
                p.data = view
                o += p.numel()
    moe._expert_flat = flat


def grouped_path_ok(x2: torch.Tensor, moe) -> bool:
    if not (x2.is_cuda and x2.dtype == torch.bfloat16):
        return False
    from ..nn.modules import Linear
    if not all(isinstance(getattr(ex, n), Linear) for ex in moe.experts for n in ("gate_proj", "up_proj", "down_proj")):
        return False
    return moe.d_model % 64 == 0 and moe.d_ff % 64 == 0


def grouped_experts_backward(xs, h, a, dys, offsets, E, stride, w_gu0, w_dn0):
    """Backward of gate_up -> SwiGLU -> down over expert-grouped rows: returns (d xs [rows, D], dW fp32 flat
    [E * stride] in the layout of the weights: [gate | up | down] per expert). All experts per launch."""
    from .fused import swiglu_backward
    dev = dys.device
    D = xs.shape[1]
    F2 = h.shape[1]
    F = F2 // 2
    dw = torch.empty(E * stride, dtype=torch.float32, device=dev)
    grouped_gemm_wgrad(dys, a, offsets, E, dw[F2 * D:], stride, F, accumulate=False)    # d W_down [D, F]
    da = grouped_gemm_rows(dys, w_dn0, stride, offsets, E, b_mn=True)                     # [rows, F]
    dh = swiglu_backward(h, da)
    grouped_gemm_wgrad(dh, xs, offsets, E, dw, stride, D, accumulate=False)              # d W_gate_up [2F, D]
    dxs = grouped_gemm_rows(dh, w_gu0, stride, offsets, E, b_mn=True)                     # [rows, D]
    return dxs, dw


def split_expert_grads(dw, E, stride, F, D):
    """Views of a flat [E * stride] gradient as the per-expert (gate, up, down) weight gradients, in bf16."""
    dwe = dw.view(E, stride)
    grads = []
    for e in range(E):
        grads += [dwe[e, :F * D].view(F, D), dwe[e, F * D:2 * F * D].view(F, D), dwe[e, 2 * F * D:].view(D, F)]
    return [g.to(torch.bfloat16) for g in grads]


def expert_weight_stack(moe):
    """(weights list [gate, up, down per expert], per-expert stride, [2F, D] view of expert 0's gate|up, expert 0's
    down): re-homes the expert weights in one flat buffer first if they are not laid out that way yet."""
    E = moe.num_experts if len(moe.experts) == moe.num_experts else len(moe.experts)
    F, D = moe.d_ff, moe.d_model
    per = 3 * F * D

    def collect():
        out = []
        for ex in moe.experts:
            out += [ex.gate_proj.weight, ex.up_proj.weight, ex.down_proj.weight]
        return out

    ws = collect()

    def laid_out():
        # one storage (adjacent but separate allocations cannot be viewed as one matrix), constant expert stride
        base_storage = ws[0].untyped_storage().data_ptr()
        if any(w.untyped_storage().data_ptr() != base_storage for w in ws):
            return False
        if E > 1 and _strided_stack(ws[0::3]) != per:
            return False
        for e in range(E):
            base, es = ws[3 * e].data_ptr(), ws[3 * e].element_size()
            if ws[3 * e + 1].data_ptr() != base + F * D * es or ws[3 * e + 2].data_ptr() != base + 2 * F * D * es:
                return False
        return all(w.is_contiguous() for w in ws)

    if not laid_out():
        fuse_expert_storage_(moe)
        ws = collect()
    w_gu0 = torch.as_strided(ws[0].detach(), (2 * F, D), (D, 1))      # gate and up of expert 0 as one [2F, D] matrix
    return ws, per, w_gu0, ws[2].detach()


class _GroupedExpertsFn(torch.autograd.Function):
    """All experts of one MoE layer as grouped tcgen05 GEMMs over expert-sorted, 128-row-padded activations:
    gather -> gate_up (grouped) -> SwiGLU -> down (grouped) -> weighted combine. Nothing is read back to the host."""

    @staticmethod
    def forward(ctx, x2, gates, idx32, counts, stride, E, k, w_gu0, w_dn0, *weights):
        T, D = x2.shape
        offsets, pos, assign, rows_cap = sort_by_expert_padded(idx32, counts)
        xs = gather_rows(x2, assign, k)
        h = grouped_gemm_rows(xs, w_gu0, stride, offsets, E)
        a = swiglu(h)
        ys = grouped_gemm_rows(a, w_dn0, stride, offsets, E)
        gates32 = gates.float().contiguous()
        out = combine_rows(ys, pos, T, k, gates32)
        ctx.save_for_backward(xs, h, a, ys, gates32, offsets, pos, assign, w_gu0, w_dn0)
        ctx.meta = (T, D, E, k, stride, len(weights), gates.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        from .fused import swiglu_backward
        xs, h, a, ys, gates32, offsets, pos, assign, w_gu0, w_dn0 = ctx.saved_tensors
        T, D, E, k, stride, nw, gdtype = ctx.meta
        dout = dout.contiguous()
        dev = dout.device
        dgate = torch.empty(T * k, dtype=torch.float32, device=dev)
        check(lib().tsb_moe_gate_grad(dout.data_ptr(), ys.data_ptr(), pos.data_ptr(), dgate.data_ptr(), T, D, k,
                                      stream_ptr(dev)), "tsb_moe_gate_grad")
        dys = gather_rows(dout, assign, k, row_scale=gates32.view(-1))          # gate-weighted dOut per sorted row
        dxs, dw = grouped_experts_backward(xs, h, a, dys, offsets, E, stride, w_gu0, w_dn0)
        F2 = h.shape[1]
        F = F2 // 2
        dx = combine_rows(dxs, pos, T, k)
        dwe = dw.view(E, stride)
        grads = []
        for e in range(E):
            grads += [dwe[e, :F * D].view(F, D), dwe[e, F * D:F2 * D].view(F, D), dwe[e, F2 * D:].view(D, F)]
        grads = [g.to(torch.bfloat16) for g in grads] if nw else []
        return (dx, dgate.view(T, k).to(gdtype), None, None, None, None, None, None, None, *grads)


def moe_ffn_grouped(x2: torch.Tensor, idx: torch.Tensor, gates: torch.Tensor, moe, counts: torch.Tensor = None):
    """x2 [T, D] bf16, idx [T, k] expert ids, gates [T, k] -> [T, D] through the grouped tcgen05 GEMM path."""
    E, k = len(moe.experts), idx.shape[1]
    ws, per, w_gu0, w_dn0 = expert_weight_stack(moe)
    idx32 = idx.to(torch.int32).contiguous()
    if counts is None:
        counts = torch.bincount(idx32.view(-1), minlength=E).to(torch.int32)
    return _GroupedExpertsFn.apply(x2.contiguous(), gates, idx32, counts, per, E, k, w_gu0, w_dn0, *ws)
