"""State-space ops: selective scan (Mamba S6 recurrence) and depthwise causal conv1d.

Reference semantics (src/ops/cpu/SelectiveScan.cpp:92-127, src/cuda/CausalConv1d.cu:16-36):
  h_t = exp(delta_t * A) * h_{t-1} + delta_t * B_t * u_t ;  y_t = <h_t, C_t> + D * u_t
with u, delta [B, L, d], A [d, N], B, C [B, L, N], D [d], optional initial state [B, d, N]; returns
(y [B, L, d], final state [B, d, N]). conv: y[b, t, c] = bias[c] + sum_k w[c, k] * x[b, t - (K-1) + k, c].
CUDA fp32 / bf16 tensors run the chunked kernels of ``csrc/ssm.cu``; the loop below is the oracle.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from .._native import check, lib, stream_ptr

P, I, L, F = _native.P, _native.I, _native.L, _native.F
_native.register_signatures({
    "tsb_selective_scan": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "tsb_selective_scan_scratch_floats": [I, I, I, I],
    "tsb_causal_conv1d": [P, P, P, P, P, I, I, I, I, I, I, P],
})
_native._RESTYPES["tsb_selective_scan_scratch_floats"] = _native.L


def selective_scan_ref(u, delta, A, B, C, D, state=None):
    Bsz, L_, d = u.shape
    N = A.shape[1]
    h = torch.zeros(Bsz, d, N, dtype=torch.float32, device=u.device) if state is None else state.float().clone()
    uf, df, Af, Bf, Cf, Df = u.float(), delta.float(), A.float(), B.float(), C.float(), D.float()
    ys = []
    for t in range(L_):
        dA = torch.exp(df[:, t, :, None] * Af[None])                       # [B, d, N]
        dBu = df[:, t, :, None] * Bf[:, t, None, :] * uf[:, t, :, None]
        h = dA * h + dBu
        ys.append((h * Cf[:, t, None, :]).sum(-1) + Df * uf[:, t])
    y = torch.stack(ys, dim=1).to(u.dtype)
    return y, h.to(u.dtype)


def selective_scan(u, delta, A, B, C, D, state: Optional[torch.Tensor] = None):
    if (u.is_cuda and u.dtype in (torch.float32, torch.bfloat16) and A.shape[1] <= 64
            and hasattr(lib(), "tsb_selective_scan")):
        Bsz, L_, d = u.shape
        N = A.shape[1]
        uc, dc, Bc, Cc = u.contiguous(), delta.contiguous(), B.contiguous(), C.contiguous()
        Af, Df = A.float().contiguous(), D.float().contiguous()
        y = torch.empty_like(uc)
        st_in = state.float().contiguous() if state is not None else None
        st_out = torch.empty(Bsz, d, N, device=u.device, dtype=torch.float32)
        floats = lib().tsb_selective_scan_scratch_floats(Bsz, L_, d, N)
        scratch = torch.empty(max(int(floats), 1), device=u.device, dtype=torch.float32)
        check(lib().tsb_selective_scan(uc.data_ptr(), dc.data_ptr(), Af.data_ptr(), Bc.data_ptr(), Cc.data_ptr(),
                                       Df.data_ptr(), st_in.data_ptr() if st_in is not None else None, y.data_ptr(),
                                       st_out.data_ptr(), scratch.data_ptr(), Bsz, L_, d, N,
                                       _native.dtype_code(u.dtype), 0, stream_ptr(u.device)), "tsb_selective_scan")
        return y, st_out.to(u.dtype)
    return selective_scan_ref(u, delta, A, B, C, D, state)


def causal_conv1d_ref(x, weight, bias, silu: bool = False):
    Bsz, L_, C = x.shape
    K = weight.shape[1]
    xp = torch.nn.functional.pad(x.float(), (0, 0, K - 1, 0))
    out = bias.float()[None, None, :].expand(Bsz, L_, C).clone()
    for k in range(K):
        out = out + xp[:, k:k + L_] * weight.float()[:, k][None, None, :]
    if silu:
        out = torch.nn.functional.silu(out)
    return out.to(x.dtype)


def causal_conv1d(x, weight, bias, silu: bool = False):
    """x [B, L, C], weight [C, K], bias [C] -> [B, L, C] (optionally followed by SiLU in the same kernel)."""
    if (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and weight.shape[1] <= 8
            and hasattr(lib(), "tsb_causal_conv1d")):
        xc = x.contiguous()
        out = torch.empty_like(xc)
        wf, bf = weight.float().contiguous(), bias.float().contiguous()
        Bsz, L_, C = xc.shape
        check(lib().tsb_causal_conv1d(xc.data_ptr(), wf.data_ptr(), bf.data_ptr(), None, out.data_ptr(), Bsz, L_, C,
                                      weight.shape[1], int(silu), _native.dtype_code(x.dtype), stream_ptr(x.device)),
              "tsb_causal_conv1d")
        return out
    return causal_conv1d_ref(x, weight, bias, silu)
