#!/usr/bin/env python
"""One transformer block forward (and backward) on random input: prints the output shape, how many entries are
finite and the L2 norm -- the sanity check of the reference's examples/llama_forward.cpp:86-175, same flags.

    python examples/llama_forward.py --d-model 64 --heads 4 --d-ff 128 --batch 2 --seq 16 --backward
    python examples/llama_forward.py --device cuda --d-model 1024 --heads 8 --d-ff 4096 --seq 256 --backward
"""
from __future__ import annotations

import argparse

from _common import pick_device, torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--d-model", type=int, default=64)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--d-ff", type=int, default=128)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=16)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.d_model % a.heads:
        raise SystemExit("error: --d-model must be a multiple of --heads")
    from tesseract_b200.nn import TransformerBlock
    dev = pick_device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    print(f"[llama_forward] config:\n  device={dev} dtype={dtype} d_model={a.d_model} heads={a.heads} d_ff={a.d_ff} "
          f"batch={a.batch} seq={a.seq}")
    torch.manual_seed(a.seed)
    block = TransformerBlock(a.d_model, a.heads, a.d_ff, max_seq_len=max(a.seq, 16), dtype=dtype, device=dev)
    x = torch.randn(a.batch, a.seq, a.d_model, device=dev, dtype=dtype, requires_grad=a.backward)
    out = block(x)
    host = out.detach().float().cpu()
    print(f"[llama_forward] out.shape = {list(out.shape)}")
    print(f"[llama_forward] finite  = {int(torch.isfinite(host).sum())} / {host.numel()}")
    print(f"[llama_forward] ||out||_2 = {float(host.double().norm()):.6f}")
    if a.backward:
        out.float().sum().backward()
        total = sum(float(p.grad.float().norm()) for p in block.parameters() if p.grad is not None)
        n = sum(1 for p in block.parameters() if p.grad is not None)
        print(f"[llama_forward] backward: sum(||grad||) = {total:.6f} over {n} parameters; "
              f"||dx|| = {float(x.grad.float().norm()):.6f}")
    print("[llama_forward] done.")
    return 0 if bool(torch.isfinite(host).all()) else 2


if __name__ == "__main__":
    raise SystemExit(main())
