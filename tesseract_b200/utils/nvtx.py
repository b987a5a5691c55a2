"""NVTX ranges around layers / phases (no-ops without CUDA); ``profile_modules`` wraps every child's forward."""
from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def range_(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def profile_modules(model: torch.nn.Module, depth: int = 2) -> list:
    """Register forward pre/post hooks that open an NVTX range named after each sub-module (down to ``depth``).
    Returns the hook handles."""
    handles = []
    for name, mod in model.named_modules():
        if not name or name.count(".") >= depth:
            continue
        handles.append(mod.register_forward_pre_hook(lambda m, a, n=name: torch.cuda.nvtx.range_push(n)
                                                     if torch.cuda.is_available() else None))
        handles.append(mod.register_forward_hook(lambda m, a, o: torch.cuda.nvtx.range_pop()
                                                 if torch.cuda.is_available() else None))
    return handles
