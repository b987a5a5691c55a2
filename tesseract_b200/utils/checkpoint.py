"""Checkpoint save / resume.

The reference only loads safetensors (src/models/Llama.cpp:638-699). Here a checkpoint is a directory -- the
``.tsrct`` bundle the reference's roadmap names but never defines (README.md:28) -- holding
  ``manifest.json``      format version, model config, step, tensor-parallel layout
  ``model.safetensors``  dense weights under Hugging Face Llama key names (TP shards are gathered on save and
                         sliced on load, so a checkpoint is independent of the parallel layout it was written with)
  ``optim.rank{r}.pt``   optimizer moments, step counter and RNG state of rank r (sharded like the parameters)
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, is_dataclass
from typing import Optional

import torch

from ..io.safetensors import load_file, save_file

FORMAT_VERSION = 1


def _config_dict(cfg) -> dict:
    d = asdict(cfg) if is_dataclass(cfg) else dict(cfg.__dict__)
    return {k: (str(v).replace("torch.", "") if isinstance(v, torch.dtype) else v) for k, v in d.items()}


def save_checkpoint(path: str, model, trainer=None, rank: int = 0, world: int = 1, extra: Optional[dict] = None) -> None:
    """All ranks call this. Rank 0 writes the weights and the manifest; every rank writes its optimizer shard."""
    os.makedirs(path, exist_ok=True)
    if hasattr(model, "gather_dense_state_dict"):
        sd = model.gather_dense_state_dict()
        layout = {"tp": model.tp.size}
    else:
        sd = model.hf_state_dict()
        layout = {"tp": 1}
    if rank == 0:
        save_file({k: v.detach().cpu() for k, v in sd.items()}, os.path.join(path, "model.safetensors"), {"format": "pt"})
        manifest = {"format": "tsrct", "version": FORMAT_VERSION, "config": _config_dict(model.config),
                    "step": trainer.steps_done if trainer is not None else 0, "layout": layout, "world": world,
                    "extra": extra or {}}
        with open(os.path.join(path, "manifest.json"), "w", encoding="utf-8") as f:
            json.dump(manifest, f, indent=1)
    if trainer is not None:
        torch.save(trainer.state_dict(), os.path.join(path, f"optim.rank{rank}.pt"))


def load_checkpoint(path: str, model, trainer=None, rank: int = 0, strict_layout: bool = True) -> dict:
    """Restore weights (sliced for tensor-parallel models) and, when present and the layout matches, this rank's
    optimizer state. Returns the manifest."""
    with open(os.path.join(path, "manifest.json"), "r", encoding="utf-8") as f:
        manifest = json.load(f)
    if manifest.get("format") != "tsrct" or manifest.get("version", 0) > FORMAT_VERSION:
        raise ValueError(f"{path}: not a readable .tsrct bundle")
    sd = load_file(os.path.join(path, "model.safetensors"))
    if hasattr(model, "load_dense_state_dict"):
        model.load_dense_state_dict(sd)
        tp_now = model.tp.size
    else:
        model.load_hf_state_dict(sd)
        tp_now = 1
    opt_path = os.path.join(path, f"optim.rank{rank}.pt")
    if trainer is not None and os.path.exists(opt_path):
        if manifest["layout"].get("tp", 1) != tp_now:
            if strict_layout:
                raise ValueError("optimizer shards were written with a different tensor-parallel size")
        else:
            state = torch.load(opt_path, map_location=trainer.device, weights_only=False)
            trainer.load_state_dict(state)
    return manifest
