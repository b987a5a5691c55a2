#!/usr/bin/env python
"""Train a Llama-shaped model on synthetic tokens (the reference's examples/llama_train.cpp:76-196, same flags,
plus model presets, bf16 and tensor/data parallelism).

    python examples/llama_train.py --steps 100 --lr 3e-3 --batch 2 --seq 16 --target-loss 0.5
    python examples/llama_train.py --device cuda --model small --batch 8 --seq 256 --steps 50
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        examples/llama_train.py --device cuda --model llama3-8b --batch 8 --seq 4096 --parallelism tp --steps 10

Like the reference it fits ONE fixed random batch (inputs = tokens[:-1], targets = tokens[1:]) and reports the
loss every few steps; with --target-loss it exits 1 when the final loss is above the gate.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

from _common import pick_device, preset, torch


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=16)
    ap.add_argument("--target-loss", type=float, default=0.0, help="<= 0 disables the convergence gate")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--dtype", default="", help="float32 | bfloat16 (default: bfloat16 on cuda, float32 on cpu)")
    ap.add_argument("--parallelism", default="auto", help="auto | tp | dp (with torchrun)")
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save", default="", help="write a resumable checkpoint bundle here at the end")
    a = ap.parse_args()

    dev = pick_device(a.device)
    dtype = {"": torch.bfloat16 if dev.type == "cuda" else torch.float32, "float32": torch.float32,
             "bfloat16": torch.bfloat16}[a.dtype]
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    if world > 1:
        import torch.distributed as dist
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo",
                                **({"device_id": dev} if dev.type == "cuda" else {}))
    from tesseract_b200.parallel import build_parallel_trainer
    from tesseract_b200.training import TrainConfig
    cfg = preset(a.model, dtype, a.seq + 1)
    tcfg = TrainConfig(lr=a.lr, micro_batch=a.micro_batch or min(a.batch, 4))
    # the tiny model on one process starts from the modules' own initialisers, like the reference's example
    trainer, plan = build_parallel_trainer(cfg, tcfg, world, rank, dev, a.parallelism, seed=a.seed,
                                           module_init=(a.model == "tiny" and world == 1))
    from tesseract_b200.parallel.launch import job_metrics, job_watchdog
    # TESSERACT_METRICS_FILE: one JSON record per step; TESSERACT_WATCHDOG_S: heartbeat + peer check before every step;
    # TESSERACT_NVTX=1: ranges around forward / backward / optimizer
    trainer.instrument(metrics=job_metrics(), watchdog=job_watchdog())
    if a.batch % plan["dp"]:
        raise SystemExit(f"error: --batch {a.batch} is not divisible by the data-parallel degree {plan['dp']}")
    g = torch.Generator().manual_seed(1234)
    batch = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=g)
    per = a.batch // plan["dp"]
    mine = batch[plan["dp_rank"] * per:(plan["dp_rank"] + 1) * per]
    mine = mine.pin_memory() if dev.type == "cuda" else mine
    if rank == 0:
        print(f"model={a.model} params={sum(p.numel() for p in trainer.model.parameters()):,} (this rank) "
              f"parallelism={plan['name']} device={dev} dtype={dtype}")
    loss, t0 = float("nan"), time.time()
    for step in range(1, a.steps + 1):
        loss = trainer.train_step(mine)
        if rank == 0 and (step == 1 or step % 10 == 0 or step == a.steps):
            print(f"step {step:5d}  loss {loss:.4f}  ({(time.time() - t0) / step * 1e3:.1f} ms/step)")
    if a.save and rank == 0:
        from tesseract_b200.utils.checkpoint import save_checkpoint
        save_checkpoint(a.save, trainer.model, trainer, extra={"step": a.steps})
        print(f"saved {a.save}")
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if a.target_loss > 0 and not loss <= a.target_loss:
        print(f"FAILED: final loss {loss:.4f} > target {a.target_loss}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
