"""Training engine: parameter arena + fused Adam + micro-batched fwd/bwd, with data-parallel gradient
reduction and the pinned-host input path.

The public call is ``Trainer.train_step(batch)`` where ``batch`` is a pinned host int64 tensor
[global_batch_per_rank, seq_len + 1]; it copies the tokens to the device, runs every micro-batch
(forward, fused lm_head + cross-entropy, backward with weight gradients accumulated straight into the
gradient arena), reduces gradients across data-parallel ranks, applies one fused Adam launch and returns
the mean loss as a Python float (one 4-byte device-to-host read).

Reference counterpart: the hot loop of examples/llama_train.cpp:164-174 (zero_grad, forward, loss,
backward, per-parameter Adam launches, loss read-back).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .optim import Adam, ParamArena
from .utils import nvtx


@dataclass
class TrainConfig:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 0.0
    micro_batch: int = 1            # sequences per forward/backward pass
    grad_dtype: torch.dtype = torch.bfloat16
    master_weights: bool = False    # fp32 master copy of bf16 parameters
    ce_chunk_rows: int = 4096
    zero_stage: int = 0             # 1: Adam moments sharded over the data-parallel ranks (parallel/zero.py)


class Trainer:
    def __init__(self, model, cfg: TrainConfig, dp_group=None, grad_reducer=None, grad_alloc=None):
        self.model, self.cfg = model, cfg
        p0 = next(model.parameters())
        gd = cfg.grad_dtype if p0.dtype != torch.float32 else torch.float32
        self.arena = ParamArena.from_module(model, grad_dtype=gd, master_weights=cfg.master_weights,
                                            grad_alloc=grad_alloc)
        self.opt = Adam(self.arena, cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.max_grad_norm)
        self.dp_group = dp_group
        self.grad_reducer = grad_reducer
        self.device = p0.device
        self._dev_batch: Optional[torch.Tensor] = None
        self._loss_host = torch.zeros((), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else None
        self.steps_done = 0
        self.metrics = None             # utils.metrics.MetricsLogger: one record per train_step
        self.watchdog = None            # utils.watchdog.RankWatchdog: heartbeat + peer check before every step
        self.nvtx = False               # NVTX ranges around the phases of a step (visible in a timeline profiler)
        self._last_step_t = None

    def instrument(self, metrics=None, watchdog=None, nvtx_ranges: Optional[bool] = None) -> "Trainer":
        """Attach a metrics logger (rank 0 writes step, loss, step time and tokens/s per ``train_step``), a rank
        watchdog (``train_step`` beats and checks the peers before it launches anything: a lost peer raises
        ``RankLost`` on the host instead of a hang in the next collective; an exception in the step is reported to
        the peers) and / or NVTX ranges (default: the ``TESSERACT_NVTX`` environment variable)."""
        import os
        if metrics is not None:
            self.metrics = metrics
        if watchdog is not None:
            self.watchdog = watchdog
        self.nvtx = bool(nvtx_ranges) if nvtx_ranges is not None else os.environ.get("TESSERACT_NVTX", "0") == "1"
        return self

    def _range(self, name: str):
        import contextlib
        return nvtx.range_(name) if self.nvtx else contextlib.nullcontext()

    # -------------------------------------------------------------------------------------------
    def step_on_device(self, batch: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a device-resident batch [B, S + 1] (int64). Returns the mean loss as a
        0-d device tensor (no host synchronisation)."""
        cfg = self.cfg
        B = batch.shape[0]
        mb = min(cfg.micro_batch, B)
        if B % mb:
            raise ValueError(f"batch of {B} sequences is not a multiple of micro_batch={mb}")
        n_micro = B // mb
        self.arena.zero_grad()
        total = torch.zeros((), device=batch.device, dtype=torch.float32)
        if self.grad_reducer is not None:
            self.grad_reducer.begin_step()
        for i in range(n_micro):
            chunk = batch[i * mb:(i + 1) * mb]
            inputs, targets = chunk[:, :-1], chunk[:, 1:]
            if self.grad_reducer is not None:
                self.grad_reducer.set_last_microbatch(i == n_micro - 1)
            with self._range(f"forward[{i}]"):
                loss = self.model.loss(inputs.contiguous(), targets.contiguous(), chunk_rows=cfg.ce_chunk_rows,
                                       loss_scale=1.0 / n_micro)
            with self._range(f"backward[{i}]"):
                loss.backward()
            total += loss.detach()
        if hasattr(self.model, "sync_replicated_grads"):
            self.arena.fold_autograd_grads()
            red_stream = getattr(self.grad_reducer, "stream", None)
            if red_stream is not None:
                # hybrid mesh: bucket all-reduces of this step may still be running on the reducer's stream over the
                # very gradients that the tensor-parallel sum below updates in place
                torch.cuda.current_stream().wait_stream(red_stream)
            self.model.sync_replicated_grads()
        if self.grad_reducer is not None:
            self.grad_reducer.finish_step()
        elif self.dp_group is not None:
            import torch.distributed as dist
            self.arena.fold_autograd_grads()
            world = dist.get_world_size(self.dp_group)
            if world > 1:
                self.arena.grad.div_(world)
                dist.all_reduce(self.arena.grad, group=self.dp_group)
        with self._range("optimizer"):
            self.opt.step()
        self.steps_done += 1
        return total / n_micro

    def train_step(self, host_batch: torch.Tensor) -> float:
        """End-to-end step from a (pinned) host batch; returns the loss as a float."""
        if self.watchdog is None and self.metrics is None:
            return self._train_step(host_batch)
        import time
        if self.watchdog is not None:
            self.watchdog.step()                         # raises RankLost before anything is launched
        t0 = time.perf_counter()
        try:
            loss = self._train_step(host_batch)
        except Exception as e:
            if self.watchdog is not None:
                self.watchdog.report_failure(f"{type(e).__name__}: {e}")
            raise
        if self.metrics is not None:
            dt = time.perf_counter() - t0
            tokens = host_batch.shape[0] * (host_batch.shape[1] - 1)
            self.metrics.log(step=self.steps_done, loss=loss, step_ms=round(dt * 1e3, 3),
                             tokens_per_s_rank=round(tokens / dt, 1))
        return loss

    def _train_step(self, host_batch: torch.Tensor) -> float:
        if self.device.type == "cuda":
            if self._dev_batch is None or self._dev_batch.shape != host_batch.shape:
                self._dev_batch = torch.empty(host_batch.shape, dtype=host_batch.dtype, device=self.device)
            self._dev_batch.copy_(host_batch, non_blocking=True)
            loss = self.step_on_device(self._dev_batch)
            self._loss_host.copy_(loss, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            return float(self._loss_host)
        return float(self.step_on_device(host_batch))

    # -------------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.steps_done, "optimizer": self.opt.state_dict(),
                "rng_cpu": torch.get_rng_state(),
                "rng_cuda": torch.cuda.get_rng_state(self.device) if self.device.type == "cuda" else None}

    def load_state_dict(self, sd: dict) -> None:
        self.steps_done = int(sd["step"])
        self.opt.load_state_dict(sd["optimizer"])
        if sd.get("rng_cpu") is not None:
            torch.set_rng_state(sd["rng_cpu"])
        if sd.get("rng_cuda") is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(sd["rng_cuda"], self.device)
