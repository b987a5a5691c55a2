"""One-node launcher: one process per rank, rendezvous on 127.0.0.1, results or the failing rank's traceback back in
the parent (the role of the fork-based launcher inside the reference's benchmarks/bench_cuda_nccl_tp.cpp:229-318).

Rules it keeps from there: the parent never creates a CUDA context (the device count comes from a throwaway child),
workers are started with the ``spawn`` method, and exit codes are aggregated -- 77 from any rank means "skipped"
(no GPU / too few GPUs), anything else non-zero is a failure. A rank that dies takes the others down with it: the
parent terminates exactly the processes it started.

    results = launch(fn, world, *args)            # fn(rank, world, *args) runs inside an initialised process group
    python -m tesseract_b200.parallel.launch --nproc 2 script.py [script args]
"""
from __future__ import annotations

import datetime
import os
import runpy
import socket
import sys
import time
import traceback
from typing import Any, Callable, List, Optional

SKIP_EXIT_CODE = 77


class LaunchError(RuntimeError):
    def __init__(self, rank: int, detail: str):
        super().__init__(f"rank {rank} failed:\n{detail}")
        self.rank, self.detail = rank, detail


class LaunchSkipped(RuntimeError):
    """A rank reported that the job cannot run here (exit code 77)."""


class Skip(Exception):
    """Raise inside a worker to report 'skipped' (for instance: fewer GPUs than ranks)."""


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _count_devices(q) -> None:
    import torch
    q.put(torch.cuda.device_count() if torch.cuda.is_available() else 0)


def device_count() -> int:
    """CUDA device count, probed in a child process so that the caller stays free of a CUDA context."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    p = ctx.Process(target=_count_devices, args=(q,))
    p.start()
    p.join(120)
    if p.is_alive():
        p.terminate()
        return 0
    return int(q.get()) if p.exitcode == 0 and not q.empty() else 0


def _worker(fn, rank: int, world: int, port: int, backend: str, timeout_s: float, q, args, init_group: bool = True) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    code = 0
    try:
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(rank)
            kw["device_id"] = torch.device("cuda", rank)
        if init_group:
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)
        try:
            q.put((rank, "ok", fn(rank, world, *args)))
        except Skip:
            raise
        except BaseException as e:
            wd = job_watchdog(timeout_s=60.0)          # tell the peers on the host before this rank goes away
            if wd is not None:
                wd.report_failure(f"{type(e).__name__}: {e}")
            raise
        finally:
            if dist.is_initialized():
                dist.destroy_process_group()
    except Skip as s:
        q.put((rank, "skip", str(s)))
        code = SKIP_EXIT_CODE
    except BaseException:
        q.put((rank, "error", traceback.format_exc()))
        code = 1
    sys.exit(code)


def job_watchdog(timeout_s: Optional[float] = None):
    """A ``utils.watchdog.RankWatchdog`` over the key-value store of the default process group, or None when no group
    is initialised or the timeout (default: ``TESSERACT_WATCHDOG_S``) is not positive. Hand it to
    ``Trainer.instrument`` / ``ServingEngine.instrument``: every step then beats, and raises ``RankLost`` on the host
    when a peer stopped beating or posted an error, before the next collective is launched."""
    import torch.distributed as dist
    from ..utils.watchdog import RankWatchdog
    if timeout_s is None:
        timeout_s = float(os.environ.get("TESSERACT_WATCHDOG_S", "0") or 0)
    if timeout_s <= 0 or not dist.is_available() or not dist.is_initialized():
        return None
    try:
        store = dist.distributed_c10d._get_default_store()
    except Exception:
        return None
    return RankWatchdog(store, dist.get_rank(), dist.get_world_size(), timeout_s=timeout_s)


def job_metrics(path: Optional[str] = None):
    """A ``utils.metrics.MetricsLogger`` writing to ``path`` (default: ``TESSERACT_METRICS_FILE``) on rank 0, or None
    when neither names a file."""
    from ..utils.metrics import MetricsLogger
    path = path or os.environ.get("TESSERACT_METRICS_FILE", "")
    if not path:
        return None
    return MetricsLogger(path, rank=int(os.environ.get("RANK", "0")))


def launch(fn: Callable, world: int, *args: Any, backend: Optional[str] = None, timeout_s: float = 600.0,
           join_timeout_s: float = 3600.0, init_group: bool = True) -> List[Any]:
    """Runs ``fn(rank, world, *args)`` on ``world`` ranks and returns the results in rank order.

    ``backend``: "nccl" (one GPU per rank), "gloo" (CPU), or None = nccl when the node has at least ``world`` GPUs.
    ``timeout_s`` is the process-group timeout (how long a collective waits for a rank that never arrives).
    ``init_group=False`` only sets the rendezvous environment (RANK, WORLD_SIZE, MASTER_*) and leaves the process
    group to ``fn`` (the command-line form: scripts written for torchrun initialise it themselves).
    """
    import torch.multiprocessing as mp
    if world < 1:
        raise ValueError("launch: world must be >= 1")
    if backend is None:
        backend = "nccl" if device_count() >= world else "gloo"
    if backend not in ("nccl", "gloo"):
        raise ValueError(f"launch: unknown backend '{backend}'")
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(fn, r, world, port, backend, timeout_s, q, args, init_group)) for r in range(world)]
    for p in procs:
        p.start()
    results: dict = {}
    failure: Optional[LaunchError] = None
    skipped: Optional[str] = None
    deadline = time.monotonic() + join_timeout_s
    try:
        while len(results) < world and failure is None:
            while not q.empty():
                rank, kind, payload = q.get()
                results[rank] = payload
                if kind == "error" and failure is None:
                    failure = LaunchError(rank, payload)
                elif kind == "skip":
                    skipped = payload or "skipped"
            dead = [r for r, p in enumerate(procs) if p.exitcode not in (None, 0, SKIP_EXIT_CODE) and r not in results]
            if dead and q.empty() and failure is None:
                failure = LaunchError(dead[0], f"process exited with code {procs[dead[0]].exitcode} without a report")
            if time.monotonic() > deadline and failure is None:
                failure = LaunchError(-1, f"no result after {join_timeout_s} s")
            time.sleep(0.02)
    finally:
        for p in procs:                 # only the processes started here, by handle
            p.join(0.5 if failure is not None else 30)
            if p.is_alive():
                p.terminate()
                p.join(10)
    if failure is not None:
        raise failure
    if skipped is not None:
        raise LaunchSkipped(skipped)
    return [results[r] for r in range(world)]


def _run_script(rank: int, world: int, script: str, argv: List[str]):
    sys.argv = [script] + list(argv)
    try:
        runpy.run_path(script, run_name="__main__")
    except SystemExit as e:
        code = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
        if code == SKIP_EXIT_CODE:
            raise Skip(f"{script} exited with {SKIP_EXIT_CODE}") from None
        if code != 0:
            raise RuntimeError(f"{script} exited with code {code}") from None
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nproc", type=int, required=True)
    ap.add_argument("--backend", default=None, choices=["nccl", "gloo"])
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("script")
    ap.add_argument("script_args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    try:
        launch(_run_script, a.nproc, a.script, a.script_args, backend=a.backend, timeout_s=a.timeout, init_group=False)
    except LaunchSkipped as s:
        print(f"skipped: {s}", file=sys.stderr)
        return SKIP_EXIT_CODE
    except LaunchError as e:
        print(str(e), file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
