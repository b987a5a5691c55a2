"""Structured metrics: JSON-lines records written by rank 0 (tokens/s, step ms, TTFT, ...), plus the
``[bench] key=value`` one-liners of the reference's bench binaries (benchmarks/bench_cuda_llama_serving.cpp:275-283)."""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Optional, TextIO


class MetricsLogger:
    def __init__(self, path: Optional[str] = None, rank: int = 0, stream: Optional[TextIO] = None):
        self.rank = rank
        self._f = open(path, "a", encoding="utf-8") if (path and rank == 0) else None
        self._stream = stream if stream is not None else (sys.stdout if rank == 0 else None)
        self.t0 = time.time()

    def log(self, **fields) -> None:
        if self.rank != 0:
            return
        rec = {"t": round(time.time() - self.t0, 6), **fields}
        line = json.dumps(rec, default=float)
        if self._f:
            self._f.write(line + "\n")
            self._f.flush()
        elif self._stream:
            self._stream.write(line + "\n")

    def bench_line(self, name: str, **fields) -> str:
        s = f"[bench] {name} " + " ".join(f"{k}={v}" for k, v in fields.items())
        if self.rank == 0 and self._stream:
            self._stream.write(s + "\n")
        return s

    def close(self) -> None:
        if self._f:
            self._f.close()
            self._f = None


def percentile(values, q: float) -> float:
    v = sorted(values)
    if not v:
        return 0.0
    i = min(len(v) - 1, max(0, int(round(q / 100.0 * (len(v) - 1)))))
    return float(v[i])
