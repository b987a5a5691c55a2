"""Registry of the ``TESSERACT_*`` environment variables (the reference scatters getenv calls:
src/ops/cpu/Attention.cpp:227-230, src/ops/cpu/GemmAvx2.cpp:38, src/core/Storage.cpp:105)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict


@dataclass(frozen=True)
class EnvVar:
    name: str
    default: str
    doc: str

    def get(self) -> str:
        return os.environ.get(self.name, self.default)


REGISTRY: Dict[str, EnvVar] = {v.name: v for v in [
    EnvVar("TESSERACT_GEMM", "tcgen05", "dense bf16 GEMM path: tcgen05 (native kernel) | cublas (library, for A/B runs)"),
    EnvVar("TESSERACT_ATTN", "tcgen05", "attention path: tcgen05 (native FlashAttention) | sdpa (library, for A/B runs)"),
    EnvVar("TESSERACT_TP_COMM", "fused", "tensor-parallel collectives: fused (GEMM + peer-memory kernel) | nccl"),
    EnvVar("TESSERACT_DEBUG", "", "non-empty: native code prints diagnostics (e.g. failed TMA descriptor encodings)"),
    EnvVar("TESSERACT_GEMM_MAX_THREADS", "0", "cap on CPU GEMV / GEMM worker threads of the host runtime (0 = all)"),
    EnvVar("TESSERACT_WATCHDOG_TIMEOUT_S", "60", "seconds without a heartbeat before a rank is declared lost"),
]}


def get(name: str) -> str:
    return REGISTRY[name].get()


def describe() -> str:
    return "\n".join(f"{v.name}={v.get()!r}  # {v.doc}" for v in REGISTRY.values())
