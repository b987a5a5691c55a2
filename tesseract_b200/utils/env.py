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
    EnvVar("TESSERACT_HOST", "native", "host runtime: native (C++ module) | python (the bit-identical Python twins)"),
    EnvVar("TESSERACT_DECODE_GEMM", "cluster", "decode-sized GEMMs: cluster (split-K reduced through DSMEM) | simple (fp32 atomics)"),
    EnvVar("TESSERACT_FLASH_FWD", "eager", "FlashAttention forward rescaling: eager | lazy (output kept in tensor memory; slower)"),
    EnvVar("TESSERACT_PREFILL_VARLEN", "1", "serving prefill attention: 1 (one variable-length launch) | 0 (one launch per prompt)"),
    EnvVar("TESSERACT_AG_KEEP", "copy", "all-gather -> GEMM: how the gathered activations are kept for backward: copy (copy engine) | kernel"),
    EnvVar("TESSERACT_AG_NSUB", "0", "all-gather -> GEMM: sub-chunks signalled per rank (0 = chosen by size; at most 2)"),
    EnvVar("TESSERACT_RMS_PREFETCH", "1", "RMSNorm forward: 1 (next row prefetched across the reduction) | 0 (plain kernel, for A/B runs)"),
    EnvVar("TESSERACT_GEMM_NO_AVX512", "0", "CPU fp32 GEMM: 1 = use the AVX2 6 x 16 tile even where AVX-512 (14 x 32) is available"),
    EnvVar("TESSERACT_SCAN_STREAM", "1", "selective scan of wide layers: 1 = single-pass kernel (state in registers, cp.async ring), 0 = three chunked passes"),
    EnvVar("TESSERACT_RMS_THREADS", "0", "RMSNorm forward threads per row: 0 (256) | 128 | 256, for A/B runs"),
    EnvVar("TESSERACT_REF_TIME_BUDGET", "780", "bench.py --impl reference: seconds the reference arm may take in total"),
    EnvVar("TESSERACT_REFERENCE_DIR", "/root/reference", "baseline/build_reference.py: source tree of the reference to build"),
    EnvVar("TESSERACT_DP_COMM", "symm", "data-parallel gradient all-reduce: symm (two-shot peer-memory kernel) | nccl"),
    EnvVar("TESSERACT_DP_CTAS", "0", "CTAs of the gradient all-reduce kernel (0 = 64)"),
    EnvVar("TESSERACT_PEAKS_FILE", "", "benchmarks: JSON file with the measured hbm_gbs / bf16_tflops of this GPU (roofline denominators)"),
    EnvVar("TESSERACT_TP_FUSED_MIN_AG", "8192", "tokens per step from which all-gather -> GEMM runs as the fused kernel"),
    EnvVar("TESSERACT_TP_FUSED_MIN_RS", "1024", "tokens per step from which GEMM -> reduce-scatter runs as the fused kernel"),
    EnvVar("TESSERACT_NVTX", "0", "1: Trainer and ServingEngine open NVTX ranges around the phases of a step"),
    EnvVar("TESSERACT_METRICS_FILE", "", "examples and the launcher: rank 0 appends one JSON record per step to this file"),
    EnvVar("TESSERACT_WATCHDOG_S", "0", "launcher and examples: > 0 attaches a rank watchdog with this heartbeat timeout in seconds"),
    EnvVar("TESSERACT_MX_FUSED_QUANT", "1", "serving, fp8 weights: 1 (RMSNorm / SwiGLU write the quantised GEMM operand directly) | 0 (separate quantiser kernel)"),
    EnvVar("TESSERACT_KERNEL_CASES_SMALL", "0", "benchmarks/kernel_cases.py: 1 runs one small shape per case (for a profiler capture)"),
    EnvVar("TESSERACT_EP_SCATTER_EPILOGUE", "1", "expert parallelism: 1 (the down projection's epilogue stores result rows into the source ranks' buffers) | 0 (separate return kernel)"),
    EnvVar("TESSERACT_PDL_ALL", "1", "decode-step kernels (quantisers, KV append, decode attention, merge): 1 (programmatic dependent launch) | 0"),
    EnvVar("TESSERACT_PDL", "1", "serving decode GEMMs: 1 (programmatic dependent launch) | 0"),
    EnvVar("TESSERACT_CPU_GEMM", "torch", "2-D fp32 CPU products of the frontend's ops.matmul: torch | native (the host runtime's GEMM, forward and backward)"),
    EnvVar("TESSERACT_DECODE_CTAS_PER_SM", "6", "paged decode attention: the key range is split until about this many CTAs per SM exist (never below 256 keys per split)"),
    EnvVar("TESSERACT_SERVE_VOCAB_PARALLEL", "1", "greedy tensor-parallel serving: 1 = the LM head is split over the ranks by vocabulary rows, 0 = replicated"),
    EnvVar("TESSERACT_SERVE_DECODE_GEMM", "auto", "serving decode GEMMs: auto | mx (fp8 weights: tensor-core block scaling) | stream (always the weight-streaming kernel) | splitk (bf16: the cluster split-K kernel) | fp8gemm (fp8 weights: never mx)"),
    EnvVar("TESSERACT_SWIGLU", "2", "SwiGLU kernels: 2 (row-wise, two vector pairs per thread) | 0 (flat kernel, for A/B runs)"),
]}


def get(name: str) -> str:
    return REGISTRY[name].get()


def describe() -> str:
    return "\n".join(f"{v.name}={v.get()!r}  # {v.doc}" for v in REGISTRY.values())
