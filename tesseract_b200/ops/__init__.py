"""Functional ops. CUDA tensors are served by the native sm_100a kernels; CPU tensors by the torch
restatement of the reference's CPU math (which doubles as the test oracle)."""
from .attention import attention_ref, flash_attention, flash_attention_packed, flash_attention_varlen_packed
from .fused import (ce_loss_and_grad_, ce_stats, cross_entropy, cross_entropy_ref, embedding, grad_to_buf,
                    merge_ce_stats, rms_norm, rms_norm_ref, rope_qkv, rope_ref, rope_tables, swiglu, swiglu_ref,
                    swiglu_silu_gate)
from . import moe  # noqa: F401
from .gemm import decode_linear, gemm_bf16, linear, matmul_nt, stream_linear
from .paged import (decode_attention_gqa, paged_attention_ref, paged_decode_attention, paged_decode_attention_int8,
                    paged_decode_attention_mx,
                    paged_prefill_attention, paged_prefill_attention_int8, prefill_attention_gqa)

__all__ = [
    "attention_ref", "flash_attention", "flash_attention_packed", "flash_attention_varlen_packed", "ce_loss_and_grad_", "ce_stats", "cross_entropy", "cross_entropy_ref",
    "embedding", "grad_to_buf", "merge_ce_stats", "rms_norm", "rms_norm_ref", "rope_qkv", "rope_ref",
    "rope_tables", "swiglu", "swiglu_ref", "swiglu_silu_gate", "decode_linear", "stream_linear", "gemm_bf16", "linear", "matmul_nt", "decode_attention_gqa", "paged_attention_ref", "paged_decode_attention",
    "paged_decode_attention_int8", "paged_decode_attention_mx", "paged_prefill_attention", "paged_prefill_attention_int8", "prefill_attention_gqa",
]
