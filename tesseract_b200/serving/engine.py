"""Device-resident continuous-batching engine (the serving fast path on a GPU).

Same scheduling contract as ``models.scheduler.ContinuousBatchingScheduler`` (FIFO admission against free KV
blocks, one token per running request per step, blocks recycled on retirement) but the whole decode step stays on
the device:

* one K and one V pool tensor for all layers ([L, num_blocks, Hkv, block, D], bf16 or INT8 + scales) and ONE block
  table [batch, max_blocks] shared by every layer, uploaded once per step (the reference rebuilds and uploads the
  tables in every layer of every step, src/nn/MultiHeadAttention.cpp:519-580);
* per layer: fused RMSNorm(+residual) -> one QKV GEMM -> fused RoPE + KV append (+INT8 quantisation) into the pool ->
  split-K paged decode attention -> o_proj -> ... -> SwiGLU FFN, every op a native sm_100a kernel;
* tokens are chosen on the device (argmax / nucleus sampling kernels); only ``batch`` int32 ids return to the host;
* the decode step is captured into CUDA graphs per batch-size bucket, so a step costs one graph launch;
* prompts admitted in the same step are prefilled together (projections and FFN batched over all their tokens,
  FlashAttention per prompt), instead of one un-batched prefill per request (src/models/Scheduler.cpp:115-124).

Tensor parallelism (``tp=TPServe(...)``, one process per GPU, every rank runs the same engine on the same requests):
attention heads and FFN columns are split over the ranks (q/k/v and gate/up column-parallel, o_proj and down_proj
row-parallel), each rank keeps the KV pool of its own KV heads, and the two partial sums per layer are combined
with the one-shot peer-memory all-reduce kernel on the decode path (inside the CUDA graph) and with NCCL on the
prefill path. Embedding, norms and lm_head are replicated, so every rank picks the same token without talking.
"""
from __future__ import annotations

import os
import time
from collections import deque

import numpy as np
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

import torch

from .. import _native, ops
from .._native import check, lib, stream_ptr
from ..models.llama import GenerateConfig, LlamaModel
from ..models.scheduler import EngineConfig
from ..nn.kv_cache import BlockAllocator

P, I, L, F = _native.P, _native.I, _native.L, _native.F
_native.register_signatures({
    "tsb_argmax_rows": [P, P, I, I, L, I, P],
    "tsb_argmax_rows_pack": [P, P, I, I, L, I, I, P],
    "tsb_argmax_rows_unpack": [P, P, I, I, I, P],
    "tsb_sample_top_p_rows": [P, P, I, I, L, F, F, _native.ctypes.c_ulonglong, _native.ctypes.c_ulonglong, I, P],
    "tsb_sample_rows": [P, P, I, I, L, F, I, F, _native.ctypes.c_ulonglong, _native.ctypes.c_ulonglong, P, I, P],
    "tsb_repetition_penalty_rows": [P, I, I, L, P, L, P, F, I, P],
})


class _Weight:
    """A projection weight as the engine holds it: bf16 [N, K] (``w``), or the E4M3 payload ``q`` [N, K] with its
    fp32 128 x 128 block scales ``s`` [ceil(N / 128), K / 128]."""
    __slots__ = ("w", "q", "s", "shape", "pow2", "atoms")

    def __init__(self, w=None, q=None, s=None, pow2=False, atoms=None):
        self.w, self.q, self.s = w, q, s
        self.atoms = atoms          # the block scales as 512-byte scale atoms (prompt-sized MX GEMM)
        self.pow2 = pow2            # every block scale is a power of two: the MX decode GEMM can take the weight
        self.shape = tuple((w if w is not None else q).shape)

    def nbytes(self) -> int:
        if self.w is not None:
            return self.w.numel() * self.w.element_size()
        return self.q.numel() + self.s.numel() * 4      # (the scale atoms of the prompt-sized GEMM are 1 / 32 more)


@dataclass
class _Req:
    id: int
    gen: GenerateConfig
    tokens: List[int]
    prompt_len: int
    generated: int = 0
    finished: bool = False
    blocks: List[int] = field(default_factory=list)
    slot: int = -1                 # row of the engine's host-side state arrays while the request holds KV blocks
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    check(lib().tsb_argmax_rows(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0),
                                _native.dtype_code(logits.dtype), stream_ptr(logits.device)), "tsb_argmax_rows")
    return out


def argmax_rows_pack(logits: torch.Tensor, packed: torch.Tensor, rank: int, world: int) -> None:
    """Vocabulary-parallel arg-max, step 1: ``packed`` [rows, 4 * world] bf16 receives this rank's best
    (value, index in three base-256 digits) per row in slot ``rank`` and zeros elsewhere; summed over the ranks it
    holds every rank's candidate exactly."""
    check(lib().tsb_argmax_rows_pack(logits.data_ptr(), packed.data_ptr(), logits.shape[0], logits.shape[1],
                                     logits.stride(0), rank, world, stream_ptr(logits.device)), "tsb_argmax_rows_pack")


def argmax_rows_unpack(summed: torch.Tensor, world: int, shard: int) -> torch.Tensor:
    """Step 2: global index of the best candidate of each summed row (rank r's shard starts at ``r * shard``)."""
    out = torch.empty(summed.shape[0], dtype=torch.int32, device=summed.device)
    check(lib().tsb_argmax_rows_unpack(summed.data_ptr(), out.data_ptr(), summed.shape[0], world, shard,
                                       stream_ptr(summed.device)), "tsb_argmax_rows_unpack")
    return out


def vocab_shard_rows(vocab: int, world: int) -> int:
    """Rows of the LM head per tensor-parallel rank (a multiple of 128, the last rank may hold fewer), or 0 when the
    vocabulary is too small for every rank to hold some."""
    shard = (vocab + world * 128 - 1) // (world * 128) * 128
    return shard if (world - 1) * shard < vocab else 0


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, step: int = 0,
                step_counter: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Temperature -> top-k (0 = off) -> top-p -> one draw per row, on the device. With ``step_counter`` (an int64
    device tensor of one element) the step is read from it when the kernel runs, so the launch can be captured in a
    CUDA graph; the caller advances the counter."""
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    check(lib().tsb_sample_rows(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0),
                                float(temperature), int(top_k), float(top_p), seed, step,
                                step_counter.data_ptr() if step_counter is not None else None,
                                _native.dtype_code(logits.dtype), stream_ptr(logits.device)), "tsb_sample_rows")
    return out


def repetition_penalty_rows_(logits: torch.Tensor, history: torch.Tensor, hist_len: torch.Tensor, penalty: float) -> None:
    """In place: every occurrence of a token in ``history[row, :hist_len[row]]`` (int32) divides its positive logit
    by ``penalty`` or multiplies its non-positive logit by it (src/models/Sampler.cpp:29-50)."""
    check(lib().tsb_repetition_penalty_rows(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0),
                                            history.data_ptr(), history.stride(0), hist_len.data_ptr(), float(penalty),
                                            _native.dtype_code(logits.dtype), stream_ptr(logits.device)),
          "tsb_repetition_penalty_rows")


def sample_top_p_rows(logits: torch.Tensor, temperature: float, top_p: float, seed: int, step: int) -> torch.Tensor:
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    check(lib().tsb_sample_top_p_rows(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1],
                                      logits.stride(0), float(temperature), float(top_p), seed, step,
                                      _native.dtype_code(logits.dtype), stream_ptr(logits.device)),
          "tsb_sample_top_p_rows")
    return out


class TPServe:
    """Tensor-parallel context of a serving engine: process group, this rank, and the peer-memory all-reduce."""

    def __init__(self, group, rank: int, world: int, device, hidden_size: int, max_batch: int = 512):
        from ..parallel.fused_tp import SymmAllReduce
        self.group, self.rank, self.world = group, rank, world
        self.max_rows = max_batch
        self.ar = SymmAllReduce(group, rank, world, device, max_batch * hidden_size)
        # a second, small instance for the arg-max candidates of a vocabulary-parallel LM head: it always uses its
        # first buffer; the all-reduces of the layers in between order two of its calls on every rank
        self.head_ar = SymmAllReduce(group, rank, world, device, max_batch * 4 * world)
        self.nccl_calls = 0

    def all_reduce_big(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        dist.all_reduce(x, group=self.group)
        self.nccl_calls += 1
        return x


class ServingEngine:
    BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)

    def __init__(self, model: LlamaModel, cfg: Optional[EngineConfig] = None, use_cuda_graph: bool = True,
                 temperature: float = 0.0, top_p: float = 1.0, seed: int = 0, tp: Optional[TPServe] = None,
                 max_prefill_tokens: int = 0, fp8_prefill: bool = False, weights: str = "bf16", top_k: int = 0,
                 repetition_penalty: float = 1.0):
        self.model, self.cfg = model, cfg or EngineConfig()
        self.tp = tp
        # weights="fp8": every layer projection and the LM head are held as E4M3 with 128 x 128 block scales (half the
        # bytes a decode step streams), the scales rounded up to powers of two. Decode-sized batches quantise the
        # activations to E4M3 with one power-of-two scale per row and 32 columns and multiply on
        # tcgen05.mma kind::mxf8f6f4.block_scale, which applies both scale sets itself (csrc/gemm_decode_mx.cu);
        # prompt-sized batches quantise the activations 1 x 128 and run the block-scaled fp8 GEMM.
        if weights not in ("bf16", "fp8"):
            raise ValueError("ServingEngine: weights must be 'bf16' or 'fp8'")
        self.weights = weights
        self.top_k, self.repetition_penalty = int(top_k), float(repetition_penalty)
        # fp8_prefill: the layer GEMMs of prefill-sized batches (more than 512 rows) run on E4M3 copies of the weights
        # with one scale per tensor and a per-call activation scale (about 2 x the bf16 GEMM rate); decode-sized
        # batches and the LM head stay bf16. Off by default: it changes the numerics of the prompt pass.
        self.fp8_prefill = bool(fp8_prefill)
        self._w8: Dict[int, tuple] = {}
        # prompt tokens admitted per step (0 = no limit): bounds the time to first token of the requests at the
        # head of the queue and the size of the prefill activations; at least one request is always admitted
        self.max_prefill_tokens = max_prefill_tokens
        import os
        self.varlen_prefill = os.environ.get("TESSERACT_PREFILL_VARLEN", "1") == "1"   # 0: one launch per prompt
        # programmatic dependent launch of the decode GEMMs: they start (and prefetch weights) under the tail of the
        # kernel before them
        self.pdl = os.environ.get("TESSERACT_PDL", "1") == "1"
        self.stream_rows = 256       # batches up to this many rows count as decode-sized
        self.decode_gemm = os.environ.get("TESSERACT_SERVE_DECODE_GEMM", "auto")   # auto | mx | stream | splitk | fp8gemm (A/B runs)
        c, mc = self.cfg, model.config
        self.device = model._device()
        if self.device.type != "cuda" or mc.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("ServingEngine needs a bf16 / fp16 model on a CUDA device "
                             "(use ContinuousBatchingScheduler for CPU or fp32 models)")
        self.H, self.Hkv, self.D = mc.num_attention_heads, mc.kv_heads(), mc.head_dim
        if tp is not None:
            if self.H % tp.world or self.Hkv % tp.world or mc.intermediate_size % tp.world:
                raise ValueError("ServingEngine: heads, KV heads and FFN width must divide over the TP ranks")
            self.H, self.Hkv = self.H // tp.world, self.Hkv // tp.world
        self.L = len(model.layers)
        self.temperature, self.top_p, self.seed = temperature, top_p, seed
        self.greedy = temperature <= 1e-6
        kv_dtype = torch.int8 if c.kv_int8 else mc.dtype
        shape = (self.L, c.num_blocks, self.Hkv, c.block_size, self.D)
        self.k_pool = torch.zeros(shape, dtype=kv_dtype, device=self.device)
        self.v_pool = torch.zeros(shape, dtype=kv_dtype, device=self.device)
        self.k_scale = self.v_scale = None
        if c.kv_int8:
            self.k_scale = torch.ones(shape[:-1], dtype=torch.float32, device=self.device)
            self.v_scale = torch.ones(shape[:-1], dtype=torch.float32, device=self.device)
        self.allocator = BlockAllocator(c.num_blocks)
        self.max_blocks = (c.max_seq_len + c.block_size - 1) // c.block_size
        self._fuse_weights()
        if self.fp8_prefill and self.weights == "bf16":
            from ..ops import fp8
            for ws in (self.wqkv, self.wo, self.wgu, self.wdown):
                for W in ws:
                    if W.w is not None and W.w.dtype == torch.bfloat16 and W.shape[1] % 128 == 0:
                        self._w8[id(W)] = fp8.quantize_tensor(W.w)
        self._step_dev = torch.zeros(1, dtype=torch.int64, device=self.device)   # sampling step counter (graph-safe)
        self.waiting: Deque[_Req] = deque()
        self.running: List[_Req] = []
        self.requests: Dict[int, _Req] = {}
        self._next_id = 0
        self.steps = 0
        self.use_cuda_graph = use_cuda_graph
        self._graphs: Dict[int, dict] = {}
        self._host_inputs: Dict[int, torch.Tensor] = {}
        # Host-side state of the resident requests as arrays indexed by a stable slot (block table, block count, last
        # token, length): a decode step packs its inputs with a few gathers instead of a Python loop over requests.
        cap = self.cfg.max_batch_size
        self._tab = np.zeros((cap, self.max_blocks), dtype=np.int32)
        self._nblk = np.zeros(cap, dtype=np.int32)
        self._last = np.zeros(cap, dtype=np.int32)
        self._len = np.zeros(cap, dtype=np.int32)
        self._free_slots = list(range(cap - 1, -1, -1))
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "prefill_s": 0.0, "decode_s": 0.0, "decode_gpu_s": 0.0,
                      "decode_steps": 0}
        self._step_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    # ------------------------------------------------------------------ weights
    def _fuse_weights(self) -> None:
        """q/k/v and gate/up become one concatenated tensor per layer (one GEMM each). Under tensor parallelism
        every tensor is this rank's shard (rows of q/k/v/gate/up, columns of o_proj/down_proj) and the full
        projection weights of the model are released."""
        self.wqkv, self.wgu, self.wo, self.wdown = [], [], [], []
        tp = self.tp
        fp8_mode = self.weights == "fp8"

        def pack(w: torch.Tensor) -> _Weight:
            if fp8_mode and w.dtype == torch.bfloat16 and w.shape[1] % 128 == 0:
                from ..ops import fp8
                # power-of-two block scales: decode-sized batches then run on the tensor core's own block scaling
                q, sc = fp8.quantize_weight(w.contiguous(), pow2=True)
                return _Weight(q=q, s=sc, pow2=True, atoms=fp8.weight_scale_atoms(sc))
            return _Weight(w=w)

        with torch.no_grad():
            for blk in self.model.layers:
                a, f = blk.attn, blk.ffn
                if tp is None:
                    w = torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], dim=0).contiguous()
                    n0, n1 = a.q_proj.weight.shape[0], a.k_proj.weight.shape[0]
                    a.q_proj.weight.data, a.k_proj.weight.data, a.v_proj.weight.data = w[:n0], w[n0:n0 + n1], w[n0 + n1:]
                    g = torch.cat([f.gate_proj.weight, f.up_proj.weight], dim=0).contiguous()
                    nf = f.gate_proj.weight.shape[0]
                    f.gate_proj.weight.data, f.up_proj.weight.data = g[:nf], g[nf:]
                    self.wqkv.append(pack(w))
                    self.wgu.append(pack(g))
                    self.wo.append(pack(a.o_proj.weight))
                    self.wdown.append(pack(f.down_proj.weight))
                    if fp8_mode:   # the bf16 originals are not needed any more
                        for lin in (a.q_proj, a.k_proj, a.v_proj, a.o_proj, f.gate_proj, f.up_proj, f.down_proj):
                            lin.weight.data = torch.empty(0, dtype=lin.weight.dtype, device=lin.weight.device)
                    continue
                r, D = tp.rank, self.D
                q0, k0 = r * self.H * D, r * self.Hkv * D
                self.wqkv.append(pack(torch.cat([a.q_proj.weight[q0:q0 + self.H * D], a.k_proj.weight[k0:k0 + self.Hkv * D],
                                                 a.v_proj.weight[k0:k0 + self.Hkv * D]], dim=0).contiguous()))
                self.wo.append(pack(a.o_proj.weight[:, q0:q0 + self.H * D].contiguous()))
                fl = f.gate_proj.weight.shape[0] // tp.world
                self.wgu.append(pack(torch.cat([f.gate_proj.weight[r * fl:(r + 1) * fl],
                                                f.up_proj.weight[r * fl:(r + 1) * fl]], dim=0).contiguous()))
                self.wdown.append(pack(f.down_proj.weight[:, r * fl:(r + 1) * fl].contiguous()))
                for lin in (a.q_proj, a.k_proj, a.v_proj, a.o_proj, f.gate_proj, f.up_proj, f.down_proj):
                    lin.weight.data = torch.empty(0, dtype=lin.weight.dtype, device=lin.weight.device)
            # Greedy tensor-parallel serving splits the LM head over the ranks by vocabulary rows: each rank streams
            # 1 / world of it, takes the arg-max of its logits and the ranks exchange (value, index) pairs through the
            # peer-memory all-reduce. Sampling and the repetition penalty need whole rows of logits: replicated head.
            V = self.model.lm_head.weight.shape[0]
            self.vocab_shard = 0
            if (tp is not None and tp.world % 2 == 0 and self.greedy and self.repetition_penalty == 1.0 and V < (1 << 24)
                    and self.model.lm_head.weight.dtype == torch.bfloat16
                    and os.environ.get("TESSERACT_SERVE_VOCAB_PARALLEL", "1") == "1"):
                self.vocab_shard = vocab_shard_rows(V, tp.world)
            if self.vocab_shard:
                v0 = tp.rank * self.vocab_shard
                self.w_head = pack(self.model.lm_head.weight[v0:min(V, v0 + self.vocab_shard)].contiguous())
            else:
                self.w_head = pack(self.model.lm_head.weight)
            tied = self.model.lm_head.weight.data_ptr() == self.model.embed_tokens.weight.data_ptr()
            if fp8_mode and self.w_head.q is not None and not tied:
                self.model.lm_head.weight.data = torch.empty(0, dtype=self.model.lm_head.weight.dtype,
                                                             device=self.model.lm_head.weight.device)

    def weight_bytes(self) -> int:
        """Bytes of projection and LM-head weights this rank streams per decode step."""
        return sum(W.nbytes() for ws in (self.wqkv, self.wo, self.wgu, self.wdown) for W in ws) + self.w_head.nbytes()

    def _mm_reduce(self, x: torch.Tensor, W: _Weight):
        """x @ W^T of a row-parallel projection. Returns the product summed over the tensor-parallel ranks, or --
        for batches that fit the peer-memory all-reduce -- ``None`` after leaving this rank's partial product in the
        all-reduce input buffer: the caller then finishes with ``_norm`` (sum + residual + RMSNorm in one kernel)."""
        tp = self.tp
        if tp is None:
            return self._mm(x, W)
        pre = isinstance(x, tuple)               # (q, sf) from a fused producer: always a bf16 decode-sized product
        T, N = (x[0] if pre else x).shape[0], W.shape[0]
        if T <= tp.max_rows and (pre or x.dtype == torch.bfloat16):
            self._mm(x, W, out=tp.ar.input_view(T, N))
            return None
        return tp.all_reduce_big(self._mm(x, W))

    def _norm(self, x, res, norm, rows: int):
        """(rmsnorm(x + res) * weight, x + res); ``x is None`` means the partial sums wait in the all-reduce buffer."""
        if x is None:
            return self.tp.ar.reduce_norm(rows, norm.weight.shape[0], res, norm.weight, norm.eps)
        if res is None:
            return ops.rms_norm(x, norm.weight, norm.eps), x
        return ops.rms_norm(x, norm.weight, norm.eps, residual=res)

    def _mx_ok(self, W: _Weight, rows: int, dtype) -> bool:
        """The decode-sized product with ``W`` runs on the MX kernel, so its producer may hand over (q, sf) directly."""
        return (W.q is not None and W.pow2 and self.decode_gemm in ("auto", "mx") and rows <= self.stream_rows
                and dtype == torch.bfloat16 and os.environ.get("TESSERACT_MX_FUSED_QUANT", "1") == "1")

    def _norm_for(self, x, res, norm, rows: int, W: _Weight):
        """``_norm`` for the input of the product with ``W``: on the MX decode path one kernel normalises and
        quantises (the bf16 result is never written); returns ((q, sf), residual) then."""
        if x is not None and self._mx_ok(W, rows, x.dtype) and x.is_contiguous() and W.shape[1] % 128 == 0:
            from ..ops import fp8
            q, sf, h = fp8.rms_norm_quant_mx(x, norm.weight, norm.eps, residual=res)
            return (q, sf), h
        return self._norm(x, res, norm, rows)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids, gen: Optional[GenerateConfig] = None) -> int:
        gen = gen or GenerateConfig()
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("add_request: empty prompt")
        V = self.model.config.vocab_size
        if any(t < 0 or t >= V for t in prompt):
            raise ValueError("add_request: prompt id outside [0, vocab_size)")
        if gen.max_new_tokens < 0 or len(prompt) + gen.max_new_tokens > self.cfg.max_seq_len:
            raise ValueError("add_request: prompt + max_new_tokens exceeds max_seq_len")
        r = _Req(self._next_id, gen, prompt, len(prompt), t_submit=time.perf_counter())
        self._next_id += 1
        self.waiting.append(r)
        self.requests[r.id] = r
        return r.id

    def has_pending(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def num_running(self) -> int:
        return len(self.running)

    def num_waiting(self) -> int:
        return len(self.waiting)

    def free_blocks(self) -> int:
        return self.allocator.num_free()

    def allocated_blocks(self) -> int:
        return self.allocator.num_used()

    def is_finished(self, rid: int) -> bool:
        return self.requests[rid].finished

    def result(self, rid: int) -> List[int]:
        r = self.requests[rid]
        if not r.finished:
            raise KeyError(f"request {rid} is not finished")
        return list(r.tokens)

    def _blocks_for(self, n: int) -> int:
        return (n + self.cfg.block_size - 1) // self.cfg.block_size

    def _grow(self, r: _Req, new_len: int) -> None:
        if r.slot < 0:
            r.slot = self._free_slots.pop()
            self._tab[r.slot] = 0
            self._nblk[r.slot] = 0
        while len(r.blocks) < self._blocks_for(new_len):
            b = self.allocator.allocate()
            self._tab[r.slot, len(r.blocks)] = b
            r.blocks.append(b)
        self._nblk[r.slot] = len(r.blocks)

    def _retire(self, r: _Req) -> None:
        for b in r.blocks:
            self.allocator.free(b)
        r.blocks = []
        if r.slot >= 0:
            self._free_slots.append(r.slot)
            r.slot = -1
        r.finished = True
        r.t_done = time.perf_counter()

    # ------------------------------------------------------------------ model pieces
    def _layer(self, li: int, x, res, positions, slots, tables, lens, prefill_bounds=None):
        blk = self.model.layers[li]
        H, Hkv, D = self.H, self.Hkv, self.D
        T = positions.shape[0]
        h, res = self._norm_for(x, res, blk.norm_1, T, self.wqkv[li])
        qkv = self._mm(h, self.wqkv[li])
        ks = self.k_scale[li] if self.k_scale is not None else None
        vs = self.v_scale[li] if self.v_scale is not None else None
        rope = self.model.rope
        dt = _native.dtype_code(qkv.dtype)
        if prefill_bounds is None:
            q = torch.empty((T, H, D), device=qkv.device, dtype=qkv.dtype)
            check(lib().tsb_kv_append_paged(qkv.data_ptr(), rope.cos.data_ptr(), rope.sin.data_ptr(), positions.data_ptr(),
                                            slots.data_ptr(), self.k_pool[li].data_ptr(), self.v_pool[li].data_ptr(),
                                            ks.data_ptr() if ks is not None else None,
                                            vs.data_ptr() if vs is not None else None, q.data_ptr(), T, H, Hkv, D,
                                            self.cfg.block_size, dt, 1, stream_ptr(qkv.device)), "tsb_kv_append_paged")
            if self._mx_ok(self.wo[li], T, q.dtype) and (H * D) % 128 == 0:
                from ..ops import paged
                # the split merge of the attention writes the quantised operand of the output projection
                o = paged.paged_decode_attention_mx(q, self.k_pool[li], self.v_pool[li], tables, lens, None, ks, vs,
                                                    max_len_hint=self.cfg.max_seq_len)
            else:
                o = ops.paged_decode_attention(q, self.k_pool[li], self.v_pool[li], tables, lens, None, ks, vs,
                                               max_len_hint=self.cfg.max_seq_len)
                o = o.view(T, H * D)
        else:
            qkv = ops.rope_qkv(qkv, rope.cos, rope.sin, num_heads=H, num_kv_heads=Hkv, head_dim=D, seq_len=1,
                               positions=positions)
            check(lib().tsb_kv_append_paged(qkv.data_ptr(), rope.cos.data_ptr(), rope.sin.data_ptr(), positions.data_ptr(),
                                            slots.data_ptr(), self.k_pool[li].data_ptr(), self.v_pool[li].data_ptr(),
                                            ks.data_ptr() if ks is not None else None,
                                            vs.data_ptr() if vs is not None else None, None, T, H, Hkv, D,
                                            self.cfg.block_size, dt, 0, stream_ptr(qkv.device)), "tsb_kv_append_paged")
            cu, max_len, spans = prefill_bounds
            q4 = qkv.view(T, H + 2 * Hkv, D)
            if self.varlen_prefill:
                # every prompt of the step in ONE variable-length attention launch
                o = ops.flash_attention_varlen_packed(q4, cu, max_len, H, Hkv).view(T, H * D)
            else:
                outs = [ops.flash_attention_packed(q4[a:b].unsqueeze(0), H, Hkv, causal=True).view(b - a, H * D)
                        for (a, b) in spans]
                o = torch.cat(outs, dim=0) if len(outs) > 1 else outs[0]
        a_out = self._mm_reduce(o, self.wo[li])
        h2, res = self._norm_for(a_out, res, blk.norm_2, T, self.wgu[li])
        gu = self._mm(h2, self.wgu[li])
        if self._mx_ok(self.wdown[li], T, gu.dtype) and gu.is_contiguous() and (gu.shape[1] // 2) % 128 == 0:
            from ..ops import fp8
            act = fp8.swiglu_quant_mx(gu)            # SwiGLU and the quantiser of the down projection in one kernel
        else:
            act = ops.swiglu(gu)
        f = self._mm_reduce(act, self.wdown[li])
        return f, res

    def _mm(self, x: torch.Tensor, W: _Weight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x @ W^T. Decode-sized batches: the weight-streaming GEMM (bf16 or block-scaled fp8 weights, bf16
        activations). Larger batches: the tcgen05 bf16 GEMM, or for fp8 weights the block-scaled fp8 GEMM with the
        activations quantised 1 x 128 (the per-tensor-scaled fp8 GEMM when ``fp8_prefill`` holds such a copy)."""
        if isinstance(x, tuple):          # (q, sf): the producer already quantised the activations (MX decode path)
            from ..ops import fp8
            return fp8.mx_linear(x[0], x[1], W.q, W.s, out=out, pdl=self.pdl)
        if x.dtype != torch.bfloat16:
            r = x @ W.w.t()
            return r if out is None else out.copy_(r)
        M = x.shape[0]
        if M <= self.stream_rows:
            # measured on B200 (layer shapes of the 8 B model, 16 .. 256 rows): bf16 weights go through the streaming
            # kernel (one CTA takes both 128-row blocks of a 129 .. 256-row batch)
            N, K = W.shape
            if W.q is None:
                if self.decode_gemm != "splitk":
                    return ops.stream_linear(x, W.w, out=out, pdl=self.pdl)
                return ops.decode_linear(x, W.w, out=out)
            # fp8 weights with power-of-two block scales: activations quantised to E4M3 with one power-of-two scale
            # per 32 columns, and both scale sets applied by the tensor core (measured on B200, layer shapes of the
            # 8 B model: 0.10 .. 0.14 ms per layer at 16 .. 256 rows against 0.15 .. 0.20 for bf16 weights)
            if W.pow2 and self.decode_gemm in ("auto", "mx") and x.stride(1) == 1 and x.stride(0) % 8 == 0:
                from ..ops import fp8
                qa, sf = fp8.quantize_act_mx(x)
                return fp8.mx_linear(qa, sf, W.q, W.s, out=out, pdl=self.pdl)
            # otherwise the streaming kernel (bf16 activations, weights widened on the fly) for the K-heavy
            # row-parallel products, the block-scaled fp8 GEMM with 1 x 128 activation scales elsewhere
            if self.decode_gemm == "stream" or (M <= 128 and K >= 2 * N):
                return ops.stream_linear(x, W.q, W.s, out=out, pdl=self.pdl)
        if W.q is not None:
            from ..ops import fp8
            if W.pow2 and self.decode_gemm in ("auto", "mx") and x.stride(1) == 1 and x.stride(0) % 8 == 0:
                # prompt-sized batches: the same operand formats on the persistent MX GEMM (the whole K range
                # accumulates in tensor memory; the fp32-scaled GEMM below has to scale every 128-deep block in registers)
                qa, sf = fp8.quantize_act_mx(x, atoms=True)
                return fp8.mx_linear(qa, sf, W.q, W.s, out=out, w_atoms=W.atoms)
            qa, sa = fp8.quantize_act(x.contiguous())
            return fp8.fp8_gemm(qa, sa, W.q, W.s, out=out)
        w8 = self._w8.get(id(W))
        if w8 is not None:
            from ..ops import fp8
            qa, sa = fp8.quantize_tensor(x)
            r = fp8.fp8_gemm_pertensor(qa, sa, w8[0], w8[1])
            return r if out is None else out.copy_(r)
        return ops.gemm_bf16(x, W.w, out=out)

    def _forward(self, tokens, positions, slots, tables, lens, prefill_bounds=None, last_rows=None):
        m = self.model
        if self.tp is not None:
            self.tp.ar.parity = 0     # every pass makes an even number of all-reduces: the two buffers strictly alternate
        x = ops.embedding(tokens, m.embed_tokens.weight)
        res = None
        for li in range(self.L):
            x, res = self._layer(li, x, res, positions, slots, tables, lens, prefill_bounds)
        h, _ = self._norm(x, res, m.norm, tokens.shape[0])
        if last_rows is not None:
            h = h.index_select(0, last_rows)
        return self._mm(h.contiguous(), self.w_head)

    def _pick(self, logits: torch.Tensor, reqs: Optional[List[_Req]] = None) -> torch.Tensor:
        """Next token per row, on the device. Greedy: arg-max. Otherwise the device sampler; its step comes from a
        device counter that is advanced right after, so the pair can sit in a captured graph."""
        if self.repetition_penalty != 1.0 and reqs is not None:
            n = len(reqs)
            width = max(len(r.tokens) for r in reqs)
            hist = torch.zeros((logits.shape[0], width), dtype=torch.int32)
            lens = torch.zeros(logits.shape[0], dtype=torch.int32)
            for i, r in enumerate(reqs):
                hist[i, :len(r.tokens)] = torch.tensor(r.tokens, dtype=torch.int32)
                lens[i] = len(r.tokens)
            repetition_penalty_rows_(logits, hist.to(logits.device), lens.to(logits.device), self.repetition_penalty)
        if self.greedy and self.vocab_shard:
            tp, T = self.tp, logits.shape[0]
            if T > tp.max_rows:
                raise ValueError("ServingEngine: more rows than the head exchange buffer holds")
            tp.head_ar.parity = 0
            argmax_rows_pack(logits, tp.head_ar.input_view(T, 4 * tp.world), tp.rank, tp.world)
            summed = tp.head_ar.reduce(T, 4 * tp.world)
            return argmax_rows_unpack(summed, tp.world, self.vocab_shard)
        if self.greedy:
            return argmax_rows(logits)
        out = sample_rows(logits, self.temperature, self.top_k, self.top_p, self.seed, step_counter=self._step_dev)
        self._step_dev.add_(1)
        return out

    # ------------------------------------------------------------------ scheduling
    def _admit(self) -> List[_Req]:
        admitted, reserved, ptoks = [], 0, 0
        while self.waiting and len(self.running) + len(admitted) < self.cfg.max_batch_size:
            head = self.waiting[0]
            if admitted and self.max_prefill_tokens > 0 and ptoks + head.prompt_len > self.max_prefill_tokens:
                break
            ptoks += head.prompt_len
            need = self._blocks_for(head.prompt_len + 1)
            if self.free_blocks() - reserved < need:
                if not self.running and not admitted:
                    raise RuntimeError("engine: the head request does not fit and nothing is running to reclaim from")
                break
            reserved += need
            admitted.append(self.waiting.popleft())
        return admitted

    @torch.no_grad()
    def _prefill(self, reqs: List[_Req]) -> None:
        t0 = time.perf_counter()
        bs = self.cfg.block_size
        toks, pos, slots, bounds, last = [], [], [], [], []
        off = 0
        for r in reqs:
            self._grow(r, r.prompt_len)
            toks += r.tokens
            pos += list(range(r.prompt_len))
            slots += [r.blocks[p // bs] * bs + p % bs for p in range(r.prompt_len)]
            bounds.append((off, off + r.prompt_len))
            off += r.prompt_len
            last.append(off - 1)
        dev = self.device
        cu = torch.tensor([0] + [b for _, b in bounds], dtype=torch.int32).to(dev, non_blocking=True)
        bounds = (cu, max(b - a for a, b in bounds), list(bounds))
        tokens = torch.tensor(toks, dtype=torch.int64).to(dev, non_blocking=True)
        meta = torch.tensor([pos, slots], dtype=torch.int32).to(dev, non_blocking=True)
        last_rows = torch.tensor(last, dtype=torch.int64).to(dev, non_blocking=True)
        logits = self._forward(tokens, meta[0], meta[1], None, None, prefill_bounds=bounds, last_rows=last_rows)
        nxt = self._pick(logits, reqs).cpu().tolist()
        now = time.perf_counter()
        for r, t in zip(reqs, nxt):
            r.t_first = now
            self._emit(r, int(t))
        self.stats["prefill_tokens"] += off
        self.stats["prefill_s"] += now - t0

    def _emit(self, r: _Req, tok: int) -> None:
        if r.gen.max_new_tokens == 0:
            self._retire(r)
            return
        r.tokens.append(tok)
        r.generated += 1
        if r.slot >= 0:
            self._last[r.slot] = tok
            self._len[r.slot] = len(r.tokens)
        if (r.gen.eos_token_id >= 0 and tok == r.gen.eos_token_id) or r.generated >= r.gen.max_new_tokens:
            self._retire(r)

    def _bucket(self, n: int) -> int:
        for b in self.BUCKETS:
            if b >= n:
                return b
        return n

    def _decode_inputs(self, reqs: List[_Req], A: int) -> torch.Tensor:
        """Packed int32 step inputs [A, 4 + max_blocks]: token, position, cache slot, length after the append,
        then the block table row. Padded rows have slot -1 and length 0."""
        bs = self.cfg.block_size
        n = len(reqs)
        buf = self._host_inputs.get(A)
        if buf is None:
            buf = torch.zeros((A, 4 + self.max_blocks), dtype=torch.int32).pin_memory()
            self._host_inputs[A] = buf
        arr = buf.numpy()
        if n:
            slots = np.fromiter((r.slot for r in reqs), dtype=np.int64, count=n)
            lens = self._len[slots]
            short = np.nonzero((lens + bs - 1) // bs > self._nblk[slots])[0]    # requests that cross into a new block
            for i in short:
                self._grow(reqs[i], int(lens[i]))
            pos = lens - 1
            arr[:n, 0] = self._last[slots]
            arr[:n, 1] = pos
            arr[:n, 4:] = self._tab[slots]
            arr[:n, 2] = self._tab[slots, pos // bs] * bs + pos % bs
            arr[:n, 3] = lens
        arr[n:, 0:2] = 0
        arr[n:, 2] = -1
        arr[n:, 3] = 0
        return buf

    @torch.no_grad()
    def warm_graphs(self, max_batch: int = 0) -> int:
        """Captures the decode graph of every batch bucket up to ``max_batch`` (default: the configured maximum) with
        all-padding inputs (slot -1, length 0: nothing is appended or attended), so that no request pays for a capture
        (about 0.1 s per bucket) in the middle of serving. Returns the number of graphs captured."""
        if not self.use_cuda_graph or self.repetition_penalty != 1.0:
            return 0
        top = self._bucket(max_batch or self.cfg.max_batch_size)
        made = 0
        for A in self.BUCKETS:
            if A > top:
                break
            if A in self._graphs:
                continue
            self._capture(A, self._decode_inputs([], A))
            made += 1
        return made

    def _run_packed(self, inp: torch.Tensor) -> torch.Tensor:
        tokens = inp[:, 0].long()
        positions, slots, lens = inp[:, 1].contiguous(), inp[:, 2].contiguous(), inp[:, 3].contiguous()
        tables = inp[:, 4:]
        return self._forward(tokens, positions, slots, tables, lens)

    @torch.no_grad()
    def _decode(self, reqs: List[_Req]) -> None:
        t0 = time.perf_counter()
        n = len(reqs)
        A = self._bucket(n) if self.use_cuda_graph else n
        host = self._decode_inputs(reqs, A)
        if self.use_cuda_graph and self.repetition_penalty == 1.0:
            g = self._graphs.get(A)
            if g is None:
                g = self._capture(A, host)
            ev = self._step_events
            g["inp"].copy_(host, non_blocking=True)
            ev[0].record()
            g["graph"].replay()
            ev[1].record()
            nxt = g["next"][:n].cpu().tolist()
            self.stats["decode_gpu_s"] += ev[0].elapsed_time(ev[1]) * 1e-3   # device time of the captured step
        else:
            logits = self._run_packed(host.to(self.device, non_blocking=True))
            nxt = self._pick(logits, reqs)[:n].cpu().tolist()
        for r, t in zip(reqs, nxt):
            self._emit(r, int(t))
        self.stats["decode_tokens"] += n
        self.stats["decode_steps"] += 1
        self.stats["decode_s"] += time.perf_counter() - t0

    def _capture(self, A: int, host: torch.Tensor) -> dict:
        dev = self.device
        g = {"inp": host.to(dev)}
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            for _ in range(2):                                # warm-up: lazy allocations, attribute settings
                logits = self._run_packed(g["inp"])
                g["next"] = self._pick(logits)
        torch.cuda.current_stream(dev).wait_stream(stream)
        torch.cuda.synchronize(dev)
        # the warm-up runs appended to the cache at the fed positions; the captured replay overwrites the same slots
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self._run_packed(g["inp"])
            g["next"] = self._pick(logits)
        g["graph"] = graph
        self._graphs[A] = g
        return g

    def instrument(self, metrics=None, watchdog=None, nvtx_ranges: Optional[bool] = None) -> "ServingEngine":
        """Attach a ``utils.metrics.MetricsLogger`` (``run`` writes one summary record; every ``log_every`` steps a
        progress record), a ``utils.watchdog.RankWatchdog`` (tensor-parallel serving: every step beats and checks the
        peers on the host before it launches a collective) and / or NVTX ranges around prefill and decode (default:
        the ``TESSERACT_NVTX`` environment variable)."""
        import os
        if metrics is not None:
            self.metrics_logger = metrics
        if watchdog is not None:
            self.watchdog = watchdog
        self.nvtx = bool(nvtx_ranges) if nvtx_ranges is not None else os.environ.get("TESSERACT_NVTX", "0") == "1"
        return self

    def _range(self, name: str):
        import contextlib
        if not getattr(self, "nvtx", False):
            return contextlib.nullcontext()
        from ..utils import nvtx
        return nvtx.range_(name)

    def step(self) -> bool:
        wd = getattr(self, "watchdog", None)
        if wd is not None:
            wd.step()
        admitted = self._admit()
        if admitted:
            with self._range(f"prefill[{len(admitted)}]"):
                self._prefill(admitted)
            self.running += [r for r in admitted if not r.finished]
        live = [r for r in self.running if not r.finished]
        if live:
            with self._range(f"decode[{len(live)}]"):
                self._decode(live)
        self.running = [r for r in self.running if not r.finished]
        self.steps += 1
        ml = getattr(self, "metrics_logger", None)
        if ml is not None and self.steps % self.log_every == 0:
            ml.log(event="serve_progress", step=self.steps, running=len(self.running), waiting=len(self.waiting),
                   decode_tokens=self.stats["decode_tokens"], prefill_tokens=self.stats["prefill_tokens"])
        return self.has_pending()

    log_every = 100

    def run(self) -> None:
        try:
            while self.has_pending():
                self.step()
        except Exception as e:
            wd = getattr(self, "watchdog", None)
            if wd is not None:
                wd.report_failure(f"{type(e).__name__}: {e}")
            raise
        ml = getattr(self, "metrics_logger", None)
        if ml is not None:
            ml.log(event="serve_summary", **self.metrics())

    # ------------------------------------------------------------------ metrics
    def metrics(self) -> dict:
        done = [r for r in self.requests.values() if r.finished and r.t_first > 0]
        ttft = sorted((r.t_first - r.t_submit) * 1e3 for r in done)
        s = self.stats
        return {
            "requests": len(done),
            "prefill_tok_s": s["prefill_tokens"] / s["prefill_s"] if s["prefill_s"] > 0 else 0.0,
            "decode_tok_s": s["decode_tokens"] / s["decode_s"] if s["decode_s"] > 0 else 0.0,
            "ttft_p50_ms": ttft[len(ttft) // 2] if ttft else 0.0,
            "steps": self.steps,
            # wall time of a decode step against the device time of its captured graph: the difference is host work
            "decode_ms_per_step": 1e3 * s["decode_s"] / max(1, s["decode_steps"]),
            "decode_gpu_ms_per_step": 1e3 * s["decode_gpu_s"] / max(1, s["decode_steps"]),
        }
