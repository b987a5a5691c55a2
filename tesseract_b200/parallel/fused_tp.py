"""Fused tensor-parallel primitives over peer-mapped ("symmetric") device memory.

``SymmetricMemory`` allocates the same buffer on every rank of a group with ``cudaMalloc``, exchanges CUDA IPC
handles over the process group and maps every peer's buffer into this process (NVLink P2P through NVSwitch).
``FusedTP`` owns the buffers the two fused kernels of ``csrc/gemm_fused_comm.cu`` need and drives them:

* ``gemm_rs``  row-parallel GEMM whose epilogue pushes each tile to the owning rank's staging slot, then one
               cross-rank barrier kernel and a local sum of the ``world`` slots;
* ``ag_gemm``  one barrier kernel ("every rank is done with its landing buffer"), then ONE kernel in which copy
               CTAs push this rank's token shard into every peer's landing buffer, destination by destination,
               and bump the receiver's per-block counters, while the other CTAs run the GEMM over the local landing
               buffer behind those counters.

The staging buffer of ``gemm_rs`` is double-buffered by call parity: it is written again only two calls later, and
every call contains a barrier that a rank can pass only after all its earlier kernels on the stream (its reads of
the previous buffer generation included) have finished -- so no second barrier per call is needed. The landing
buffer of ``ag_gemm`` is single: the barrier comes first in the call, so when a peer starts to write, this rank has
finished everything it enqueued before (the GEMM and the weight-gradient GEMM that read the previous contents).
All device-side waits are bounded and report through the status word (``_native.read_status``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List

import torch

from .. import _native
from .._native import check, lib

P, I, L, F = _native.P, _native.I, _native.L, _native.F
PP = ctypes.POINTER(ctypes.c_void_p)
_native.register_signatures({
    "tsb_symm_alloc": [L, PP],
    "tsb_symm_free": [P],
    "tsb_ipc_export": [P, P],
    "tsb_ipc_open": [P, PP],
    "tsb_ipc_close": [P],
    "tsb_symm_barrier": [PP, I, I, I, P],
    "tsb_symm_barrier_limit": [PP, I, I, I, L, P],
    "tsb_reduce_slots": [P, P, I, L, P],
    "tsb_allreduce_oneshot": [PP, PP, P, P, L, I, I, P],
    "tsb_allreduce_twoshot": [PP, PP, P, L, I, I, I, I, F, I, I, L, P],
    "tsb_allreduce_norm_oneshot": [PP, PP, P, P, P, P, P, I, I, F, I, I, P],
    "tsb_gemm_rs": [P, P, PP, I, I, I, L, L, I, I, I, I, P],
    "tsb_gemm_ag": [P, PP, PP, P, P, P, I, I, I, I, I, I, L, L, I, I, I, I, P, P],
})


def _wrap_i32(v: int) -> int:
    """A monotonically growing counter as the int32 the kernels compare modulo 2^32."""
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v >= (1 << 31) else v


class _RawCuda:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__`` (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmetricMemory:
    """One equally-sized buffer per rank; ``ptrs[r]`` is rank r's buffer as mapped in THIS process."""

    def __init__(self, group, rank: int, world: int, nbytes: int, device):
        import torch.distributed as dist
        self.group, self.rank, self.world, self.nbytes = group, rank, world, nbytes
        local = ctypes.c_void_p()
        check(lib().tsb_symm_alloc(nbytes, ctypes.byref(local)), "tsb_symm_alloc")
        self.local_ptr = local.value
        handle = ctypes.create_string_buffer(64)
        check(lib().tsb_ipc_export(self.local_ptr, handle), "tsb_ipc_export")
        handles: List[bytes] = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local_ptr)
                continue
            out = ctypes.c_void_p()
            check(lib().tsb_ipc_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(out)), "tsb_ipc_open")
            self.ptrs.append(out.value)
            self._opened.append(out.value)
        self.ptr_array = (ctypes.c_void_p * world)(*self.ptrs)
        self.local = torch.as_tensor(_RawCuda(self.local_ptr, nbytes), device=device)   # uint8 view

    def offset_ptr_array(self, byte_offset: int):
        return (ctypes.c_void_p * self.world)(*[p + byte_offset for p in self.ptrs])

    def close(self) -> None:
        for p in self._opened:
            lib().tsb_ipc_close(p)
        self._opened = []
        if self.local_ptr:
            lib().tsb_symm_free(self.local_ptr)
            self.local_ptr = 0


class FusedTP:
    def __init__(self, group, rank: int, world: int, device, comm_ctas: int = 16):
        if world > 8:
            raise ValueError("FusedTP supports at most 8 ranks (one NVSwitch domain)")
        self.group, self.rank, self.world, self.device = group, rank, world, torch.device(device)
        self.comm_ctas = comm_ctas          # kept for callers that still pass it; the kernel no longer has copy CTAs
        self.pads = SymmetricMemory(group, rank, world, 256, device)
        self.epoch = 0
        self._land: SymmetricMemory = None     # [M, K] bf16 landing buffer of ag_gemm
        self._stage: SymmetricMemory = None    # 2 x [world, rows_per_rank, N] bf16
        self._land_half = self._stage_half = 0
        self._stage_calls = 0
        self._flag_ints = 1 << 16
        self._flagmem = SymmetricMemory(group, rank, world, 4 * self._flag_ints, device)   # zero-initialised
        self._flag_next = 0
        self._flags: Dict[tuple, list] = {}    # (rows per rank, K) -> [int offset, calls, nsub]
        self.keep_mode = os.environ.get("TESSERACT_AG_KEEP", "copy")   # "copy" (copy engine, side stream) | "kernel"
        self._keep_stream = None
        self._keep_event = None
        self.trace = None                   # int64 [SMs, 8] to receive per-CTA phase timestamps of ag_gemm (diagnostics)
        self.calls = {"gemm_rs": 0, "ag_gemm": 0, "barrier": 0}

    # ------------------------------------------------------------------ plumbing
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def barrier(self) -> None:
        self.epoch += 1
        check(lib().tsb_symm_barrier(self.pads.ptr_array, self.rank, self.world, _wrap_i32(self.epoch),
                                     self._stream()), "tsb_symm_barrier")
        self.calls["barrier"] += 1

    def _ensure(self, which: str, half_bytes: int) -> SymmetricMemory:
        cur = getattr(self, which)
        if cur is None or cur.nbytes < 2 * half_bytes:
            # (re)allocation is collective: every rank reaches this with the same sizes
            torch.cuda.synchronize(self.device)
            if cur is not None:
                import torch.distributed as dist
                dist.barrier(group=self.group)
                cur.close()
            cur = SymmetricMemory(self.group, self.rank, self.world, 2 * half_bytes, self.device)
            setattr(self, which, cur)
            setattr(self, which + "_half", half_bytes)
        return cur

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        """reduce_scatter_rows(x [M, K] @ op(w)^T) -> [M / world, N]."""
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if M % (128 * self.world) or N % 8 or x.stride(1) != 1 or w.stride(1) != 1:
            raise ValueError("gemm_rs: M must be a multiple of 128 * world and N of 8, rows contiguous")
        rpr = M // self.world
        stage = self._ensure("_stage", M * N * 2)
        parity = self._stage_calls & 1
        self._stage_calls += 1
        off = parity * self._stage_half
        check(lib().tsb_gemm_rs(x.data_ptr(), w.data_ptr(), stage.offset_ptr_array(off), M, N, K, x.stride(0),
                                w.stride(0), int(b_mn), rpr, self.rank, self.world, self._stream()), "tsb_gemm_rs")
        self.barrier()
        out = torch.empty((rpr, N), device=x.device, dtype=torch.bfloat16)
        check(lib().tsb_reduce_slots(stage.local_ptr + off, out.data_ptr(), self.world, rpr * N, self._stream()),
              "tsb_reduce_slots")
        self.calls["gemm_rs"] += 1
        return out

    # ------------------------------------------------------------------ all-gather -> GEMM
    def wait_keep(self) -> None:
        """Make the current stream wait for the last copy of gathered rows out of the landing buffer."""
        if self._keep_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self._keep_event)
            self._keep_event = None

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False, keep: bool = True,
                phase_mask: int = 3):
        """(all_gather_rows(x_local [M / world, K]) @ op(w)^T, gathered x [M, K]).

        With ``keep=False`` the gathered rows are returned as a view of the landing buffer: valid until the next
        ``ag_gemm`` call on this object (enough for a weight-gradient GEMM issued right after). With ``keep=True``
        they are copied out of the landing buffer by the copy engine on a side stream (``keep_mode="copy"``, the
        default: the copy overlaps the kernels that follow; consumers call ``wait_keep()``) or by the push warps
        of the kernel itself (``keep_mode="kernel"``).
        ``phase_mask`` is for measurements only: 1 runs the push half alone, 2 the multiply half alone over the data
        the last push delivered."""
        rpr, K = x_local.shape
        M = rpr * self.world
        N = w.shape[1] if b_mn else w.shape[0]
        if rpr % 128 or N % 8 or K % 8 or w.stride(1) != 1:
            raise ValueError("ag_gemm: rows per rank must be a multiple of 128, N and K of 8")
        x_local = x_local.contiguous()
        land = self._ensure("_land", (M * K * 2 + 1) // 2)
        ent = self._flags.get((rpr, K))
        if ent is None:
            # sub-chunks per shard: finer arrival granularity for small groups; every sub-chunk costs each SM a
            # pipeline restart and a system-scope fence, so there are few
            nsub = 1
            limit = int(os.environ.get("TESSERACT_AG_NSUB", "0")) or (2 if self.world <= 2 else 1)
            while nsub * 2 <= limit and (rpr // 128) % (nsub * 2) == 0 and rpr * K * 2 // (nsub * 2) >= (8 << 20):
                nsub *= 2
            if self._flag_next + self.world * nsub > self._flag_ints:
                raise RuntimeError("ag_gemm: out of arrival counters")
            ent = [self._flag_next, 0, nsub]
            self._flag_next += self.world * nsub
            self._flags[(rpr, K)] = ent
        if phase_mask & 1:
            ent[1] += 1
        off, calls, nsub = ent
        self.wait_keep()                                   # the previous contents have been copied out
        self.barrier()                                     # every rank is done with its landing buffer
        in_kernel = keep and (self.keep_mode == "kernel" or phase_mask != 3)
        x_full = torch.empty((M, K), device=x_local.device, dtype=torch.bfloat16) if in_kernel else None
        y = torch.empty((M, N), device=x_local.device, dtype=torch.bfloat16)
        check(lib().tsb_gemm_ag(x_local.data_ptr(), land.ptr_array, self._flagmem.offset_ptr_array(4 * off),
                                x_full.data_ptr() if in_kernel else None, w.data_ptr(), y.data_ptr(), _wrap_i32(calls),
                                nsub, phase_mask, M, N, K, w.stride(0), y.stride(0), int(b_mn), rpr, self.rank, self.world,
                                self.trace.data_ptr() if self.trace is not None else None, self._stream()),
              "tsb_gemm_ag")
        self.calls["ag_gemm"] += 1
        if not in_kernel:
            landed = land.local[:M * K * 2].view(torch.bfloat16).view(M, K)
            if not keep:
                return y, landed
            main = torch.cuda.current_stream(self.device)
            if self._keep_stream is None:
                self._keep_stream = torch.cuda.Stream(self.device)
            self._keep_stream.wait_stream(main)
            with torch.cuda.stream(self._keep_stream):
                # allocated on the stream that writes it: if the caller drops the tensor early (a forward pass
                # under no_grad), the caching allocator reuses the block only after this copy in stream order ...
                x_full = torch.empty((M, K), device=x_local.device, dtype=torch.bfloat16)
                x_full.copy_(landed, non_blocking=True)
                self._keep_event = torch.cuda.Event()
                self._keep_event.record(self._keep_stream)
            x_full.record_stream(main)      # ... and its readers on the main stream are known to the allocator too
        return y, x_full

    def close(self) -> None:
        for m in (self.pads, self._land, self._stage, self._flagmem):
            if m is not None:
                m.close()


class SymmAllReduce:
    """Latency-optimised all-reduce of small bf16 tensors over peer memory (``csrc/allreduce_oneshot.cu``), for
    tensor-parallel decode. Usage per call: write the partial into ``input_view(rows, cols)`` (it alternates
    between two symmetric buffers), then ``reduce(rows, cols)`` returns the sum in a regular local tensor. All
    pointers and the epoch counter live on the device, so the pair can be captured in a CUDA graph."""

    def __init__(self, group, rank: int, world: int, device, max_elems: int):
        if world > 8:
            raise ValueError("SymmAllReduce supports at most 8 ranks (one NVSwitch domain)")
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.max_elems = (max_elems + 7) // 8 * 8
        self.half_bytes = self.max_elems * 2
        self.buf = SymmetricMemory(group, rank, world, 2 * self.half_bytes, device)
        self.flags = SymmetricMemory(group, rank, world, 256, device)
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._ptrs = [self.buf.offset_ptr_array(0), self.buf.offset_ptr_array(self.half_bytes)]
        self.parity = 0
        self.calls = 0

    def input_view(self, rows: int, cols: int) -> torch.Tensor:
        n = rows * cols
        if n > self.max_elems or n % 8:
            raise ValueError("SymmAllReduce: message larger than the buffer or not a multiple of 8 elements")
        off = self.parity * self.half_bytes
        return self.buf.local[off:off + n * 2].view(torch.bfloat16).view(rows, cols)

    def reduce(self, rows: int, cols: int) -> torch.Tensor:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        check(lib().tsb_allreduce_oneshot(self._ptrs[self.parity], self.flags.ptr_array, self.state.data_ptr(),
                                          out.data_ptr(), rows * cols, self.rank, self.world,
                                          torch.cuda.current_stream(self.device).cuda_stream), "tsb_allreduce_oneshot")
        self.parity ^= 1
        self.calls += 1
        return out

    def reduce_norm(self, rows: int, cols: int, residual, weight: torch.Tensor, eps: float):
        """The all-reduce fused with the residual add and RMSNorm that follow it in a transformer block: returns
        ``(rmsnorm(h) * weight, h)`` with ``h = sum over ranks + residual`` (``residual`` may be None)."""
        y = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        h = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
        check(lib().tsb_allreduce_norm_oneshot(self._ptrs[self.parity], self.flags.ptr_array, self.state.data_ptr(),
                                               residual.data_ptr() if residual is not None else None,
                                               weight.data_ptr(), y.data_ptr(), h.data_ptr(), rows, cols, float(eps),
                                               self.rank, self.world,
                                               torch.cuda.current_stream(self.device).cuda_stream),
              "tsb_allreduce_norm_oneshot")
        self.parity ^= 1
        self.calls += 1
        return y, h

    def close(self) -> None:
        self.buf.close()
        self.flags.close()


class SymmGradAllReduce:
    """In-place all-reduce of ranges of ONE large symmetric buffer (the gradient arena of data-parallel ranks) with the
    two-shot peer-memory kernel of ``csrc/allreduce_twoshot.cu``: no NCCL, one launch per range, bounded waits.

    ``buffer`` is the ``SymmetricMemory`` that holds the data; ``all_reduce_(byte_offset, n_elems, dtype, scale)``
    reduces that range on every rank (every rank must issue the same calls in the same order, on any stream)."""

    def __init__(self, buffer: SymmetricMemory, ctas: int = 0):
        self.buf = buffer
        self.rank, self.world = buffer.rank, buffer.world
        self.device = buffer.local.device
        self.flags = SymmetricMemory(buffer.group, buffer.rank, buffer.world, 256, self.device)
        self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self.ctas = ctas or int(os.environ.get("TESSERACT_DP_CTAS", "0"))
        self.calls = 0
        self.bytes = 0

    def all_reduce_(self, byte_offset: int, n_elems: int, dtype: torch.dtype, scale: float = 1.0,
                    phase_mask: int = 7, limit_cycles: int = 0) -> None:
        code = {torch.bfloat16: 1, torch.float32: 0}.get(dtype)
        if code is None:
            raise ValueError("SymmGradAllReduce: bf16 or fp32 data only")
        if byte_offset % 16 or n_elems % (8 if code else 4):
            raise ValueError("SymmGradAllReduce: ranges start on 16 bytes and hold whole 16-byte vectors")
        if phase_mask & 1:
            self.epoch += 1
        check(lib().tsb_allreduce_twoshot(self.buf.offset_ptr_array(byte_offset), self.flags.ptr_array,
                                          self.state.data_ptr(), n_elems, code, self.rank, self.world,
                                          _wrap_i32(self.epoch), float(scale), self.ctas, phase_mask, limit_cycles,
                                          torch.cuda.current_stream(self.device).cuda_stream),
              "tsb_allreduce_twoshot")
        self.calls += 1
        self.bytes += n_elems * (2 if code else 4)

    def close(self) -> None:
        self.flags.close()
