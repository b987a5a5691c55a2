"""KV caches: contiguous, INT8-quantised, paged and INT8-paged, plus the block allocator and the shared
per-layer pools.

Behaviour follows the reference (include/tesseract/nn/KVCacheBase.hpp:25-44, src/nn/KVCache.cpp:20-159,
src/nn/QuantizedKVCache.cpp:86-160, src/nn/BlockAllocator.cpp:7-52, src/nn/PagedKVPool.cpp:27-29,
src/nn/PagedKVCache.cpp:59-283):
  * contiguous cache [B, Hkv, max_len, D], zero-initialised, ``append`` of [B, Hkv, Sn, D] raises on
    overflow, ``set_current_len`` rewinds (speculative decoding, graph capture);
  * INT8 cache: one symmetric scale per (batch, head, token) row = absmax / 127 (1.0 for an all-zero
    row), round-half-even, clip to +-127, fp32 scales; reads return the dequantised prefix;
  * paged: LIFO block allocator whose first allocation is block 0, pools [num_blocks, Hkv, block, D]
    (+ fp32 scales [num_blocks, Hkv, block]), a request of length L owns ceil(L / block) blocks and
    ``reset`` frees only its own blocks.
"""
from __future__ import annotations

from typing import List, Optional

import torch


def quantize_kv_per_token(x: torch.Tensor):
    """x [..., D] -> (int8 [..., D], fp32 scale [...]); scale = absmax / 127, 1.0 for an all-zero row."""
    xf = x.float()
    absmax = xf.abs().amax(dim=-1)
    scale = torch.where(absmax > 0, absmax / 127.0, torch.ones_like(absmax))
    q = torch.clamp(torch.round(xf / scale.unsqueeze(-1)), -127, 127).to(torch.int8)
    return q, scale


def dequantize_kv_per_token(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return (q.float() * scale.unsqueeze(-1)).to(dtype)


class KVCacheBase:
    """Interface shared by every cache: ``append``, ``keys_view``, ``values_view`` and the geometry getters."""

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def keys_view(self) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def values_view(self) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def batch(self) -> int:
        return self._batch

    def num_heads(self) -> int:
        return self._heads

    def head_dim(self) -> int:
        return self._dim

    def current_len(self) -> int:
        return self._len

    def max_len(self) -> int:
        return self._max_len

    def _check_append(self, k: torch.Tensor, v: torch.Tensor) -> int:
        if k.dim() != 4 or k.shape != v.shape:
            raise ValueError("KV cache append expects k and v of identical shape [B, Hkv, S_new, D]")
        B, H, Sn, D = k.shape
        if (B, H, D) != (self._batch, self._heads, self._dim):
            raise ValueError(f"KV cache append: got [B={B}, H={H}, D={D}], cache is "
                             f"[{self._batch}, {self._heads}, {self._dim}]")
        if self._len + Sn > self._max_len:
            raise RuntimeError(f"KV cache overflow: {self._len} + {Sn} > max_len {self._max_len}")
        return Sn


class KVCache(KVCacheBase):
    def __init__(self, batch: int, num_heads: int, max_len: int, head_dim: int, dtype=torch.float32, device=None):
        self._batch, self._heads, self._max_len, self._dim = batch, num_heads, max_len, head_dim
        self._len = 0
        self.k = torch.zeros(batch, num_heads, max_len, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)

    def append(self, k, v):
        Sn = self._check_append(k, v)
        self.k[:, :, self._len:self._len + Sn] = k
        self.v[:, :, self._len:self._len + Sn] = v
        self._len += Sn

    def keys_view(self):
        return self.k[:, :, :self._len]

    def values_view(self):
        return self.v[:, :, :self._len]

    def reset(self):
        self._len = 0

    def set_current_len(self, n: int):
        if n < 0 or n > self._max_len:
            raise ValueError("set_current_len out of range")
        self._len = n


class QuantizedKVCache(KVCacheBase):
    def __init__(self, batch: int, num_heads: int, max_len: int, head_dim: int, dtype=torch.float32, device=None):
        self._batch, self._heads, self._max_len, self._dim = batch, num_heads, max_len, head_dim
        self._len = 0
        self.dtype = dtype
        self.k_q = torch.zeros(batch, num_heads, max_len, head_dim, dtype=torch.int8, device=device)
        self.v_q = torch.zeros_like(self.k_q)
        self.k_scale = torch.ones(batch, num_heads, max_len, dtype=torch.float32, device=device)
        self.v_scale = torch.ones_like(self.k_scale)

    def append(self, k, v):
        Sn = self._check_append(k, v)
        sl = slice(self._len, self._len + Sn)
        self.k_q[:, :, sl], self.k_scale[:, :, sl] = quantize_kv_per_token(k)
        self.v_q[:, :, sl], self.v_scale[:, :, sl] = quantize_kv_per_token(v)
        self._len += Sn

    def keys_view(self):
        return dequantize_kv_per_token(self.k_q[:, :, :self._len], self.k_scale[:, :, :self._len], self.dtype)

    def values_view(self):
        return dequantize_kv_per_token(self.v_q[:, :, :self._len], self.v_scale[:, :, :self._len], self.dtype)

    def reset(self):
        self._len = 0

    def set_current_len(self, n: int):
        if n < 0 or n > self._max_len:
            raise ValueError("set_current_len out of range")
        self._len = n

    def bytes(self) -> int:
        return 2 * (self.k_q.numel() + self.k_scale.numel() * 4)


def _native_block_allocator(num_blocks: int):
    import os
    if os.environ.get("TESSERACT_HOST", "") == "python":
        return None
    from .. import _native
    host = _native.host()
    return host.BlockAllocator(num_blocks) if host is not None else None


class BlockAllocator:
    """Free list of block ids; LIFO, seeded so that the first allocation returns block 0. Backed by the native
    host runtime (csrc/host/sampler.cpp `BlockAllocator`) when that is built."""

    def __new__(cls, num_blocks: int):
        if num_blocks > 0 and cls is BlockAllocator:
            nat = _native_block_allocator(num_blocks)
            if nat is not None:
                return nat
        return super().__new__(cls)

    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("BlockAllocator needs at least one block")
        self._num = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))
        self._used = set()

    def allocate(self) -> int:
        if not self._free:
            raise RuntimeError("BlockAllocator: out of KV blocks")
        b = self._free.pop()
        self._used.add(b)
        return b

    def free(self, block: int) -> None:
        if block not in self._used:
            raise RuntimeError(f"BlockAllocator: double free or foreign block {block}")
        self._used.remove(block)
        self._free.append(block)

    def num_free(self) -> int:
        return len(self._free)

    def num_blocks(self) -> int:
        return self._num

    def num_used(self) -> int:
        return len(self._used)


class PagedKVPool:
    """One layer's shared pool: K and V tensors [num_blocks, Hkv, block_size, D] and their allocator."""

    def __init__(self, num_blocks: int, num_heads: int, block_size: int, head_dim: int, dtype=torch.float32,
                 device=None):
        self.num_blocks, self.num_heads, self.block_size, self.head_dim = num_blocks, num_heads, block_size, head_dim
        self.dtype = dtype
        self.k = torch.zeros(num_blocks, num_heads, block_size, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.allocator = BlockAllocator(num_blocks)

    quantized = False


class QuantizedPagedKVPool:
    """INT8 pool [num_blocks, Hkv, block, D] with fp32 scales [num_blocks, Hkv, block]."""

    def __init__(self, num_blocks: int, num_heads: int, block_size: int, head_dim: int, dtype=torch.float32,
                 device=None):
        self.num_blocks, self.num_heads, self.block_size, self.head_dim = num_blocks, num_heads, block_size, head_dim
        self.dtype = dtype  # dtype reads are dequantised to
        self.k = torch.zeros(num_blocks, num_heads, block_size, head_dim, dtype=torch.int8, device=device)
        self.v = torch.zeros_like(self.k)
        self.k_scale = torch.ones(num_blocks, num_heads, block_size, dtype=torch.float32, device=device)
        self.v_scale = torch.ones_like(self.k_scale)
        self.allocator = BlockAllocator(num_blocks)

    quantized = True


class PagedKVCache(KVCacheBase):
    """Per-request view (batch 1) over a shared pool: a block table grown on demand."""

    def __init__(self, pool, max_len: int):
        self.pool = pool
        self._batch, self._heads, self._dim = 1, pool.num_heads, pool.head_dim
        self._max_len = max_len
        self._len = 0
        self.block_table: List[int] = []

    def _ensure_blocks(self, new_len: int) -> None:
        bs = self.pool.block_size
        need = (new_len + bs - 1) // bs
        while len(self.block_table) < need:
            self.block_table.append(self.pool.allocator.allocate())

    def _write(self, k, v, start: int, Sn: int) -> None:
        bs = self.pool.block_size
        pos = start
        off = 0
        while off < Sn:
            blk = self.block_table[pos // bs]
            slot = pos % bs
            n = min(bs - slot, Sn - off)
            self._store(blk, slot, n, k[0, :, off:off + n], v[0, :, off:off + n])
            pos += n
            off += n

    def _store(self, blk, slot, n, k, v):
        self.pool.k[blk, :, slot:slot + n] = k
        self.pool.v[blk, :, slot:slot + n] = v

    def append(self, k, v):
        Sn = self._check_append(k, v)
        self._ensure_blocks(self._len + Sn)
        self._write(k, v, self._len, Sn)
        self._len += Sn

    def reserve(self, n_new: int) -> None:
        """Allocate blocks for ``n_new`` more tokens without writing them (a fused kernel appends)."""
        if self._len + n_new > self._max_len:
            raise RuntimeError(f"KV cache overflow: {self._len} + {n_new} > max_len {self._max_len}")
        self._ensure_blocks(self._len + n_new)

    def advance(self, n_new: int) -> None:
        self._len += n_new

    def _gather(self, pool_t: torch.Tensor) -> torch.Tensor:
        bs = self.pool.block_size
        if self._len == 0:
            return pool_t.new_zeros((1, self._heads, 0) + tuple(pool_t.shape[3:]))
        idx = torch.tensor(self.block_table[: (self._len + bs - 1) // bs], device=pool_t.device)
        g = pool_t.index_select(0, idx)                  # [nb, H, bs, ...]
        g = g.transpose(0, 1).reshape(self._heads, -1, *pool_t.shape[3:])[:, :self._len]
        return g.unsqueeze(0)

    def keys_view(self):
        return self._gather(self.pool.k)

    def values_view(self):
        return self._gather(self.pool.v)

    def reset(self):
        for b in self.block_table:
            self.pool.allocator.free(b)
        self.block_table = []
        self._len = 0

    def set_current_len(self, n: int):
        bs = self.pool.block_size
        if n < 0 or n > len(self.block_table) * bs:
            raise ValueError("set_current_len: no blocks cover that length")
        self._len = n

    def num_blocks_held(self) -> int:
        return len(self.block_table)


class QuantizedPagedKVCache(PagedKVCache):
    def _store(self, blk, slot, n, k, v):
        kq, ks = quantize_kv_per_token(k)
        vq, vs = quantize_kv_per_token(v)
        self.pool.k[blk, :, slot:slot + n] = kq
        self.pool.v[blk, :, slot:slot + n] = vq
        self.pool.k_scale[blk, :, slot:slot + n] = ks
        self.pool.v_scale[blk, :, slot:slot + n] = vs

    def keys_view(self):
        return dequantize_kv_per_token(self._gather(self.pool.k), self._gather(self.pool.k_scale), self.pool.dtype)

    def values_view(self):
        return dequantize_kv_per_token(self._gather(self.pool.v), self._gather(self.pool.v_scale), self.pool.dtype)


class SSMStateCache:
    """Mamba decode state: causal-conv window [B, K-1, d_inner] and SSM state [B, d_inner, N]
    (include/tesseract/nn/SSMStateCache.hpp:25-62)."""

    def __init__(self, batch: int, d_inner: int, d_state: int, d_conv: int, dtype=torch.float32, device=None):
        self.conv_state = torch.zeros(batch, d_conv - 1, d_inner, dtype=dtype, device=device)
        self.ssm_state = torch.zeros(batch, d_inner, d_state, dtype=dtype, device=device)

    def reset(self):
        self.conv_state.zero_()
        self.ssm_state.zero_()
