"""Host sampler: repetition penalty -> temperature -> top-k -> top-p -> multinomial draw.

Order and tie rules are the reference's (src/models/Sampler.cpp:29-116): the penalty is applied once per
occurrence in ``prev_tokens`` (x > 0 ? x / pen : x * pen); temperature <= 1e-6 means argmax (lowest index
on ties) and bypasses top-k / top-p; top-k keeps ties at the k-th value; top-p keeps the smallest prefix
(by descending logit) whose cumulative mass reaches p and always the first token; the draw walks the
survivors in index order against ``u * denom`` with ``u`` from ``uniform_real_distribution<double>`` on a
``mt19937_64`` seeded with ``seed``. The generator is re-implemented here (and natively in the host
runtime) so that seeded sequences are reproducible bit for bit; greedy decoding never touches it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np


@dataclass
class SamplingParams:
    temperature: float = 1.0         # <= 0 => greedy
    top_k: int = 0                   # 0 => disabled
    top_p: float = 1.0               # 1.0 => disabled
    repetition_penalty: float = 1.0  # 1.0 => disabled


class MT19937_64:
    """std::mt19937_64 (Matsumoto & Nishimura, 64-bit variant)."""

    NN, MM = 312, 156
    MATRIX_A = 0xB5026F5AA96619E9
    UM, LM = 0xFFFFFFFF80000000, 0x7FFFFFFF
    MASK = 0xFFFFFFFFFFFFFFFF

    def __init__(self, seed: int = 5489):
        self.seed(seed)

    def seed(self, seed: int) -> None:
        mt = [0] * self.NN
        mt[0] = seed & self.MASK
        for i in range(1, self.NN):
            mt[i] = (6364136223846793005 * (mt[i - 1] ^ (mt[i - 1] >> 62)) + i) & self.MASK
        self.mt, self.idx = mt, self.NN

    def _twist(self) -> None:
        mt, NN, MM = self.mt, self.NN, self.MM
        for i in range(NN):
            x = (mt[i] & self.UM) | (mt[(i + 1) % NN] & self.LM)
            mt[i] = mt[(i + MM) % NN] ^ (x >> 1) ^ (self.MATRIX_A if x & 1 else 0)
        self.idx = 0

    def next_u64(self) -> int:
        if self.idx >= self.NN:
            self._twist()
        x = self.mt[self.idx]
        self.idx += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & self.MASK

    def uniform_double(self) -> float:
        """libstdc++ ``uniform_real_distribution<double>(0, 1)``: one 64-bit draw scaled by 2^-64, clamped
        below 1."""
        r = float(self.next_u64()) / 18446744073709551616.0
        if r >= 1.0:
            r = float(np.nextafter(1.0, 0.0))
        return r


def argmax_lowest_index(x: np.ndarray) -> int:
    return int(np.argmax(x))  # numpy returns the first maximal index


def sample_from_logits(logits: np.ndarray, params: SamplingParams, prev_tokens: Sequence[int],
                       rng: MT19937_64) -> int:
    work = np.array(logits, dtype=np.float32, copy=True).reshape(-1)
    V = work.shape[0]
    if V == 0:
        raise ValueError("sample_from_logits: empty logits")
    if params.repetition_penalty != 1.0 and len(prev_tokens):
        pen = np.float32(params.repetition_penalty)
        for t in prev_tokens:
            if 0 <= t < V:
                work[t] = work[t] / pen if work[t] > 0 else work[t] * pen
    if params.temperature <= 1e-6:
        return argmax_lowest_index(work)
    work *= np.float32(1.0) / np.float32(params.temperature)      # float arithmetic, as in the native sampler
    ninf = np.float32(-np.inf)
    if 0 < params.top_k < V:
        kth = np.partition(work, V - params.top_k)[V - params.top_k]
        work[work < kth] = ninf
    if params.top_p < 1.0:
        # the nucleus is a prefix of the order (value descending, index ascending on ties); only that prefix is
        # sorted: all entries not below the K-th largest value, K growing until the prefix reaches top_p
        finite_all = work != ninf
        e_all = np.where(finite_all, np.exp((work - work.max()).astype(np.float64)), 0.0)
        denom = float(np.cumsum(e_all)[-1])
        K = 256
        while True:
            if K >= V:
                cand = np.arange(V)
            else:
                kth = np.partition(work, V - K)[V - K]
                cand = np.nonzero(work >= kth)[0]
            order = cand[np.argsort(-work[cand], kind="stable")]
            cum = np.cumsum(e_all[order] / denom)
            hit = np.nonzero((work[order] != ninf) & (cum >= float(np.float32(params.top_p))))[0]   # top_p is a float
            if hit.size or cand.size >= V:
                break
            K *= 8
        if hit.size:
            drop = np.ones(V, dtype=bool)
            drop[order[:int(hit[0]) + 1]] = False
            work[drop] = ninf
    maxv = work.max()
    finite = work != ninf
    e = np.where(finite, np.exp((work - maxv).astype(np.float64)), 0.0)
    denom = float(np.cumsum(e)[-1])
    if not denom > 0.0:
        raise RuntimeError("sample_from_logits: degenerate distribution")
    r = rng.uniform_double() * denom
    rem = np.subtract.accumulate(np.concatenate(([r], e)))[1:]
    hit = np.nonzero(finite & (rem <= 0.0))[0]
    if hit.size:
        return int(hit[0])
    return argmax_lowest_index(work)


def _host_module():
    """The native host runtime (csrc/host), or None when it is not built or TESSERACT_HOST=python."""
    import os
    if os.environ.get("TESSERACT_HOST", "") == "python":
        return None
    from .. import _native
    return _native.host()


class Sampler:
    """Owns the RNG of one request (src/models/Sampler.hpp `Sampler`). Runs in the native host runtime
    (std::mt19937_64 and the same pipeline in C++, csrc/host/sampler.cpp) when that is built; the Python
    implementation above is its bit-identical twin."""

    def __init__(self, params: Optional[SamplingParams] = None, seed: int = 0, native: Optional[bool] = None):
        self.params = params or SamplingParams()
        host = _host_module() if native in (None, True) else None
        if native is True and host is None:
            raise RuntimeError("Sampler: the native host runtime is not built")
        self._native = None
        if host is not None:
            self._native = host.HostSampler(float(self.params.temperature), int(self.params.top_k),
                                            float(self.params.top_p), float(self.params.repetition_penalty),
                                            int(seed) & 0xFFFFFFFFFFFFFFFF)
        self.rng = MT19937_64(seed) if self._native is None else None

    def sample(self, logits, prev_tokens: Sequence[int] = ()) -> int:
        lg = np.asarray(logits, dtype=np.float32)
        if self._native is not None:
            return int(self._native.sample(lg.reshape(-1), np.asarray(list(prev_tokens), dtype=np.int64)))
        return sample_from_logits(lg, self.params, prev_tokens, self.rng)

    def reseed(self, seed: int) -> None:
        if self._native is not None:
            self._native.reseed(int(seed) & 0xFFFFFFFFFFFFFFFF)
        else:
            self.rng.seed(seed)
