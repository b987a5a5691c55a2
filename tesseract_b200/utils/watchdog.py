"""Host-side failure detection for multi-rank jobs.

Every rank publishes a heartbeat counter in the job's key-value store (the torch.distributed TCPStore or any
object with ``set`` / ``get``); ``RankWatchdog.check()`` -- called between steps, before the next launch -- raises
``RankLost`` when a peer's heartbeat is older than the timeout or when a peer has posted an error. A failing rank
calls ``report_failure`` from its exception handler so that the others learn of it on the host instead of waiting
in a collective. Device-side waits are bounded separately (status word of the native library). Nothing here
touches a GPU: faults are injected in tests by raising on the host, by a rank that stops beating or never joins.

The reference has no failure detection (NCCL errors become exceptions, src/distributed/NcclCommBackend.cpp:23-38).
"""
from __future__ import annotations

import time
from typing import Dict, Optional


class RankLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} lost: {reason}")
        self.rank, self.reason = rank, reason


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process simulation)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}

    def set(self, k: str, v) -> None:
        self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        return self._d[k]

    def check(self, keys) -> bool:
        return all(k in self._d for k in keys)


class RankWatchdog:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0, prefix: str = "tsb/hb", clock=time.time):
        self.store, self.rank, self.world, self.timeout_s, self.prefix, self.clock = store, rank, world, timeout_s, prefix, clock
        self._beats = 0
        self._seen: Dict[int, tuple] = {}   # rank -> (last counter, local time it changed)
        self.beat()

    def _key(self, r: int, what: str) -> str:
        return f"{self.prefix}/{what}/{r}"

    def beat(self) -> None:
        self._beats += 1
        self.store.set(self._key(self.rank, "beat"), str(self._beats))

    def report_failure(self, message: str) -> None:
        self.store.set(self._key(self.rank, "error"), message[:500])

    def _try_get(self, key: str) -> Optional[bytes]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key)
        except Exception:
            return None

    def check(self) -> None:
        """Raise RankLost if a peer reported an error or stopped beating; call it between steps."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            err = self._try_get(self._key(r, "error"))
            if err:
                raise RankLost(r, err.decode(errors="replace"))
            raw = self._try_get(self._key(r, "beat"))
            count = int(raw) if raw else 0
            last = self._seen.get(r)
            if last is None or count != last[0]:
                self._seen[r] = (count, now)
            elif now - last[1] > self.timeout_s:
                raise RankLost(r, f"no heartbeat for {now - last[1]:.1f} s" if count else "never joined")

    def step(self) -> None:
        self.beat()
        self.check()
