"""HTTP-side generation batcher: bounded admission, grouping of compatible requests, batch window, drain.

The engine batches continuously on its own (every scheduling round packs whatever is resident), so what the HTTP
layer adds is *co-arrival*: requests that reach the server within ``window_ms`` of each other and are compatible
(same route family, sampler family, streaming mode) are held until the window of their group closes or the group
reaches ``max_batch``, and are then released together, so that their submissions land in the same engine command batch
and their prefill chunks are packed into the same forward pass.  With a window of 0 every request is released at once
and the batcher degenerates to a bounded counter.  Role of the reference's ``_GenerationBatcher``
(``hipengine/server/api.py:3552-4500``: queue bound, compatible-request grouping, batch window ``:424``, drain).
"""
from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional

from .errors import APIError


@dataclass
class _Group:
    key: Hashable
    opened: float
    waiters: List[asyncio.Future] = field(default_factory=list)
    timer: Optional[asyncio.TimerHandle] = None


class GenerationBatcher:
    def __init__(self, limit: int, window_ms: float = 0.0, max_batch: int = 64):
        self.limit = limit
        self.window_s = max(0.0, window_ms) / 1e3
        self.max_batch = max(1, max_batch)
        self.in_flight = 0
        self.closing = False
        self.lock = threading.Lock()
        self.groups: Dict[Hashable, _Group] = {}
        self.stats = {"batches": 0, "requests": 0, "max_batch_seen": 0, "window_wait_seconds": 0.0,
                      "rejected_busy": 0, "flush_full": 0, "flush_window": 0, "flush_drain": 0}

    # -- bounded admission (synchronous part; raises the API error the route returns)
    def enter(self) -> None:
        with self.lock:
            if self.closing:
                raise APIError("engine_unavailable", "server is shutting down")
            if self.in_flight >= self.limit:
                self.stats["rejected_busy"] += 1
                raise APIError("engine_busy", f"{self.in_flight} requests already queued", retry_after=1.0)
            self.in_flight += 1

    def leave(self) -> None:
        with self.lock:
            self.in_flight = max(0, self.in_flight - 1)

    # -- grouping + window
    @staticmethod
    def compat_key(route: str, stream: bool, greedy: bool, logprobs: bool, constrained: bool) -> Hashable:
        """Requests with equal keys may share a release: same route family and sampler family; streaming and
        non-streaming requests are released separately (their consumers have different latency needs)."""
        return (route, bool(stream), bool(greedy), bool(logprobs), bool(constrained))

    async def admit(self, key: Hashable) -> float:
        """Wait until this request's group is released; returns the seconds spent waiting."""
        t0 = time.perf_counter()
        if self.window_s <= 0.0:
            self._count_batch(1, 0.0)
            return 0.0
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        grp = self.groups.get(key)
        if grp is None:
            grp = self.groups[key] = _Group(key, time.perf_counter())
            grp.timer = loop.call_later(self.window_s, self._flush, key, "flush_window")
        grp.waiters.append(fut)
        if len(grp.waiters) >= self.max_batch:
            self._flush(key, "flush_full")
        await fut
        waited = time.perf_counter() - t0
        self.stats["window_wait_seconds"] += waited
        return waited

    def _flush(self, key: Hashable, why: str) -> None:
        grp = self.groups.pop(key, None)
        if grp is None:
            return
        if grp.timer is not None:
            grp.timer.cancel()
        self._count_batch(len(grp.waiters), 0.0)
        self.stats[why] += 1
        for fut in grp.waiters:
            if not fut.done():
                fut.set_result(None)

    def _count_batch(self, n: int, _wait: float) -> None:
        self.stats["batches"] += 1
        self.stats["requests"] += n
        self.stats["max_batch_seen"] = max(self.stats["max_batch_seen"], n)

    def drain(self) -> None:
        """Shutdown: refuse new work and release every held group at once."""
        self.closing = True
        for key in list(self.groups):
            self._flush(key, "flush_drain")

    def snapshot(self) -> Dict[str, float]:
        s = dict(self.stats)
        s["in_flight"] = self.in_flight
        s["limit"] = self.limit
        s["window_ms"] = self.window_s * 1e3
        s["max_batch"] = self.max_batch
        s["open_groups"] = len(self.groups)
        s["mean_batch"] = (s["requests"] / s["batches"]) if s["batches"] else 0.0
        return s
