"""Observability helpers: device stage timers, NVTX ranges, a launch census and a flight recorder.

Counterparts in the reference: per-stage timing rows (``LOAD_TIMING``, prefill / decode stage timers in
``hipengine/runtime/qwen35_gguf_runner.py``), the launch-census counters its decode-graph work relies on, and the
bounded in-memory event log its server attaches to failure reports.  All four are opt-in and cost nothing when off.
"""
from __future__ import annotations

import collections
import contextlib
import json
import threading
import time
from typing import Any, Deque, Dict, Iterator, List, Optional

import torch


class StageTimer:
    """Named stages timed with CUDA events on the current stream (or wall clock on CPU).

    Events are only recorded, never synchronised, inside ``stage``; ``summary`` synchronises once and reads all of
    them, so timing a decode step does not serialise it.
    """

    def __init__(self, enabled: bool = True, use_cuda: Optional[bool] = None):
        self.enabled = enabled
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self._pending: List[Any] = []
        self._wall: Dict[str, List[float]] = collections.defaultdict(list)

    @contextlib.contextmanager
    def stage(self, name: str) -> Iterator[None]:
        if not self.enabled:
            yield
            return
        if self.use_cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._pending.append((name, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._wall[name].append(1e3 * (time.perf_counter() - t0))

    def summary(self) -> Dict[str, Dict[str, float]]:
        if self.use_cuda and self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self._wall[name].append(a.elapsed_time(b))
            self._pending.clear()
        out = {}
        for name, xs in self._wall.items():
            s = sorted(xs)
            out[name] = {"count": len(xs), "total_ms": sum(xs), "mean_ms": sum(xs) / len(xs),
                         "p50_ms": s[len(s) // 2], "max_ms": s[-1]}
        return out

    def reset(self) -> None:
        self._pending.clear()
        self._wall.clear()


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True) -> Iterator[None]:
    """NVTX range visible to profilers; a no-op without CUDA."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class LaunchCensus:
    """Counts kernel launches of the native library per labelled region (reads ``core.native.launch_count``)."""

    def __init__(self) -> None:
        self.counts: Dict[str, int] = collections.defaultdict(int)
        self.calls: Dict[str, int] = collections.defaultdict(int)

    @contextlib.contextmanager
    def region(self, label: str) -> Iterator[None]:
        from ..core import native
        k0 = native.launch_count()
        try:
            yield
        finally:
            self.counts[label] += native.launch_count() - k0
            self.calls[label] += 1

    def report(self) -> Dict[str, Dict[str, float]]:
        return {k: {"launches": v, "calls": self.calls[k], "per_call": v / max(1, self.calls[k])}
                for k, v in self.counts.items()}


class FlightRecorder:
    """Bounded ring of recent engine events (admissions, rounds, failures) for post-mortems.

    Thread-safe; ``dump`` returns a JSON-serialisable list, newest last.  The engine service attaches it to the
    ``unhealthy`` report so a failed server can say what it was doing.
    """

    def __init__(self, capacity: int = 512):
        self.capacity = capacity
        self._events: Deque[Dict[str, Any]] = collections.deque(maxlen=capacity)
        self._lock = threading.Lock()
        self._seq = 0

    def record(self, kind: str, **fields: Any) -> None:
        with self._lock:
            self._seq += 1
            self._events.append({"seq": self._seq, "t": time.time(), "kind": kind, **fields})

    def dump(self, last: Optional[int] = None) -> List[Dict[str, Any]]:
        with self._lock:
            ev = list(self._events)
        return ev if last is None else ev[-last:]

    def dump_json(self, last: Optional[int] = None) -> str:
        return json.dumps(self.dump(last), default=str)

    def __len__(self) -> int:
        return len(self._events)
