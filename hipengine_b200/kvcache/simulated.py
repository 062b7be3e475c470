"""Host-only KV backend for conformance tests of schedulers and admission logic.

Same surface as the GPU runner's KV handling (admit with shared prefix, append, fork copy-on-write, release,
capacity report) on top of the real ``PagePool`` / ``RadixCache`` with no device memory, so host tests exercise
the production bookkeeping.  Reference: ``hipengine/kvcache/simulated.py:53,313`` (``SimulatedKVBackend``,
``create_fake_kv_backend``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

from .pool import KVLease, PagePool, PoolExhausted
from .radix import PrefixCompatibilityKey, RadixCache


class SimulatedKVBackend:
    def __init__(self, capacity_tokens: int, page_tokens: int = 16, prefix_cache: bool = True):
        self.page = page_tokens
        self.pool = PagePool(capacity_tokens // page_tokens + 1, page_tokens)
        self.radix = RadixCache(page_tokens, PrefixCompatibilityKey("simulated", page_tokens=page_tokens))
        self.radix.on_retain = self.pool.retain_cache
        self.radix.on_release = lambda pages: self.pool.release_cache(pages)
        self.radix.page_refcount = lambda p: self.pool.refcount[p]
        self.pool.evict_hook = self.radix.evict
        self.use_prefix = prefix_cache
        self.writes: Dict[int, int] = {}          # page -> tokens written (what a device backend would hold)

    def admit(self, rid: int, prompt: Sequence[int], max_tokens: int) -> Optional[KVLease]:
        """Returns the lease (``lease.cached_tokens`` tokens already present) or None when the pool is full."""
        match = self.radix.match(list(prompt)) if self.use_prefix else None
        shared = match.pages if match and match.tokens else []
        try:
            lease = self.pool.admit(rid, len(prompt) + max_tokens, shared_prefix=shared, now_tokens=len(prompt))
        except PoolExhausted:
            return None
        lease.cached_tokens = match.tokens if shared else 0
        for p in lease.pages[len(shared):]:
            self.writes[p] = self.page
        return lease

    def append(self, lease: KVLease, upto_tokens: int) -> None:
        before = len(lease.pages)
        self.pool.append_pages(lease, upto_tokens)
        for p in lease.pages[before:]:
            self.writes[p] = self.page

    def publish_prefix(self, prompt: Sequence[int], lease: KVLease) -> int:
        n = (len(prompt) // self.page) * self.page if self.use_prefix else 0
        if n:
            self.radix.insert(list(prompt[:n]), lease.pages[:n // self.page])
        return n

    def release(self, rid: int) -> None:
        self.pool.release(rid)

    def capacity(self) -> Dict[str, object]:
        return {"kv_pool": self.pool.snapshot(), "prefix_cache": self.radix.snapshot_stats()}


def create_fake_kv_backend(kind: str = "paged", capacity_tokens: int = 4096, **kw) -> SimulatedKVBackend:
    if kind not in ("paged", "paged_noprefix"):
        raise ValueError(f"unknown fake KV backend {kind!r}")
    return SimulatedKVBackend(capacity_tokens, prefix_cache=(kind == "paged"), **kw)
