"""Global paged KV pool: host-side page accounting with refcounts, credit reservations and leases.

State machine and API follow the reference's ``GlobalKVPoolSet``
(``hipengine/kvcache/global_pool.py:26-34`` page states, ``:225-283`` append/truncate,
``:480-498`` in-flight epochs, ``:506-518`` cache retain/release, ``:593`` assert_conserved).  Prefixes are shared
at page boundaries only and a request always owns its last, partial page, so no page is ever written while shared
and the reference's copy-on-write step has nothing to do here.  Pages are ``page_tokens`` (16 by default) tokens wide; the device tensors they
index live in the executor (one ``[n_pages, 2, Hkv, page, D]`` tensor per full-attention layer), so a page
id addresses the same slot in every layer.  Page 0 is reserved as a write sink for padded rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, Iterable, List, Optional, Sequence


class PageState(str, Enum):
    FREE = "free"
    ACTIVE_PRIVATE = "active_private"
    ACTIVE_SHARED = "active_shared"
    CACHED_EVICTABLE = "cached_evictable"
    PINNED_SESSION = "pinned_session"
    RESERVED_CREDIT = "reserved_credit"
    IN_FLIGHT = "in_flight"


class PoolExhausted(RuntimeError):
    """Not enough free or evictable pages to satisfy a request."""


@dataclass
class KVLease:
    """Pages held by one request: a shared (read-only, refcounted) prefix then private pages."""
    owner: int
    pages: List[int] = field(default_factory=list)
    n_shared: int = 0            # leading pages that are shared with the prefix cache / other leases
    credit: int = 0              # reserved-but-unmaterialised growth pages
    tokens: int = 0              # tokens written so far

    @property
    def private_pages(self) -> List[int]:
        return self.pages[self.n_shared:]


class PagePool:
    def __init__(self, n_pages: int, page_tokens: int = 16, reserved: int = 1):
        if n_pages <= reserved:
            raise ValueError("pool needs at least one usable page")
        self.n_pages = n_pages
        self.page_tokens = page_tokens
        self.reserved = reserved
        self.refcount = [0] * n_pages
        self.cached = [False] * n_pages           # retained by the prefix cache
        self.pinned = [False] * n_pages
        self.in_flight: Dict[int, int] = {}       # page -> epoch
        self.free: List[int] = list(range(n_pages - 1, reserved - 1, -1))
        self.credit_total = 0
        self.leases: Dict[int, KVLease] = {}
        self.epoch = 0
        self.evict_hook: Optional[Callable[[int], List[int]]] = None  # asks the prefix cache to give pages back
        self.stats = {"grants": 0, "truncated": 0, "evictions": 0, "peak_used": 0}

    # -- queries
    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_tokens - 1) // self.page_tokens

    @property
    def n_free(self) -> int:
        return len(self.free)

    @property
    def n_available(self) -> int:
        """Pages an admission may count on: free minus growth credits already promised."""
        return len(self.free) - self.credit_total

    def n_evictable(self) -> int:
        return sum(1 for p in range(self.reserved, self.n_pages)
                   if self.cached[p] and self.refcount[p] == 0 and not self.pinned[p])

    def state_of(self, p: int) -> PageState:
        if p in self.in_flight:
            return PageState.IN_FLIGHT
        if self.pinned[p]:
            return PageState.PINNED_SESSION
        if self.refcount[p] == 0:
            return PageState.CACHED_EVICTABLE if self.cached[p] else PageState.FREE
        if self.refcount[p] > 1 or self.cached[p]:
            return PageState.ACTIVE_SHARED
        return PageState.ACTIVE_PRIVATE

    # -- allocation
    def _take(self, n: int) -> List[int]:
        if n > len(self.free) and self.evict_hook is not None:
            got = self.evict_hook(n - len(self.free))
            self.stats["evictions"] += len(got)
        if n > len(self.free):
            raise PoolExhausted(f"need {n} pages, {len(self.free)} free")
        out = [self.free.pop() for _ in range(n)]
        used = self.n_pages - self.reserved - len(self.free)
        self.stats["peak_used"] = max(self.stats["peak_used"], used)
        return out

    def admit(self, owner: int, total_tokens: int, shared_prefix: Sequence[int] = (), now_tokens: int = 0) -> KVLease:
        """Create a lease able to grow to ``total_tokens``.

        ``shared_prefix`` pages are referenced (not copied).  Pages covering ``now_tokens`` are materialised;
        the rest of the budget is held as growth credit so a running request can never starve mid-decode.
        """
        if owner in self.leases:
            raise ValueError(f"owner {owner} already holds a lease")
        need_total = self.pages_for(total_tokens)
        n_sh = len(shared_prefix)
        need_now = max(self.pages_for(now_tokens), n_sh) - n_sh
        credit = max(0, need_total - n_sh - need_now)
        # Reference the shared prefix FIRST: from here on its pages are neither counted as reclaimable nor offered
        # to the eviction hook, so making room for the private pages can never hand a matched prefix page back as
        # one of this lease's own pages.
        for p in shared_prefix:
            self.refcount[p] += 1
        try:
            if need_now + credit > self.n_available + self._reclaimable():
                raise PoolExhausted(f"request needs {need_now + credit} pages; {self.n_available} available")
            pages = self._take(need_now)
        except PoolExhausted:
            for p in shared_prefix:
                self._unref(p)
            raise
        for p in pages:
            self.refcount[p] = 1
        lease = KVLease(owner, list(shared_prefix) + pages, n_sh, credit, 0)
        self.credit_total += credit
        self.leases[owner] = lease
        self.stats["grants"] += 1
        return lease

    def _reclaimable(self) -> int:
        return self.n_evictable() if self.evict_hook is not None else 0

    def append_pages(self, lease: KVLease, upto_tokens: int) -> List[int]:
        """Materialise pages so the lease covers ``upto_tokens`` (drawn from its credit first)."""
        need = self.pages_for(upto_tokens) - len(lease.pages)
        if need <= 0:
            return []
        from_credit = min(need, lease.credit)
        if need - from_credit > self.n_available + self._reclaimable():
            raise PoolExhausted("growth beyond the admitted budget does not fit")
        lease.credit -= from_credit
        self.credit_total -= from_credit
        pages = self._take(need)
        for p in pages:
            self.refcount[p] = 1
        lease.pages += pages
        return pages

    def truncate_pages(self, lease: KVLease, keep_tokens: int) -> List[int]:
        """Drop pages past ``keep_tokens`` (speculative rollback); dropped pages return to credit."""
        keep = max(self.pages_for(keep_tokens), lease.n_shared)
        dropped = lease.pages[keep:]
        lease.pages = lease.pages[:keep]
        for p in dropped:
            self._unref(p)
        lease.credit += len(dropped)
        self.credit_total += len(dropped)
        lease.tokens = min(lease.tokens, keep_tokens)
        self.stats["truncated"] += len(dropped)
        return dropped

    def release(self, owner: int) -> None:
        lease = self.leases.pop(owner, None)
        if lease is None:
            return
        for p in lease.pages:
            self._unref(p)
        self.credit_total -= lease.credit
        lease.pages, lease.credit = [], 0

    def _unref(self, p: int) -> None:
        self.refcount[p] -= 1
        if self.refcount[p] < 0:
            raise AssertionError(f"page {p} refcount underflow")
        if self.refcount[p] == 0 and not self.cached[p] and not self.pinned[p] and p not in self.in_flight:
            self.free.append(p)

    # -- prefix-cache retention
    def retain_cache(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.cached[p] = True

    def release_cache(self, pages: Iterable[int]) -> List[int]:
        freed = []
        for p in pages:
            if not self.cached[p]:
                continue
            self.cached[p] = False
            if self.refcount[p] == 0 and not self.pinned[p] and p not in self.in_flight:
                self.free.append(p)
                freed.append(p)
        return freed

    def pin(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.pinned[p] = True

    def unpin(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.pinned[p] = False
            if self.refcount[p] == 0 and not self.cached[p] and p not in self.in_flight and p not in self.free:
                self.free.append(p)

    # -- in-flight epochs: pages a launched graph may still read cannot be recycled until the epoch retires
    def mark_in_flight(self, pages: Iterable[int]) -> int:
        self.epoch += 1
        for p in pages:
            self.in_flight[p] = self.epoch
        return self.epoch

    def retire_epoch(self, epoch: int) -> None:
        done = [p for p, e in self.in_flight.items() if e <= epoch]
        for p in done:
            del self.in_flight[p]
            if self.refcount[p] == 0 and not self.cached[p] and not self.pinned[p] and p not in self.free:
                self.free.append(p)

    # -- invariants
    def assert_conserved(self) -> None:
        free = set(self.free)
        if len(free) != len(self.free):
            raise AssertionError("duplicate page on the free list")
        refs = [0] * self.n_pages
        for lease in self.leases.values():
            for p in lease.pages:
                refs[p] += 1
        for p in range(self.reserved, self.n_pages):
            if refs[p] != self.refcount[p]:
                raise AssertionError(f"page {p}: refcount {self.refcount[p]} but {refs[p]} lease references")
            idle = self.refcount[p] == 0 and not self.cached[p] and not self.pinned[p] and p not in self.in_flight
            if idle != (p in free):
                raise AssertionError(f"page {p}: idle={idle} but on_free_list={p in free}")
        if self.credit_total != sum(l.credit for l in self.leases.values()):
            raise AssertionError("credit accounting drifted")
        if self.credit_total > len(self.free) + self.n_evictable():
            raise AssertionError("more growth credit promised than pages that can be produced")

    def snapshot(self) -> Dict[str, int]:
        used = self.n_pages - self.reserved - len(self.free)
        return {"pages_total": self.n_pages - self.reserved, "pages_free": len(self.free), "pages_used": used,
                "pages_cached": sum(self.cached), "pages_credit": self.credit_total,
                "page_tokens": self.page_tokens, "leases": len(self.leases), **self.stats}
