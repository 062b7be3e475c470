"""Named-resource ledger with fit-aware admission.

Every device-memory consumer that scales with traffic (KV pages, recurrent-state slots, snapshot slots, verify
journals, scratch) registers a capacity; a request's admission is a *claim set* that either fits as a whole or is
refused as a whole (``ResourceUnavailable``), never partially.  Follows the reference's ``ResourceLedger``
(``hipengine/kvcache/ledger.py``) and its ``ResourceClaim(Set)`` contracts (``hipengine/kvcache/backend.py``).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class ResourceUnavailable(RuntimeError):
    def __init__(self, resource: str, requested: int, available: int):
        super().__init__(f"resource {resource!r}: requested {requested}, available {available}")
        self.resource, self.requested, self.available = resource, requested, available


@dataclass(frozen=True)
class ResourceClaim:
    resource: str
    amount: int


@dataclass
class ClaimSet:
    owner: str
    claims: Tuple[ResourceClaim, ...]
    released: bool = False


@dataclass
class _Resource:
    capacity: int
    used: int = 0
    peak: int = 0
    refused: int = 0
    holders: Dict[str, int] = field(default_factory=dict)


class ResourceLedger:
    def __init__(self) -> None:
        self._res: Dict[str, _Resource] = {}
        self._lock = threading.Lock()

    def register(self, name: str, capacity: int) -> None:
        with self._lock:
            if name in self._res:
                raise ValueError(f"resource {name!r} already registered")
            self._res[name] = _Resource(int(capacity))

    def resize(self, name: str, capacity: int) -> None:
        with self._lock:
            r = self._res[name]
            if capacity < r.used:
                raise ResourceUnavailable(name, r.used, capacity)
            r.capacity = int(capacity)

    def available(self, name: str) -> int:
        r = self._res[name]
        return r.capacity - r.used

    def fits(self, claims: List[ResourceClaim]) -> Optional[ResourceClaim]:
        """First claim that does not fit, or None when the whole set fits."""
        need: Dict[str, int] = {}
        for c in claims:
            need[c.resource] = need.get(c.resource, 0) + c.amount
        for name, amt in need.items():
            if name not in self._res:
                return ResourceClaim(name, amt)
            if amt > self.available(name):
                return ResourceClaim(name, amt)
        return None

    def acquire(self, owner: str, claims: List[ResourceClaim]) -> ClaimSet:
        with self._lock:
            bad = self.fits(claims)
            if bad is not None:
                r = self._res.get(bad.resource)
                if r is not None:
                    r.refused += 1
                raise ResourceUnavailable(bad.resource, bad.amount, self.available(bad.resource) if r else 0)
            for c in claims:
                r = self._res[c.resource]
                r.used += c.amount
                r.peak = max(r.peak, r.used)
                r.holders[owner] = r.holders.get(owner, 0) + c.amount
            return ClaimSet(owner, tuple(claims))

    def release(self, cs: ClaimSet) -> None:
        with self._lock:
            if cs.released:
                return
            for c in cs.claims:
                r = self._res[c.resource]
                r.used -= c.amount
                left = r.holders.get(cs.owner, 0) - c.amount
                if left <= 0:
                    r.holders.pop(cs.owner, None)
                else:
                    r.holders[cs.owner] = left
            cs.released = True

    def snapshot(self) -> Dict[str, Dict[str, int]]:
        with self._lock:
            return {n: {"capacity": r.capacity, "used": r.used, "peak": r.peak, "refused": r.refused,
                        "holders": len(r.holders)} for n, r in self._res.items()}
