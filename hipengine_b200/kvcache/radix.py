"""Radix prefix cache over complete KV pages, with recurrent-state snapshots for hybrid models.

Like the reference's ``RadixCache`` / ``BackendRadixCache`` (``hipengine/kvcache/radix.py:134-386``,
``hipengine/kvcache/backend_prefix.py:27,119-600``) the trie is indexed at complete KV-block boundaries
only, entries are scoped by a compatibility key (model / quant / layout / RoPE identity), and eviction is
LRU over unreferenced leaves with an optional TTL and per-tenant quota.  A hybrid Gated-DeltaNet model
cannot resume from KV pages alone: reuse is possible only at a boundary that also holds a snapshot of the
conv window and GDN state (``hipengine/runtime/qwen35_gguf_prefix_state.py:1-60``), so ``match`` returns
the deepest boundary carrying a snapshot when ``require_snapshot`` is set.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PrefixCompatibilityKey:
    model: str
    quant: str = ""
    kv_storage: str = "bf16"
    page_tokens: int = 16
    rope: str = ""
    adapter: str = ""
    multimodal: str = ""


@dataclass
class _Node:
    parent: Optional["_Node"]
    key: Tuple[int, ...]
    page: int
    depth: int                                  # blocks from the root (1-based)
    children: Dict[Tuple[int, ...], "_Node"] = field(default_factory=dict)
    snapshot: Optional[int] = None              # snapshot slot id holding the recurrent state at this boundary
    last_used: float = 0.0
    tenant: str = ""


@dataclass
class PrefixMatch:
    tokens: int = 0
    pages: List[int] = field(default_factory=list)
    snapshot: Optional[int] = None
    node: Optional[_Node] = None


class RadixCache:
    def __init__(self, page_tokens: int = 16, compat: Optional[PrefixCompatibilityKey] = None,
                 ttl_seconds: Optional[float] = None, tenant_quota_pages: Optional[int] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.block = page_tokens
        self.compat = compat
        self.ttl = ttl_seconds
        self.quota = tenant_quota_pages
        self.clock = clock
        self.root = _Node(None, (), -1, 0)
        self.n_nodes = 0
        self.tenant_pages: Dict[str, int] = {}
        self.stats = {"lookups": 0, "hits": 0, "hit_tokens": 0, "inserted_pages": 0, "evicted_pages": 0}
        # callbacks wired by the owner: page retention in the pool and snapshot slot recycling
        self.on_retain: Callable[[List[int]], None] = lambda pages: None
        self.on_release: Callable[[List[int]], None] = lambda pages: None
        self.on_snapshot_free: Callable[[int], None] = lambda sid: None
        # called for every block that ``evict`` is about to drop, while its page and snapshot slot still hold their
        # content: (token path from the root, page id, snapshot slot or None); a cold tier hooks in here
        self.on_evict_node: Optional[Callable[[List[int], int, Optional[int]], None]] = None
        # same for a snapshot slot that ``evict_snapshot`` takes away from a block that stays cached
        self.on_evict_snapshot: Optional[Callable[[List[int], int], None]] = None
        self.page_refcount: Callable[[int], int] = lambda p: 0

    # -- lookup
    def match(self, tokens: Sequence[int], require_snapshot: bool = False, max_tokens: Optional[int] = None,
              compat: Optional[PrefixCompatibilityKey] = None) -> PrefixMatch:
        """Longest cached block-aligned prefix of ``tokens`` (never the whole prompt: one token must remain)."""
        self.stats["lookups"] += 1
        if compat is not None and self.compat is not None and compat != self.compat:
            return PrefixMatch()
        limit = len(tokens) - 1 if max_tokens is None else min(max_tokens, len(tokens) - 1)
        node = self.root
        best = PrefixMatch()
        pages: List[int] = []
        now = self.clock()
        nblk = max(0, limit) // self.block
        for b in range(nblk):
            key = tuple(tokens[b * self.block:(b + 1) * self.block])
            child = node.children.get(key)
            if child is None or (self.ttl is not None and now - child.last_used > self.ttl):
                break
            node = child
            pages.append(node.page)
            node.last_used = now
            if not require_snapshot or node.snapshot is not None:
                best = PrefixMatch((b + 1) * self.block, list(pages), node.snapshot, node)
        if best.tokens:
            self.stats["hits"] += 1
            self.stats["hit_tokens"] += best.tokens
        return best

    # -- insertion
    def insert(self, tokens: Sequence[int], pages: Sequence[int], snapshots: Optional[Dict[int, int]] = None,
               tenant: str = "") -> int:
        """Publish the complete blocks of ``tokens`` backed by ``pages``.

        ``snapshots`` maps a token count (block-aligned) to a snapshot slot id.  Returns the number of
        newly inserted pages.  Blocks already present keep their existing page (the caller's duplicate
        page stays private to the caller).
        """
        snapshots = snapshots or {}
        nblk = min(len(tokens) // self.block, len(pages))
        node = self.root
        new_pages: List[int] = []
        now = self.clock()
        for b in range(nblk):
            key = tuple(tokens[b * self.block:(b + 1) * self.block])
            child = node.children.get(key)
            if child is None:
                if self.quota is not None and self.tenant_pages.get(tenant, 0) >= self.quota:
                    break
                child = _Node(node, key, pages[b], b + 1, tenant=tenant)
                node.children[key] = child
                self.n_nodes += 1
                self.tenant_pages[tenant] = self.tenant_pages.get(tenant, 0) + 1
                new_pages.append(pages[b])
            child.last_used = now
            sid = snapshots.get((b + 1) * self.block)
            if sid is not None:
                if child.snapshot is not None and child.snapshot != sid:
                    self.on_snapshot_free(sid)       # boundary already has one; give the duplicate back
                else:
                    child.snapshot = sid
            node = child
        if new_pages:
            self.on_retain(new_pages)
            self.stats["inserted_pages"] += len(new_pages)
        return len(new_pages)

    # -- eviction
    def _leaves(self) -> List[_Node]:
        out: List[_Node] = []
        stack = [self.root]
        while stack:
            n = stack.pop()
            if not n.children and n is not self.root:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def evict(self, n_pages: int) -> List[int]:
        """Evict up to ``n_pages`` unreferenced leaf pages in strict least-recently-used order; returns the freed
        page ids.  A parent that becomes a leaf when its last child goes joins the candidates at once (heap), so an
        old interior node is taken before a recently used leaf."""
        import heapq
        freed: List[int] = []
        heap = [(l.last_used, id(l), l) for l in self._leaves() if self.page_refcount(l.page) == 0]
        heapq.heapify(heap)
        while heap and len(freed) < n_pages:
            _, _, leaf = heapq.heappop(heap)
            if leaf.children or self.page_refcount(leaf.page) != 0:
                continue
            parent = leaf.parent
            if self.on_evict_node is not None:
                self.on_evict_node(self.token_path(leaf), leaf.page, leaf.snapshot)
            self._remove(leaf)
            freed.append(leaf.page)
            if (parent is not None and parent is not self.root and not parent.children
                    and self.page_refcount(parent.page) == 0):
                heapq.heappush(heap, (parent.last_used, id(parent), parent))
        if freed:
            self.on_release(freed)
            self.stats["evicted_pages"] += len(freed)
        return freed

    @staticmethod
    def token_path(node: _Node) -> List[int]:
        keys = []
        while node is not None and node.parent is not None:
            keys.append(node.key)
            node = node.parent
        out: List[int] = []
        for k in reversed(keys):
            out.extend(k)
        return out

    def evict_snapshot(self) -> Optional[int]:
        """Free the least-recently-used snapshot slot (its pages stay cached).  Returns the slot id."""
        best: Optional[_Node] = None
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n.snapshot is not None and (best is None or n.last_used < best.last_used):
                best = n
            stack.extend(n.children.values())
        if best is None:
            return None
        if self.on_evict_snapshot is not None:
            self.on_evict_snapshot(self.token_path(best), best.snapshot)
        sid, best.snapshot = best.snapshot, None
        return sid

    def _remove(self, node: _Node) -> None:
        if node.parent is not None:
            node.parent.children.pop(node.key, None)
        if node.snapshot is not None:
            self.on_snapshot_free(node.snapshot)
            node.snapshot = None
        self.n_nodes -= 1
        self.tenant_pages[node.tenant] = self.tenant_pages.get(node.tenant, 1) - 1

    def clear(self) -> List[int]:
        pages: List[int] = []
        stack = list(self.root.children.values())
        while stack:
            n = stack.pop()
            pages.append(n.page)
            if n.snapshot is not None:
                self.on_snapshot_free(n.snapshot)
            stack.extend(n.children.values())
        self.root.children.clear()
        self.n_nodes = 0
        self.tenant_pages.clear()
        if pages:
            self.on_release(pages)
        return pages

    def assert_consistent(self) -> None:
        seen = set()
        stack = [self.root]
        count = 0
        while stack:
            n = stack.pop()
            for k, c in n.children.items():
                assert c.parent is n and c.key == k and c.depth == n.depth + 1
                assert c.page not in seen, "a page is published twice"
                seen.add(c.page)
                count += 1
                stack.append(c)
        assert count == self.n_nodes

    def snapshot_stats(self) -> Dict[str, int]:
        return {"nodes": self.n_nodes, **self.stats}
