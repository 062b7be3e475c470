"""GPU model runner: sm_100a executor + decode graphs + paged pool + radix prefix cache.

Admission follows the reference's resident runner (``hipengine/generation/qwen35_gguf.py:7999-8060``):
``positions = len(prompt) + max_tokens``, ``pages = ceil(positions / page)``, longest block-aligned radix
match -> shared pages (+ recurrent-state snapshot restore for hybrid models), rest of the budget held as
growth credit.  Prefill packs the chunks of several requests into one forward; decode replays a whole-step
CUDA graph for the resident rows.  Prefix reuse for hybrid Gated-DeltaNet models is only possible at
boundaries that carry a conv/GDN state snapshot (``hipengine/runtime/qwen35_gguf_prefix_state.py:1-60``), so
prefill is split at ``snapshot_interval_tokens`` and the state is copied into a snapshot slot there.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import EngineConfig
from ..kvcache.pool import KVLease, PagePool, PoolExhausted
from ..kvcache.radix import PrefixCompatibilityKey, RadixCache
from ..models.decode_graph import DecodeGraphRunner
from ..models.executor import GEMV_MAX_ROWS, PAGE, HybridExecutor, make_batch
from ..ops import kernels as K
from .runner import BaseRunner, ExecutionFailure
from .scheduler import GenerationAdmissionRejected, RequestState
from .types import TokenLogprob


class GpuRunner(BaseRunner):
    def __init__(self, weights, config: EngineConfig, eos_token_id: Optional[int] = None,
                 executor: Optional[HybridExecutor] = None):
        self.config = config
        self.cfg = weights.config if weights is not None else executor.cfg
        self.vocab = self.cfg.vocab
        self.eos_token_id = eos_token_id
        self.max_slots = config.scheduler.max_active_requests
        self.max_context = min(config.max_sequence_length, self.cfg.max_context)
        self.page = config.kv.page_tokens
        assert self.page == PAGE, "the attention kernels are built for 16-token pages"
        self.use_prefix = config.kv.prefix_cache != "off"
        self.n_snap = config.kv.max_snapshots if (self.use_prefix and self.cfg.is_hybrid) else 0
        pages_per_slot = (self.max_context + self.page - 1) // self.page
        from ..config import resolve_pool_pages
        n_pages = resolve_pool_pages(config.kv, self.cfg.kv_bytes_per_token(), self.max_slots, pages_per_slot)
        if executor is not None:
            self.ex = executor
            self.max_slots = min(self.max_slots, executor.max_slots)
            self.n_snap = min(self.n_snap, max(0, executor.max_slots - self.max_slots))
            n_pages = executor.n_pages
        else:
            # an explicit index: "cuda" alone means "this thread's current device", which differs between the
            # constructing thread and the engine's driver thread on every rank but the first
            dev = torch.device("cuda", torch.cuda.current_device())
            from ..models import make_executor
            self.ex = make_executor(weights, device=dev, max_slots=self.max_slots + self.n_snap,
                                    max_context=self.max_context, n_pages=n_pages)
        self.device = self.ex.device
        self.pool = PagePool(n_pages, self.page)
        self.radix = RadixCache(self.page, PrefixCompatibilityKey(self.cfg.arch, kv_storage=config.kv.storage,
                                                                  page_tokens=self.page,
                                                                  rope=f"{self.cfg.rope_theta}:{self.cfg.rope_dim}"))
        self.radix.on_retain = self.pool.retain_cache
        # optional cold tier: blocks the radix cache evicts are kept, compressed, in host memory or on disk and are
        # brought back at admission when that beats recomputing them (single-GPU engines only: the ranks of a
        # tensor-parallel job would have to take identical restore decisions)
        self.cold = None
        self.cold_snap: Dict[str, bool] = {}
        if config.kv.cold_tier_bytes > 0 and self.use_prefix and executor is None:
            from ..kvcache.tiering import ColdTier
            self.cold = ColdTier(config.kv.cold_tier_bytes, config.kv.cold_tier_dir)
            self.radix.on_evict_node = self._offload_block
            self.radix.on_evict_snapshot = self._offload_snapshot
        self.radix.on_release = lambda pages: self.pool.release_cache(pages)
        self.radix.page_refcount = lambda p: self.pool.refcount[p]
        self.radix.on_snapshot_free = self._free_snapshot
        self.pool.evict_hook = self.radix.evict
        self.free_slots = list(range(self.max_slots - 1, -1, -1))
        self.free_snaps = list(range(self.max_slots + self.n_snap - 1, self.max_slots - 1, -1))
        # every traffic-scaled device resource besides KV pages (which the pool accounts for with its own credits) is
        # claimed through the ledger: a request is admitted only if its whole claim set fits
        from ..kvcache.ledger import ResourceLedger
        self.ledger = ResourceLedger()
        self.ledger.register("state_slots", self.max_slots)
        self.ledger.register("snapshot_slots", self.n_snap)
        self._claims: Dict[str, Any] = {}
        self._snap_claims: Dict[int, Any] = {}
        # kernel launches of the native library per phase (prefill / decode / speculative), part of snapshot()
        from ..utils.tracing import LaunchCensus
        self.census = LaunchCensus()
        self.graphs = DecodeGraphRunner(self.ex, max_rows=self.max_slots, use_graphs=config.use_cuda_graphs)
        self.resident_key: Tuple[int, ...] = ()
        self.pinned_ids = torch.zeros(max(self.max_slots, 8), dtype=torch.int64).pin_memory()
        # the kernels' status word rides along with every per-step read-back (see _sync_checked)
        self.pinned_status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.status_word = K.status_tensor(self.device)
        self.stats = {"prefix_hits": 0, "prefix_hit_tokens": 0, "snapshots_taken": 0, "h2d_bytes": 0, "d2h_bytes": 0}
        # Speculative decoding: a provider drafts (the checkpoint's own NextN block, ``speculative/mtp.py``, or a
        # host drafter over the token history, ``speculative/providers.py``), the target verifies the chain
        self.mtp = None
        if config.speculative.mode not in ("off", "", None):
            from ..speculative.providers import SpeculativeProviderConfig, build_speculative_provider
            self.mtp = build_speculative_provider(
                self.ex, SpeculativeProviderConfig(name=config.speculative.mode,
                                                   max_depth=max(1, config.speculative.draft_depth),
                                                   hot_vocab=config.speculative.hot_vocab,
                                                   draft_model=config.speculative.draft_model),
                max_requests=min(self.max_slots, 8))
        self.supports_mtp = self.mtp is not None
        self.spec_uses_history = self.mtp is not None and hasattr(self.mtp, "drafter")
        # hot-vocabulary draft head: per-request rule over the request's own committed tokens decides, cycle by
        # cycle, whether the NextN draft may score only the leading slice of the head
        self.draft_vocab = None
        if getattr(self.mtp, "draft_head_rows", 0) > 0:
            from ..speculative.draft_vocab import DraftVocabBook
            self.draft_vocab = DraftVocabBook(self.mtp.draft_head_rows)

    # ------------------------------------------------------------------ snapshots
    def _free_snapshot(self, sid: int) -> None:
        if sid not in self.free_snaps:
            self.free_snaps.append(sid)
        claim = self._snap_claims.pop(sid, None)
        if claim is not None:
            self.ledger.release(claim)

    def _alloc_snapshot(self) -> Optional[int]:
        if self.free_snaps:
            from ..kvcache.ledger import ResourceClaim
            sid = self.free_snaps.pop()
            self._snap_claims[sid] = self.ledger.acquire(f"snapshot:{sid}", [ResourceClaim("snapshot_slots", 1)])
            return sid
        sid = self.radix.evict_snapshot()      # reuses a slot that is already claimed
        return sid

    def _copy_state(self, src: int, dst: int) -> None:
        for t in self.ex.conv_state.values():
            t[dst].copy_(t[src])
        for t in self.ex.gdn_state.values():
            t[dst].copy_(t[src])

    # ------------------------------------------------------------------ cold tier
    def _offload_block(self, tokens: List[int], page: int, snapshot: Optional[int]) -> None:
        """Radix eviction hook: keep the block's KV rows (and the recurrent-state snapshot at its boundary)."""
        from ..kvcache.tiering import prefix_key
        arrays = {f"kv.{i}": t[page] for i, t in self.ex.kv.items()}
        if snapshot is not None:
            arrays.update(self._snapshot_arrays(snapshot))
        key = prefix_key(self.radix.compat, tokens)
        if self.cold.put(key, arrays, {"tokens": len(tokens), "snapshot": snapshot is not None}) is not None:
            self.cold_snap[key] = snapshot is not None or (key + ".s") in self.cold
            self.stats["cold_offloaded_blocks"] = self.stats.get("cold_offloaded_blocks", 0) + 1

    def _snapshot_arrays(self, sid: int) -> Dict[str, torch.Tensor]:
        out = {f"conv.{i}": t[sid] for i, t in self.ex.conv_state.items()}
        out.update({f"gdn.{i}": t[sid] for i, t in self.ex.gdn_state.items()})
        return out

    def _offload_snapshot(self, tokens: List[int], sid: int) -> None:
        """A snapshot slot is being recycled while its block stays cached: keep the state as its own object."""
        from ..kvcache.tiering import prefix_key
        key = prefix_key(self.radix.compat, tokens)
        if self.cold.put(key + ".s", self._snapshot_arrays(sid), {"tokens": len(tokens)}) is not None:
            self.cold_snap[key] = True

    def _restore_from_cold(self, prompt: Sequence[int], matched_tokens: int) -> int:
        """Extend the usable cached prefix of ``prompt`` (``matched_tokens`` so far) with content of the cold tier:
        evicted blocks get fresh pages, and for hybrid models the recurrent state of the last restored boundary
        gets a snapshot slot (its block may be cold too, or still cached with its snapshot slot recycled).
        Returns the number of tokens by which the usable prefix grew."""
        from ..kvcache.tiering import prefix_key, restore_is_worthwhile
        page, hybrid = self.page, self.cfg.is_hybrid
        limit = (len(prompt) - 1) // page
        present = self.radix.match(prompt, require_snapshot=False)      # blocks whose pages are still in the pool
        b0 = present.tokens // page
        keys = [prefix_key(self.radix.compat, prompt[:(b + 1) * page]) for b in range(limit)]
        run, stored, raw = [], 0, 0
        for b in range(b0, limit):
            info = self.cold.index.get(keys[b])
            if info is None:
                break
            run.append(keys[b])
            stored += info.stored_bytes
            raw += max(info.raw_bytes, info.stored_bytes)
        end = b0 + len(run)                          # blocks available in pool + cold
        if hybrid:                                   # usable only up to a boundary whose state is available
            while end * page > matched_tokens and not self.cold_snap.get(keys[end - 1], False):
                end -= 1
        if end * page <= matched_tokens:
            return 0
        n = max(0, end - b0)                         # cold blocks that need pages
        run = run[:n]
        if not restore_is_worthwhile(end * page - matched_tokens, stored, raw,
                                     self.config.kv.cold_restore_prefill_tok_s):
            self.stats["cold_declined"] = self.stats.get("cold_declined", 0) + 1
            return 0
        held = list(present.pages)
        for pg in held:                              # the blocks still cached must survive the steps below
            self.pool.refcount[pg] += 1
        try:
            short = n + 1 - (len(self.pool.free) - self.pool.credit_total)
            if n and short > 0:
                self.radix.evict(short)
                if len(self.pool.free) - self.pool.credit_total < n + 1:
                    return 0
            loaded = []
            for key in run:
                got = self.cold.get(key)
                if got is None:                      # dropped or corrupt
                    return 0
                loaded.append(got[0])
            sid, state = None, None
            if hybrid:
                if loaded and end == b0 + n and any(k.startswith("conv.") for k in loaded[-1]):
                    state = loaded[-1]
                else:
                    got = self.cold.get(keys[end - 1] + ".s")
                    if got is None:
                        return 0
                    state = got[0]
                sid = self._alloc_snapshot()
                if sid is None:
                    return 0
            new_pages = self.pool._take(n) if n else []
            for pg, arrays in zip(new_pages, loaded):
                for i, t in self.ex.kv.items():
                    t[pg].copy_(arrays[f"kv.{i}"])
            if sid is not None:
                for i, t in self.ex.conv_state.items():
                    t[sid].copy_(state[f"conv.{i}"])
                for i, t in self.ex.gdn_state.items():
                    t[sid].copy_(state[f"gdn.{i}"])
            pages = (held + new_pages)[:end]
            self.radix.insert(prompt[:end * page], pages, {end * page: sid} if sid is not None else None)
            for pg in new_pages:                     # a block the trie did not take (quota) goes back to the pool
                if not self.pool.cached[pg]:
                    self.pool.free.append(pg)
        finally:
            for pg in held:
                self.pool.refcount[pg] -= 1
        self.stats["cold_restored_blocks"] = self.stats.get("cold_restored_blocks", 0) + n
        self.stats["cold_restored_tokens"] = self.stats.get("cold_restored_tokens", 0) + end * page - matched_tokens
        self.stats["h2d_bytes"] += raw
        return end * page - matched_tokens

    # ------------------------------------------------------------------ admission
    def admit(self, rs: RequestState) -> bool:
        total = rs.total_budget_tokens
        if total > self.max_context:
            raise GenerationAdmissionRejected(
                f"context_overflow: prompt {rs.prompt_len} + max_tokens {rs.req.max_tokens} exceeds {self.max_context}")
        from ..kvcache.ledger import ResourceClaim, ResourceUnavailable
        try:
            claim = self.ledger.acquire(str(rs.rid), [ResourceClaim("state_slots", 1)])
        except ResourceUnavailable:
            return False
        prompt = rs.req.prompt_token_ids
        match = self.radix.match(prompt, require_snapshot=self.cfg.is_hybrid) if self.use_prefix else None
        if self.cold is not None and len(self.cold) and match is not None:
            if self._restore_from_cold(prompt, match.tokens):
                match = self.radix.match(prompt, require_snapshot=self.cfg.is_hybrid)
        shared = match.pages if match and match.tokens else []
        try:
            lease = self.pool.admit(rs.rid, total, shared_prefix=shared, now_tokens=rs.prompt_len)
        except PoolExhausted:
            self.ledger.release(claim)
            if self.pool.pages_for(total) > self.pool.n_pages - self.pool.reserved:
                raise GenerationAdmissionRejected("context_overflow: request exceeds the whole KV pool") from None
            return False
        self._claims[str(rs.rid)] = claim
        slot = self.free_slots.pop()
        rs.slot = slot
        rs.runner_data = lease
        self.ex.reset_slot(slot)
        if self.mtp is not None:
            self.mtp.reset_slot(slot)
        if shared:
            if self.cfg.is_hybrid and match.snapshot is not None:
                self._copy_state(match.snapshot, slot)
            rs.prefilled = rs.cached_tokens = match.tokens
            self.stats["prefix_hits"] += 1
            self.stats["prefix_hit_tokens"] += match.tokens
        self._write_block_table(slot, lease)
        return True

    def _write_block_table(self, slot: int, lease: KVLease, start: int = 0) -> None:
        pages = lease.pages[start:]
        if pages:
            t = torch.tensor(pages, dtype=torch.int32)
            self.ex.block_table[slot, start:start + len(pages)].copy_(t, non_blocking=True)
            self.stats["h2d_bytes"] += 4 * len(pages)

    def _ensure_pages(self, rs: RequestState, upto_tokens: int) -> None:
        lease: KVLease = rs.runner_data
        before = len(lease.pages)
        self.pool.append_pages(lease, upto_tokens)
        if len(lease.pages) > before:
            self._write_block_table(rs.slot, lease, before)

    # ------------------------------------------------------------------ prefill
    def prefill(self, work: List[Tuple[RequestState, int]]) -> Dict[int, Tuple[int, Optional[TokenLogprob]]]:
        with self.census.region("prefill"):
            return self._prefill_impl(work)

    @torch.no_grad()
    def _prefill_impl(self, work: List[Tuple[RequestState, int]]) -> Dict[int, Tuple[int, Optional[TokenLogprob]]]:
        out: Dict[int, Tuple[int, Optional[TokenLogprob]]] = {}
        interval = self.config.kv.snapshot_interval_tokens if self.n_snap else 0
        # split every chunk at snapshot boundaries, then run the sub-chunks round by round as packed batches
        plans: List[List[Tuple[int, int]]] = []
        for rs, n in work:
            cur, end, parts = rs.prefilled, rs.prefilled + n, []
            while cur < end:
                nxt = end
                if interval:
                    b = (cur // interval + 1) * interval
                    nxt = min(end, b)
                parts.append((cur, nxt))
                cur = nxt
            plans.append(parts)
        rounds = max(len(p) for p in plans)
        try:
            for r in range(rounds):
                segs, owners = [], []
                for (rs, n), parts in zip(work, plans):
                    if r < len(parts):
                        a, b = parts[r]
                        self._ensure_pages(rs, b)
                        toks = rs.req.prompt_token_ids[a:b]
                        segs.append((rs.slot, a, toks))
                        owners.append((rs, a, b))
                        rs.telemetry.h2d_bytes += 24 * (b - a)      # ids (int64) + slot / pos / segment (int32)
                batch = make_batch(segs, self.device)
                self.stats["h2d_bytes"] += 8 * batch.T + 16 * batch.T
                h = self.ex.forward(batch)
                if self.mtp is not None:
                    self.mtp.after_prefill(batch, h)
                row = 0
                last_rows = []
                for rs, a, b in owners:
                    row += b - a
                    if b >= rs.prompt_len:
                        last_rows.append((rs, row - 1))
                    if interval and b % interval == 0 and b < rs.prompt_len:
                        self._snapshot(rs, b)
                if last_rows:
                    idx = torch.tensor([i for _, i in last_rows], device=self.device)
                    logits = self.ex.logits(h.index_select(0, idx))
                    toks = self._sample_rows([rs for rs, _ in last_rows], logits)
                    for (rs, _), t in zip(last_rows, toks):
                        out[rs.rid] = t
        except torch.cuda.OutOfMemoryError as exc:
            raise ExecutionFailure([rs.rid for rs, _ in work], "prefill", f"out of memory: {exc}", "partial") from exc
        self.resident_key = ()
        return out

    def _snapshot(self, rs: RequestState, n_tokens: int) -> None:
        """Copy the slot's recurrent state into a snapshot slot and publish the prefix [0, n_tokens)."""
        sid = self._alloc_snapshot()
        if sid is None:
            return
        self._copy_state(rs.slot, sid)
        lease: KVLease = rs.runner_data
        self.radix.insert(rs.req.prompt_token_ids[:n_tokens], lease.pages[:n_tokens // self.page], {n_tokens: sid})
        self.stats["snapshots_taken"] += 1

    # ------------------------------------------------------------------ device status
    def _sync_checked(self, phase: str) -> None:
        """The per-step stream synchronise, with the kernels' status word read back in the same breath.

        A kernel whose bounded wait gave up (an mbarrier, or a peer rank's flag in the tensor-parallel collectives)
        skips its update and records a code; tokens computed after that are wrong and, with several ranks, the
        replicas no longer agree.  That is not containable per request: raise, so that the engine service records
        itself unhealthy and fails what is in flight."""
        self.pinned_status.copy_(self.status_word, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.stats["d2h_bytes"] += 16
        code = int(self.pinned_status[0])
        if code != 0:
            self.status_word.zero_()
            raise K.DeviceStatusError(f"{phase}: a kernel reported status {code} (a bounded wait gave up); "
                                      "device state is incomplete")

    # ------------------------------------------------------------------ sampling
    def _sample_rows(self, rows: List[RequestState], logits: torch.Tensor) -> List[Tuple[int, Optional[TokenLogprob]]]:
        """logits: fp32 [R, V] on the device.  Plain rows use the device sampler; processed rows the host law."""
        R = len(rows)
        res: List[Optional[Tuple[int, Optional[TokenLogprob]]]] = [None] * R
        plain = [i for i, rs in enumerate(rows) if not rs.forced and not self._needs_processing(rs)]
        if plain:
            params = K.pack_sample_params([(rows[i].req.temperature, rows[i].req.top_k, rows[i].req.top_p,
                                            rows[i].req.min_p, rows[i].seed, rows[i].sample_counter) for i in plain],
                                          self.device)
            sub = logits if len(plain) == R else logits.index_select(0, torch.tensor(plain, device=self.device))
            ids = torch.empty(len(plain), dtype=torch.int64, device=self.device)
            K.sample_rows(sub, params, ids)
            host = self.pinned_ids[:len(plain)]
            host.copy_(ids, non_blocking=True)
            self._sync_checked("sample")
            self.stats["d2h_bytes"] += 8 * len(plain)
            toks = host.tolist()
            for i in plain:
                rows[i].telemetry.d2h_bytes += 8
            for j, i in enumerate(plain):
                lp = None
                if rows[i].req.logprobs:
                    lp = self._device_logprobs(rows[i], sub[j:j + 1], toks[j])
                res[i] = (int(toks[j]), lp)
        for i, rs in enumerate(rows):
            if res[i] is None:
                res[i] = self.sample_host(rs, logits[i])
                self.stats["d2h_bytes"] += 4 * self.vocab
                rs.telemetry.d2h_bytes += 4 * self.vocab
        return res  # type: ignore

    def _device_logprobs(self, rs: RequestState, row: torch.Tensor, tok: int) -> TokenLogprob:
        t = rs.req.temperature if rs.req.temperature > 0 else 1.0
        chosen = torch.tensor([tok], dtype=torch.int64, device=self.device)
        ids, lps, clp = K.topn_logprobs(row, rs.req.top_logprobs, t, chosen)
        top = tuple((int(a), float(b)) for a, b in zip(ids[0].tolist(), lps[0].tolist()))
        return TokenLogprob(tok, float(clp[0].item()), top)

    # ------------------------------------------------------------------ decode
    def decode(self, rows: List[RequestState]) -> List[Tuple[int, Optional[TokenLogprob]]]:
        with self.census.region("decode"):
            return self._decode_impl(rows)

    @torch.no_grad()
    def _decode_impl(self, rows: List[RequestState]) -> List[Tuple[int, Optional[TokenLogprob]]]:
        R = len(rows)
        key = tuple(rs.rid for rs in rows)
        for rs in rows:
            self._ensure_pages(rs, rs.position)
        if key != self.resident_key:
            # the resident set changed (admission, finish, or a prefill ran): reinstall rows on the device
            self.graphs.set_rows([rs.slot for rs in rows], [rs.last_token for rs in rows],
                                 [rs.position - 1 for rs in rows])
            self.stats["h2d_bytes"] += 24 * R
            for rs in rows:
                rs.telemetry.h2d_bytes += 24
            self.resident_key = key
        max_ctx = max(rs.position for rs in rows)
        all_greedy = all(rs.req.temperature == 0.0 and not rs.forced and not self._needs_processing(rs)
                         and not rs.req.logprobs for rs in rows)
        if all_greedy:
            self.graphs.step(R, max_ctx, greedy=True)
            host = self.pinned_ids[:R]
            host.copy_(self.graphs.next_ids[:R], non_blocking=True)
            self._sync_checked("decode")
            self.stats["d2h_bytes"] += 8 * R
            for rs in rows:
                rs.telemetry.d2h_bytes += 8
            return [(int(t), None) for t in host.tolist()]
        self.graphs.step(R, max_ctx, greedy=False)
        res = self._sample_rows(rows, self.graphs.logits[:R])
        self.graphs.next_ids[:R].copy_(torch.tensor([t for t, _ in res], dtype=torch.int64), non_blocking=True)
        self.graphs.publish(R)
        self.stats["h2d_bytes"] += 8 * R
        return res

    # ------------------------------------------------------------------ speculative decoding (MTP)
    def speculative_eligible(self, rs: RequestState) -> bool:
        from ..speculative.serving import resolve_mtp_serving_plan
        d = resolve_mtp_serving_plan(self.config.speculative.mode and "on", self.supports_mtp, rs.req.temperature,
                                     self._needs_processing(rs), bool(rs.forced), bool(rs.req.logprobs),
                                     depth=self.config.speculative.draft_depth,
                                     requested=True)
        return d.use_mtp

    def speculative_cycle(self, rows: List[RequestState]):
        with self.census.region("speculative_cycle"):
            return self._speculative_cycle_impl(rows)

    @torch.no_grad()
    def _speculative_cycle_impl(self, rows: List[RequestState]):
        from ..speculative.contracts import SpecCycleResult
        from ..speculative.policy import plan_draft_depth
        if len(rows) > self.mtp.max_requests:
            return [SpecCycleResult([t], 0, 0) for t, _ in self.decode(rows)]
        depth = self.mtp.max_depth
        for rs in rows:
            remaining = rs.remaining()
            room = rs.total_budget_tokens - rs.position
            depth = min(depth, plan_draft_depth(self.mtp.max_depth, remaining, room, rs.telemetry.speculative_drafted,
                                                rs.telemetry.speculative_accepted,
                                                adaptive=self.config.speculative.adaptive_depth))
        if depth < 1:
            return [SpecCycleResult([t], 0, 0) for t, _ in self.decode(rows)]
        for rs in rows:
            self._ensure_pages(rs, rs.position + depth)
        kw = {}
        if self.spec_uses_history:
            kw["histories"] = [list(rs.req.prompt_token_ids) + rs.generated for rs in rows]
        if self.draft_vocab is not None:
            kw["small_head"] = self.draft_vocab.decide(
                [self.draft_vocab.fits(rs.rid, rs.req.prompt_token_ids, rs.generated, rs.last_token) for rs in rows])
        try:
            got = self.mtp.cycle([rs.slot for rs in rows], [rs.last_token for rs in rows],
                                 [rs.position - 1 for rs in rows], depth,
                                 [rs.req.temperature for rs in rows], [rs.seed for rs in rows],
                                 [rs.sample_counter for rs in rows], **kw)
        except torch.cuda.OutOfMemoryError as exc:
            raise ExecutionFailure([rs.rid for rs in rows], "verify", f"out of memory: {exc}", "partial") from exc
        if got is None:                 # the drafter had nothing to propose: plain decode step
            return [SpecCycleResult([t], 0, 0) for t, _ in self.decode(rows)]
        res, _txn = got
        if self.spec_uses_history:
            depth = res[0].drafted
            for rs, c in zip(rows, res):
                self.mtp.drafter.observe(list(rs.req.prompt_token_ids) + rs.generated + list(c.tokens))
        for rs, c in zip(rows, res):
            # KV rollback: the cycle reserved pages for every draft; keep those of the accepted prefix (+ the next
            # token) and hand the rest back to the request's credit
            lease = rs.runner_data
            if lease is not None:
                self.pool.truncate_pages(lease, rs.position + c.accepted + 1)
            rs.sample_counter += 2 * (depth + 1)
            rs.telemetry.d2h_bytes += 8 * (depth + 2)
            rs.telemetry.h2d_bytes += 24 * (depth + 1)
        self.stats["d2h_bytes"] += 8 * (depth + 2) * len(rows)
        self.resident_key = ()          # the decode graph's resident rows no longer match the cursors
        return res

    # ------------------------------------------------------------------ release / lifecycle
    def release(self, rs: RequestState) -> None:
        lease: Optional[KVLease] = rs.runner_data
        if lease is not None:
            if self.use_prefix and not self.cfg.is_hybrid and rs.prefilled >= self.page:
                n = (min(rs.prefilled, rs.prompt_len) // self.page) * self.page
                self.radix.insert(rs.req.prompt_token_ids[:n], lease.pages[:n // self.page])
            self.pool.release(rs.rid)
            rs.runner_data = None
        if rs.slot is not None and rs.slot not in self.free_slots and rs.slot < self.max_slots:
            self.free_slots.append(rs.slot)
        claim = self._claims.pop(str(rs.rid), None)
        if claim is not None:
            self.ledger.release(claim)
        if self.draft_vocab is not None:
            self.draft_vocab.drop(rs.rid)
        if rs.rid in self.resident_key:
            self.resident_key = ()

    def close(self) -> None:
        """Drop the captured decode graphs: in a multi-rank job they hold library collectives, which must be gone
        before the process group is destroyed."""
        self.graphs.graphs.clear()
        self.graphs._execs.clear()

    def reset(self) -> None:
        for rid in list(self.pool.leases):
            self.pool.release(rid)
        self.radix.clear()
        self.free_slots = list(range(self.max_slots - 1, -1, -1))
        self.free_snaps = list(range(self.max_slots + self.n_snap - 1, self.max_slots - 1, -1))
        for claim in self._claims.values():
            self.ledger.release(claim)
        self._claims.clear()
        for claim in self._snap_claims.values():
            self.ledger.release(claim)
        self._snap_claims.clear()
        if self.draft_vocab is not None:
            self.draft_vocab.clear()
        self.resident_key = ()

    def capacity(self) -> Dict[str, Any]:
        return {"backend": "cuda_sm100a", "max_slots": self.max_slots, "max_context": self.max_context,
                "free_slots": len(self.free_slots), "kv_pool": self.pool.snapshot(),
                "resources": self.ledger.snapshot(),
                "speculative": self.mtp.capability().as_dict() if self.mtp is not None else None,
                "prefix_cache": self.radix.snapshot_stats(), "state_bytes": self.ex.state_bytes(),
                "kv_bytes_per_token": self.cfg.kv_bytes_per_token(),
                "recurrent_state_bytes_per_request": self.cfg.recurrent_state_bytes(),
                # resident weight bytes: the quantised device layouts (there is no widened copy of any of them)
                "weight_bytes": sum(w.data.numel() * w.data.element_size() for w in
                                    {id(w): w for w in self.ex.dw.values()}.values())}

    def snapshot(self) -> Dict[str, Any]:
        return {"launch_census": self.census.report(), "pool": self.pool.snapshot(), "prefix": self.radix.snapshot_stats(), "graphs": dict(self.graphs.stats, kernels_per_graph=None),
                "draft_vocab": self.draft_vocab.as_dict() if self.draft_vocab is not None else None,
                **self.stats}
