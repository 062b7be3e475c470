"""NextN / MTP chain speculation on the GPU executor: draft K tokens with the checkpoint's trailing NextN block,
verify the chain with one target forward, accept on the device, commit by journal copy.

Cycle for a request whose last committed token ``t0`` sits at position ``p`` (not yet fed to the target):
  draft   d1 = argmax NextN(t0, h[p-1]) ... dK, each step feeding the block's own hidden forward;
  verify  target forward over rows [t0, d1 .. dK] at positions p .. p+K; linear-attention layers journal their
          conv / delta-net state after every row instead of updating the live state;
  accept  greedy: longest prefix with d_{i+1} == argmax(row i); sampled: exact min(1, p/q) rule (``csrc/spec.cu``);
  commit  live recurrent state <- journal row n, cursors += n + 1, h[p+n] kept for the next cycle.  KV rows past
          the accepted prefix are simply overwritten by the next cycle (positions rewind, pages stay).
Stages are recorded through ``SpecTransaction``.  Reference flow: ``hipengine/runtime/qwen35_gguf_mtp.py``
(transactional proposal + verify) and ``hipengine/speculative/gguf_mtp.py`` (seed rows, draft proposals).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..models.executor import GEMV_MAX_ROWS, BatchDesc, make_batch
from ..ops import kernels as K
from .contracts import SpecCycleResult, SpeculativeCapability
from .transaction import SpecTransaction, Stage


class ChainVerifyCycle:
    """Verify / accept / commit for chains of drafted tokens, whatever proposed them (the NextN block below, or a
    host-side drafter such as prompt lookup, ``speculative/providers.py``).  Holds the journal and the small device
    buffers of the accept and commit kernels."""

    def __init__(self, ex, max_depth: int = 3, max_requests: int = 8):
        self.ex = ex
        self.max_depth = max_depth
        self.max_requests = max_requests
        dev = ex.device
        self.max_rows = max_requests * (max_depth + 1)
        self.journal = None                       # allocated on first use (large)
        self.n_accept = torch.zeros(max_requests, dtype=torch.int32, device=dev)
        self.commit_row = torch.zeros(max_requests, dtype=torch.int32, device=dev)
        self.hidden_row = torch.zeros(max_requests, dtype=torch.int32, device=dev)
        self.am_ids = torch.zeros(self.max_rows, dtype=torch.int64, device=dev)
        self.stats = {"cycles": 0, "drafted": 0, "accepted": 0}

    def capability(self) -> SpeculativeCapability:
        return SpeculativeCapability(provider="host_drafts", max_depth=self.max_depth,
                                     widths=tuple(range(1, self.max_requests + 1)), attachment="none")

    # hooks of drafters that keep device state per slot (the NextN block does)
    def reset_slot(self, slot: int) -> None:
        pass

    def after_prefill(self, batch: BatchDesc, h: torch.Tensor) -> None:
        pass

    def _after_commit(self, slot_t: torch.Tensor, hid: torch.Tensor, R: int, raw: Optional[torch.Tensor] = None) -> None:
        """``hid``: post-norm hidden rows of the verify forward, ``raw``: its residual rows before the output norm;
        ``self.hidden_row[:R]`` indexes the row whose logits produced each request's last emitted token."""

    def _verify_accept_commit(self, txn: SpecTransaction, slots, positions, t0: torch.Tensor, drafts: torch.Tensor,
                              temperature, seeds, counters) -> List[SpecCycleResult]:
        """Target forward over R chains [t0, d1..dK] with journalled recurrent state, device accept, one host
        read-back, commit by journal copy.  ``txn`` must be in stage DRAFTED."""
        ex, cfg, dev = self.ex, self.ex.cfg, self.ex.device
        R, Kd = drafts.shape
        if self.journal is None:
            self.journal = ex.alloc_journal(self.max_rows)
        sampled = temperature is not None and any(t > 0 for t in temperature)
        slot_t = torch.tensor(list(slots), dtype=torch.int64, device=dev)
        T = R * (Kd + 1)
        vb = make_batch([(s, p, [0] * (Kd + 1)) for s, p in zip(slots, positions)], dev)
        vb.tokens = torch.cat([t0[:, None], drafts], 1).reshape(-1).contiguous()
        journal = {"conv": {i: t[:T] for i, t in self.journal["conv"].items()},
                   "gdn": {i: t[:T] for i, t in self.journal["gdn"].items()}}
        # a verify chain must see the numerics of plain decode (the int8 GEMV path), or a near-tie could make the
        # verifier disagree with what autoregressive decoding would have produced: keep chains of up to 8 rows there
        saved_small = ex.small_rows
        if T <= GEMV_MAX_ROWS:
            ex.small_rows = GEMV_MAX_ROWS
        try:
            h = ex.forward(vb, journal=journal)
        finally:
            ex.small_rows = saved_small
        logits = ex.scratch.get("mtp_logits", (T, cfg.vocab), torch.float32)
        hid = ex.scratch.get("mtp_vhid", (T, cfg.hidden), torch.float32)
        for r0 in range(0, T, GEMV_MAX_ROWS):
            r1 = min(T, r0 + GEMV_MAX_ROWS)
            ex.logits(h[r0:r1], out=logits[r0:r1], hidden_out=hid[r0:r1])
        txn.advance(Stage.VERIFIED)
        # ---- accept
        out = torch.empty(R, Kd + 1, dtype=torch.int64, device=dev)
        if not sampled:
            tgt = self.am_ids[:T]
            for r0 in range(0, T, GEMV_MAX_ROWS):
                r1 = min(T, r0 + GEMV_MAX_ROWS)
                ex.greedy(logits[r0:r1], tgt[r0:r1])
            K.spec_accept_greedy(drafts, tgt.view(R, Kd + 1), self.n_accept[:R], out)
        else:
            temp = torch.tensor([max(float(t), 1e-6) for t in temperature], dtype=torch.float32, device=dev)
            sd = torch.tensor([int(s) & (2 ** 63 - 1) for s in (seeds or [0] * R)], dtype=torch.int64, device=dev)
            ct = torch.tensor([int(c) & (2 ** 63 - 1) for c in (counters or [0] * R)], dtype=torch.int64, device=dev)
            K.spec_accept_sampled(logits.view(R, Kd + 1, cfg.vocab), None, drafts, temp, sd, ct, self.n_accept[:R], out)
        txn.advance(Stage.ACCEPTED)
        # ---- readback (the only host sync of the cycle)
        n_host = self.n_accept[:R].tolist()
        out_host = out.tolist()
        txn.advance(Stage.READBACK)
        # ---- commit: journal row n -> live state, hidden of row n -> next cycle's seed
        txn.advance(Stage.COMMITTING)
        pos_t = torch.tensor(list(positions), dtype=torch.int32, device=dev)
        tok_t = torch.empty(R, dtype=torch.int64, device=dev)
        K.spec_commit(self.n_accept[:R], out, tok_t, pos_t, None, self.commit_row[:R], self.hidden_row[:R])
        ex.commit_journal(journal, vb.seg_slot, self.commit_row[:R])
        self._after_commit(slot_t, hid, R, raw=h)
        txn.advance(Stage.COMMITTED)
        res = []
        for r in range(R):
            n = int(n_host[r])
            res.append(SpecCycleResult([int(x) for x in out_host[r][:n + 1]], Kd, n, list(txn.trace)))
            self.stats["drafted"] += Kd
            self.stats["accepted"] += n
        self.stats["cycles"] += 1
        return res

    @torch.no_grad()
    def cycle_with_drafts(self, slots: Sequence[int], last_tokens: Sequence[int], positions: Sequence[int],
                          drafts: Sequence[Sequence[int]], temperature: Optional[Sequence[float]] = None,
                          seeds: Optional[Sequence[int]] = None, counters: Optional[Sequence[int]] = None
                          ) -> Tuple[List[SpecCycleResult], SpecTransaction]:
        """One cycle whose chains come from the host: ``drafts[r]`` are the K tokens proposed after
        ``last_tokens[r]`` (all rows the same K).  A deterministic drafter is a one-hot proposal distribution, so
        the sampled rule accepts token d with probability p(d) and resamples from p with d removed."""
        dev = self.ex.device
        R, Kd = len(slots), len(drafts[0])
        assert 1 <= Kd <= self.max_depth and R <= self.max_requests and all(len(d) == Kd for d in drafts)
        txn = SpecTransaction(list(range(R)))
        txn.advance(Stage.RESERVED)
        txn.advance(Stage.TARGET_OPEN)
        txn.advance(Stage.PROVIDER_OPEN)
        t0 = torch.tensor(list(last_tokens), dtype=torch.int64, device=dev)
        d = torch.tensor([list(x) for x in drafts], dtype=torch.int64, device=dev)
        txn.advance(Stage.DRAFTED)
        return self._verify_accept_commit(txn, slots, positions, t0, d, temperature, seeds, counters), txn


class MTPCycle(ChainVerifyCycle):
    def __init__(self, ex, max_depth: int = 3, max_requests: int = 8, draft_head_rows: int = 0):
        assert ex.has_nextn, "checkpoint has no NextN block"
        super().__init__(ex, max_depth, max_requests)
        self.h_prev = torch.zeros(ex.max_slots, ex.cfg.hidden, dtype=torch.float32, device=ex.device)  # per slot
        # hot-vocabulary draft head: rows of the head slice a cycle may draft with (0: always the full head); the
        # caller says per cycle, with ``small_head=True``, that every row's recent tokens lie inside the slice
        self.draft_head_rows = int(draft_head_rows) if 0 < int(draft_head_rows) < ex.cfg.vocab else 0

    def capability(self) -> SpeculativeCapability:
        return SpeculativeCapability(provider="nextn_mtp", max_depth=self.max_depth,
                                     widths=tuple(range(1, self.max_requests + 1)),
                                     graph_capture=isinstance(self, GraphedMTPCycle),
                                     draft_head_rows=self.draft_head_rows)

    def _after_commit(self, slot_t: torch.Tensor, hid: torch.Tensor, R: int, raw: Optional[torch.Tensor] = None) -> None:
        picked = self.ex.scratch.get("mtp_pick", (R, self.ex.cfg.hidden), torch.float32)
        K.gather_rows_f32(hid, self.hidden_row[:R], picked)
        self.h_prev.index_copy_(0, slot_t, picked)

    # ------------------------------------------------------------------ prompt side
    def reset_slot(self, slot: int) -> None:
        self.h_prev[slot].zero_()

    def after_prefill(self, batch: BatchDesc, h: torch.Tensor) -> None:
        """Feed the prompt rows of ``batch`` through the NextN block so its KV covers the prompt, and keep the
        last post-norm hidden of every segment.  ``h`` is the target's residual output for the batch rows."""
        ex, cfg = self.ex, self.ex.cfg
        T = batch.T
        hid = ex.scratch.get("mtp_hid", (T, cfg.hidden), torch.float32)
        K.rmsnorm_rows(h, ex.f32["output_norm.weight"], hid, cfg.rms_eps)
        hprev = ex.scratch.get("mtp_hprev", (T, cfg.hidden), torch.float32)
        r0 = 0
        for (slot, pos0, n) in batch.segs_host:
            hprev[r0].copy_(self.h_prev[slot])
            if n > 1:
                hprev[r0 + 1:r0 + n].copy_(hid[r0:r0 + n - 1])
            self.h_prev[slot].copy_(hid[r0 + n - 1])
            r0 += n
        ex.nextn_forward(batch, hprev)

    # ------------------------------------------------------------------ one cycle
    @torch.no_grad()
    def cycle(self, slots: Sequence[int], last_tokens: Sequence[int], positions: Sequence[int], depth: int,
              temperature: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
              counters: Optional[Sequence[int]] = None, draft_override: Optional[torch.Tensor] = None,
              small_head: bool = False) -> Tuple[List[SpecCycleResult], SpecTransaction]:
        """positions[r] = position of last_tokens[r].  temperature None/0 -> greedy verification.
        ``draft_override`` (int64 [R, depth]) replaces the NextN proposals after they are computed (the block
        still runs, so its KV stays in step); used to test acceptance paths with known chains.
        ``small_head`` drafts with the first ``draft_head_rows`` rows of the head (verification is unchanged)."""
        ex, cfg, dev = self.ex, self.ex.cfg, self.ex.device
        R, Kd = len(slots), depth
        assert 1 <= Kd <= self.max_depth and R <= self.max_requests
        txn = SpecTransaction(list(range(R)))
        txn.advance(Stage.RESERVED)
        slot_t = torch.tensor(list(slots), dtype=torch.int64, device=dev)
        t0 = torch.tensor(list(last_tokens), dtype=torch.int64, device=dev)
        drafts = torch.empty(R, Kd, dtype=torch.int64, device=dev)
        txn.advance(Stage.TARGET_OPEN)
        # ---- draft: K passes of the NextN block, R rows each
        txn.advance(Stage.PROVIDER_OPEN)
        cur = t0
        hprev = self.h_prev.index_select(0, slot_t)
        hid_next = ex.scratch.get("mtp_hid_next", (R, cfg.hidden), torch.float32)
        ids = self.am_ids[:R]
        for j in range(Kd):
            b = make_batch([(s, p + j, [0]) for s, p in zip(slots, positions)], dev)
            b.tokens = cur
            h = ex.nextn_forward(b, hprev)
            lg = ex.nextn_logits(h, hidden_out=hid_next, head_rows=self.draft_head_rows if small_head else 0)
            for r0 in range(0, R, GEMV_MAX_ROWS):
                r1 = min(R, r0 + GEMV_MAX_ROWS)
                ex.greedy(lg[r0:r1], ids[r0:r1])
            drafts[:, j].copy_(ids)
            cur = drafts[:, j].contiguous()
            hprev = hid_next.clone()
        if draft_override is not None:
            drafts.copy_(draft_override.to(dev))
        txn.advance(Stage.DRAFTED)
        res = self._verify_accept_commit(txn, slots, positions, t0, drafts, temperature, seeds, counters)
        return res, txn


class GraphedMTPCycle(MTPCycle):
    """The greedy NextN cycle -- propose(K) -> verify -> accept -> commit -> cursor update -- captured as ONE CUDA
    graph per (rows, depth, context bucket, draft-head rows) and launched through the native cycle launcher with
    the full stage mask; the only read-back is the accept counts (returned by the launcher) and the emitted ids.

    Everything a cycle reads is resident on the device and advanced by the graph itself: slots, the last committed
    token and its position per row, the per-slot hidden seed of the NextN block.  A following cycle over the same
    rows needs no host -> device copy at all; rows are (re)installed only when the host's view of (slot, token,
    position) differs from what the previous cycle left (admission, a finished row, a plain decode step between).
    Sampled verification, override drafts and chains of more than 8 verify rows take the eager path of the parent.
    Reference: ``hipengine/speculative/native_cycle_graph.cpp:1-300`` (one native call per cycle over a captured
    graph, stage mask PROPOSE | VERIFY | ACCEPT | COMMIT | UPDATE_CURSORS).
    """

    def __init__(self, ex, max_depth: int = 3, max_requests: int = 8, draft_head_rows: int = 0):
        super().__init__(ex, max_depth, max_requests, draft_head_rows)
        dev, cfg = ex.device, ex.cfg
        R, Kd = max_requests, max_depth
        T = self.max_rows
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        i64 = lambda *s: torch.zeros(*s, dtype=torch.int64, device=dev)
        self.slot, self.slot64, self.tok, self.pos = i32(R), i64(R), i64(R), i32(R)
        self.dpos, self.dctx, self.dcur = i32(Kd, R), i32(Kd, R), i64(Kd, R)
        self.drafts, self.out = i64(R, Kd), i64(R, Kd + 1)
        self.vtok, self.vslot, self.vpos, self.vctx = i64(T), i32(T), i32(T), i32(T)
        self.hp = torch.zeros(R, cfg.hidden, dtype=torch.float32, device=dev)
        self.hid_next = torch.zeros(Kd, R, cfg.hidden, dtype=torch.float32, device=dev)
        self.vlogits = torch.empty(GEMV_MAX_ROWS, cfg.vocab, dtype=torch.float32, device=dev)
        self.vhid = torch.empty(GEMV_MAX_ROWS, cfg.hidden, dtype=torch.float32, device=dev)
        self.picked = torch.empty(R, cfg.hidden, dtype=torch.float32, device=dev)
        self.seg_r = torch.arange(R + 1, dtype=torch.int32, device=dev)
        self.graphs = {}
        self._consts = {}
        self._mirror = None                     # host view of (slots, tokens, positions) the device rows hold
        self.graph_stats = {"captures": 0, "replays": 0, "installs": 0, "eager": 0, "kernels_per_graph": {}}

    # ------------------------------------------------------------------ resident rows
    def _install(self, slots, tokens, positions) -> None:
        n = len(slots)
        self.slot[:n].copy_(torch.tensor(slots, dtype=torch.int32), non_blocking=True)
        self.slot64[:n].copy_(torch.tensor(slots, dtype=torch.int64), non_blocking=True)
        self.tok[:n].copy_(torch.tensor(tokens, dtype=torch.int64), non_blocking=True)
        self.pos[:n].copy_(torch.tensor(positions, dtype=torch.int32), non_blocking=True)
        self.graph_stats["installs"] += 1

    def _const(self, R: int, Kd: int):
        key = (R, Kd)
        c = self._consts.get(key)
        if c is None:
            dev = self.ex.device
            T = R * (Kd + 1)
            c = {"seg_start": torch.arange(R + 1, dtype=torch.int32, device=dev) * (Kd + 1),
                 "tok_seg": torch.arange(T, dtype=torch.int32, device=dev) // (Kd + 1),
                 "off": torch.arange(Kd + 1, dtype=torch.int32, device=dev)[None, :]}
            if Kd != self.max_depth:            # contiguous [R, Kd] / [R, Kd + 1] buffers of their own
                c["drafts_k"] = torch.zeros(R, Kd, dtype=torch.int64, device=dev)
                c["out_k"] = torch.zeros(R, Kd + 1, dtype=torch.int64, device=dev)
            self._consts[key] = c
        return c

    # ------------------------------------------------------------------ the cycle body (graph-safe: no host reads)
    def _body(self, R: int, Kd: int, max_ctx: int, head_rows: int = 0) -> None:
        ex = self.ex
        c = self._const(R, Kd)
        T = R * (Kd + 1)
        slot, tok, pos = self.slot[:R], self.tok[:R], self.pos[:R]
        # ---- propose: K passes of the NextN block
        torch.index_select(self.h_prev, 0, self.slot64[:R], out=self.hp[:R])
        cur, hp = tok, self.hp[:R]
        for j in range(Kd):
            torch.add(pos, j, out=self.dpos[j, :R])
            torch.add(pos, j + 1, out=self.dctx[j, :R])
            b = BatchDesc(cur, slot, self.dpos[j, :R], self.dctx[j, :R], self.seg_r[:R + 1], slot, self.seg_r[:R],
                          R, R, max_ctx)
            h = ex.nextn_forward(b, hp)
            lg = ex.nextn_logits(h, hidden_out=self.hid_next[j, :R], head_rows=head_rows)
            ex.greedy(lg[:R], self.dcur[j, :R])
            self.drafts[:R, j].copy_(self.dcur[j, :R])
            cur, hp = self.dcur[j, :R], self.hid_next[j, :R]
        # ---- verify: target forward over [t0, d1 .. dK] per row, recurrent state journalled per verify row
        vt = self.vtok[:T].view(R, Kd + 1)
        vt[:, 0].copy_(tok)
        vt[:, 1:].copy_(self.drafts[:R, :Kd])
        self.vslot[:T].view(R, Kd + 1).copy_(slot[:, None].expand(R, Kd + 1))
        torch.add(pos[:, None], c["off"], out=self.vpos[:T].view(R, Kd + 1))
        torch.add(self.vpos[:T], 1, out=self.vctx[:T])
        vb = BatchDesc(self.vtok[:T], self.vslot[:T], self.vpos[:T], self.vctx[:T], c["seg_start"], slot,
                       c["tok_seg"], T, R, max_ctx)
        journal = {"conv": {i: t[:T] for i, t in self.journal["conv"].items()},
                   "gdn": {i: t[:T] for i, t in self.journal["gdn"].items()}}
        h = ex.forward(vb, journal=journal)
        ex.logits(h, out=self.vlogits[:T], hidden_out=self.vhid[:T])
        # ---- accept + commit + cursors
        tgt = self.am_ids[:T]
        ex.greedy(self.vlogits[:T], tgt)
        K.spec_accept_greedy(self.drafts[:R, :Kd] if Kd == self.max_depth else self._drafts_k(R, Kd),
                             tgt.view(R, Kd + 1), self.n_accept[:R], self._out_k(R, Kd))
        K.spec_commit(self.n_accept[:R], self._out_k(R, Kd), tok, pos, None, self.commit_row[:R],
                      self.hidden_row[:R])
        ex.commit_journal(journal, slot, self.commit_row[:R])
        K.gather_rows_f32(self.vhid[:T], self.hidden_row[:R], self.picked[:R])
        self.h_prev.index_copy_(0, self.slot64[:R], self.picked[:R])

    def _drafts_k(self, R: int, Kd: int) -> torch.Tensor:
        """Contiguous [R, Kd] view of the drafts for a depth below the maximum (own buffer per depth)."""
        buf = self._const(R, Kd)["drafts_k"]
        buf.copy_(self.drafts[:R, :Kd])
        return buf

    def _out_k(self, R: int, Kd: int) -> torch.Tensor:
        if Kd == self.max_depth:
            return self.out[:R]
        return self._const(R, Kd)["out_k"]

    def _snapshot(self, R: int):
        ex = self.ex
        sl = self.slot64[:R]
        return {"tok": self.tok.clone(), "pos": self.pos.clone(), "hprev": self.h_prev[sl].clone(), "sl": sl,
                "conv": {i: t[sl].clone() for i, t in ex.conv_state.items()},
                "gdn": {i: t[sl].clone() for i, t in ex.gdn_state.items()}}

    def _restore(self, s) -> None:
        ex = self.ex
        self.tok.copy_(s["tok"])
        self.pos.copy_(s["pos"])
        self.h_prev[s["sl"]] = s["hprev"]
        for i, t in ex.conv_state.items():
            t[s["sl"]] = s["conv"][i]
        for i, t in ex.gdn_state.items():
            t[s["sl"]] = s["gdn"][i]

    # ------------------------------------------------------------------ one cycle
    @torch.no_grad()
    def cycle(self, slots, last_tokens, positions, depth, temperature=None, seeds=None, counters=None,
              draft_override=None, small_head=False):
        from ..core import runtime as RT
        from ..models.decode_graph import ctx_bucket
        ex = self.ex
        R, Kd = len(slots), depth
        sampled = temperature is not None and any(t > 0 for t in temperature)
        if (sampled or draft_override is not None or R * (Kd + 1) > GEMV_MAX_ROWS or R > self.max_requests
                or not 1 <= Kd <= self.max_depth):
            self.graph_stats["eager"] += 1
            self._mirror = None
            return super().cycle(slots, last_tokens, positions, depth, temperature, seeds, counters, draft_override,
                                 small_head)
        if self.journal is None:
            self.journal = ex.alloc_journal(self.max_rows)
        want = (tuple(slots), tuple(int(t) for t in last_tokens), tuple(int(p) for p in positions))
        if want != self._mirror:
            self._install(*want)
        txn = SpecTransaction(list(range(R)))
        for st in (Stage.RESERVED, Stage.TARGET_OPEN, Stage.PROVIDER_OPEN):
            txn.advance(st)
        head_rows = self.draft_head_rows if small_head else 0
        key = (R, Kd, ctx_bucket(max(positions) + Kd + 1), head_rows)
        saved_small = ex.small_rows
        ex.small_rows = GEMV_MAX_ROWS           # verify rows see the numerics of plain decode (see the parent)
        try:
            g = self.graphs.get(key)
            if g is None:
                snap = self._snapshot(R)
                self._body(R, Kd, key[2], head_rows)   # warm-up: scratch growth and function attributes settle
                torch.cuda.synchronize()
                self._restore(snap)
                k0 = K.launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._body(R, Kd, key[2], head_rows)
                self.graph_stats["kernels_per_graph"][key] = K.launch_count() - k0
                self._restore(snap)
                self.graphs[key] = g
                self.graph_stats["captures"] += 1
        finally:
            ex.small_rows = saved_small
        exec_h = RT.graph_exec_handle(g)
        n_host = None
        if exec_h:
            ctl = RT.make_control(RT.STAGES_FULL_CYCLE, R, Kd, wait=True,
                                  status_word=K.status_tensor(ex.device).data_ptr(),
                                  n_accept=self.n_accept.data_ptr())
            res = RT.cycle_launch(ctl, exec_h, torch.cuda.current_stream().cuda_stream)
            if res.rc != 0:
                raise RuntimeError(f"native cycle launch failed: rc={res.rc}")
            if res.device_status != 0:
                raise K.DeviceStatusError(f"device status {res.device_status} after a speculative cycle")
            n_host = [int(res.n_accept[r]) for r in range(R)]
        else:
            g.replay()
        K.add_launches(self.graph_stats["kernels_per_graph"][key])
        self.graph_stats["replays"] += 1
        for st in (Stage.DRAFTED, Stage.VERIFIED, Stage.ACCEPTED):
            txn.advance(st)
        out_host = self._out_k(R, Kd).tolist()          # the emitted ids: the cycle's one read-back besides counts
        if n_host is None:
            n_host = self.n_accept[:R].tolist()
        txn.advance(Stage.READBACK)
        txn.advance(Stage.COMMITTING)
        txn.advance(Stage.COMMITTED)
        res_l = []
        new_tok, new_pos = [], []
        for r in range(R):
            n = int(n_host[r])
            res_l.append(SpecCycleResult([int(x) for x in out_host[r][:n + 1]], Kd, n, list(txn.trace)))
            new_tok.append(int(out_host[r][n]))
            new_pos.append(int(positions[r]) + n + 1)
            self.stats["drafted"] += Kd
            self.stats["accepted"] += n
        self.stats["cycles"] += 1
        self._mirror = (tuple(slots), tuple(new_tok), tuple(new_pos))
        return res_l, txn

    def reset_slot(self, slot: int) -> None:
        super().reset_slot(slot)
        self._mirror = None

    def after_prefill(self, batch, h) -> None:
        super().after_prefill(batch, h)
        self._mirror = None
