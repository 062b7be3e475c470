"""The resident engine loop: one tick = lifetime probes -> admission -> (prefill | decode) -> commit.

Mirrors ``ResidentEngineLoop`` (``hipengine/generation/engine_loop.py:2318-4041``): policies ``protect_decode``
(default), ``protect_ttft``, ``fair`` and ``token_budget`` (``:68``); chunked prefill; failure containment
(``contain_execution_failure`` ``:2869-2987``: a runner may fail only the affected rows, anything else is
fatal); cooperative cancellation and deadlines probed before admission and after every step (``:2629-2708``).
The loop is single-threaded and owns the runner; ``EngineService`` drives it from its driver thread.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..config import EngineConfig
from .runner import BaseRunner, ExecutionFailure
from .scheduler import DECODE, FINISHED, PREFILL, GenerationAdmissionRejected, RequestState, Scheduler
from .types import FinishDetails, GenerationRequest, TokenLogprob

POLICIES = ("protect_decode", "protect_ttft", "fair", "token_budget")


class EngineLoop:
    def __init__(self, runner: BaseRunner, config: EngineConfig, tokenizer=None):
        if config.scheduler.policy not in POLICIES:
            raise ValueError(f"unknown scheduling policy {config.scheduler.policy!r}; expected one of {POLICIES}")
        self.runner = runner
        self.config = config
        sc = config.scheduler
        dec = tokenizer.decode if tokenizer is not None else None
        enc = tokenizer.encode if tokenizer is not None else None
        self.sched = Scheduler(min(sc.max_active_requests, runner.max_slots), sc.max_pending_requests,
                               runner.eos_token_id, dec, enc)
        self.sched.tokenizer = tokenizer
        self.on_event: Callable[[RequestState], None] = lambda rs: None
        self._fair_toggle = False
        self.ticks = 0
        self.recent_prefill: List[Dict[str, Any]] = []
        # ranks of a parallel group take cancel / deadline decisions from rank 0 (see parallel/serving.py)
        self.external_lifetimes = False

    # ------------------------------------------------------------------ front door
    def submit(self, req: GenerationRequest) -> RequestState:
        if len(req.prompt_token_ids) + req.max_tokens > self.runner.max_context:
            raise GenerationAdmissionRejected(
                f"context_overflow: prompt {len(req.prompt_token_ids)} + max_tokens {req.max_tokens} "
                f"exceeds max context {self.runner.max_context}")
        return self.sched.submit(req)

    def cancel(self, rid: int, reason: str = "cancelled") -> bool:
        rs = self.sched.cancel(rid, reason)
        if rs is None:
            return False
        self._release(rs)
        self.on_event(rs)
        return True

    def idle(self) -> bool:
        return not self.sched.pending and not self.sched.active

    # ------------------------------------------------------------------ tick
    def tick(self) -> int:
        """One scheduling round.  Returns the number of tokens (prompt + generated) processed."""
        self.ticks += 1
        if not self.external_lifetimes:
            self._probe_lifetimes()
        self.sched.admit_pending(self.runner.admit)
        for rs in self.sched.drain_rejected():
            self.on_event(rs)
        sc = self.config.scheduler
        has_prefill = bool(self.sched.prefill_rows())
        has_decode = bool(self.sched.decode_rows())
        done = 0
        if sc.policy == "token_budget":
            if has_decode:
                done += self._run_decode()
            if has_prefill:
                done += self._run_prefill(sc.round_prefill_token_budget)
        elif sc.policy == "protect_ttft":
            if has_prefill:
                done += self._run_prefill(sc.round_prefill_token_budget)
            elif has_decode:
                done += self._run_decode()
        elif sc.policy == "fair":
            self._fair_toggle = not self._fair_toggle
            if has_prefill and (self._fair_toggle or not has_decode):
                done += self._run_prefill(sc.max_prefill_chunk_tokens * sc.fair_prefill_burst_chunks, round_robin=True)
            elif has_decode:
                done += self._run_decode()
        else:  # protect_decode: resident rows never wait behind more than one prefill chunk
            if has_decode:
                done += self._run_decode()
            if has_prefill:
                done += self._run_prefill(sc.max_prefill_chunk_tokens)
        return done

    # ------------------------------------------------------------------ phases
    def expired(self) -> List[Tuple[int, str]]:
        """(request id, reason) of every request whose cancellation token fired or whose deadline passed: what
        ``_probe_lifetimes`` would cancel.  The leader of a parallel group turns these into broadcast commands."""
        now = time.time()
        out: List[Tuple[int, str]] = []
        for rs in list(self.sched.active.values()) + list(self.sched.pending):
            tok = rs.req.cancellation_token
            if tok is not None and getattr(tok, "cancelled", False):
                out.append((rs.rid, "cancelled"))
            elif rs.req.deadline_at is not None and now >= rs.req.deadline_at:
                out.append((rs.rid, "deadline_exceeded"))
        return out

    def _probe_lifetimes(self) -> None:
        now = time.time()
        for rs in list(self.sched.active.values()) + list(self.sched.pending):
            tok = rs.req.cancellation_token
            if tok is not None and getattr(tok, "cancelled", False):
                self.cancel(rs.rid, "cancelled")
            elif rs.req.deadline_at is not None and now >= rs.req.deadline_at:
                self.cancel(rs.rid, "deadline_exceeded")

    def _run_prefill(self, budget: int, round_robin: bool = False) -> int:
        sc = self.config.scheduler
        work = self.sched.next_prefill_work(sc.max_prefill_chunk_tokens, budget, round_robin)
        if not work:
            return 0
        t0 = time.perf_counter()
        try:
            firsts = self.runner.prefill(work)
        except ExecutionFailure as f:
            self._contain(f)
            return 0
        n = 0
        for rs, cnt in work:
            if rs.status == FINISHED:
                continue
            self.sched.record_prefill(rs, cnt)
            n += cnt
            if rs.rid in firsts:
                tok, lp = firsts[rs.rid]
                self._commit_token(rs, tok, lp)
        self.recent_prefill.append({"tokens": n, "rows": len(work), "seconds": time.perf_counter() - t0})
        self.recent_prefill = self.recent_prefill[-16:]
        return n

    def _run_decode(self) -> int:
        rows = self.sched.next_decode_work(self.config.scheduler.round_decode_row_budget)
        if not rows:
            return 0
        if (self.config.speculative.mode not in ("off", "", None) and self.runner.supports_mtp
                and hasattr(self.runner, "speculative_cycle")):
            spec_rows = [rs for rs in rows if self.runner.speculative_eligible(rs)]
            if spec_rows and len(spec_rows) == len(rows):
                return self._run_speculative(rows)
        try:
            res = self.runner.decode(rows)
        except ExecutionFailure as f:
            self._contain(f)
            return 0
        self.sched.counters["decode_steps"] += 1
        for rs, (tok, lp) in zip(rows, res):
            if rs.status != FINISHED:
                self._commit_token(rs, tok, lp)
        return len(rows)

    def _run_speculative(self, rows: List[RequestState]) -> int:
        try:
            results = self.runner.speculative_cycle(rows)
        except ExecutionFailure as f:
            self._contain(f)
            return 0
        n = 0
        for rs, cyc in zip(rows, results):
            self.sched.counters["spec_cycles"] += 1
            self.sched.counters["spec_drafted"] += cyc.drafted
            self.sched.counters["spec_accepted"] += cyc.accepted
            rs.telemetry.speculative_cycles += 1
            rs.telemetry.speculative_drafted += cyc.drafted
            rs.telemetry.speculative_accepted += cyc.accepted
            for tok in cyc.tokens:
                if rs.status == FINISHED:
                    break
                self._commit_token(rs, tok, None)
                n += 1
        return n

    def _commit_token(self, rs: RequestState, tok: int, lp: Optional[TokenLogprob]) -> None:
        finished = self.sched.record_token(rs, tok, lp)
        if finished:
            self._release(rs)
        self.on_event(rs)

    def _release(self, rs: RequestState) -> None:
        try:
            self.runner.release(rs)
        except Exception:
            pass

    def _contain(self, f: ExecutionFailure) -> None:
        """Fail only the rows the runner named; their slots and pages are reclaimed."""
        for rid in f.request_ids:
            rs = self.sched.fail(rid, f"execution_failed[{f.phase}/{f.mutation}]: {f}")
            if rs is not None:
                self._release(rs)
                self.on_event(rs)

    def fail_all(self, message: str) -> None:
        for rs in list(self.sched.active.values()) + list(self.sched.pending):
            r = self.sched.fail(rs.rid, message)
            if r is not None:
                self._release(r)
                self.on_event(r)

    def snapshot(self) -> Dict[str, Any]:
        s = self.sched.snapshot()
        s.update({"ticks": self.ticks, "policy": self.config.scheduler.policy,
                  "recent_prefill": list(self.recent_prefill), "runner": self.runner.snapshot()})
        return s
