"""Deterministic engine simulator and load harness (test substrate; no model, no GPU).

``SimulatedRunner`` implements the runner protocol with a cost model instead of a forward pass: a prefill chunk
costs ``prefill_us_per_token`` per token, a decode step ``decode_us_base + decode_us_per_row * rows``; tokens are a
hash of (prompt, index), so every schedule of the same requests produces the same outputs.  Time is *virtual*
(a counter the harness reads), so a 256-request Poisson scenario runs in milliseconds and yields exact TTFT /
ITL / throughput figures for a given policy.  Mirrors the reference's ``DeterministicEngineSimulator``
(``hipengine/generation/concurrency2_simulator.py:212``) and ``run_load_scenario`` / ``poisson_arrivals``
(``hipengine/generation/load_harness.py:65``).
"""
from __future__ import annotations

import hashlib
import math
import random
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..config import EngineConfig
from ..kvcache.simulated import SimulatedKVBackend
from .runner import BaseRunner, ExecutionFailure
from .scheduler import GenerationAdmissionRejected, RequestState
from .types import GenerationRequest, TokenLogprob


def _tok(prompt: Sequence[int], index: int, vocab: int) -> int:
    h = hashlib.blake2b(repr((tuple(prompt[-8:]), len(prompt), index)).encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") % vocab


class SimulatedRunner(BaseRunner):
    def __init__(self, config: EngineConfig, vocab: int = 1024, kv_capacity_tokens: int = 1 << 20,
                 prefill_us_per_token: float = 90.0, decode_us_base: float = 8000.0, decode_us_per_row: float = 150.0,
                 fail_decode_for: Sequence[int] = (), fail_decode_admission: Sequence[int] = (),
                 eos_token_id: Optional[int] = None, spec_depth: int = 0, spec_accept_rate: float = 0.0,
                 spec_max_requests: int = 8):
        """``fail_decode_for``: request ids whose next decode (or speculative cycle) raises a contained failure;
        ``fail_decode_admission``: the same, naming requests by admission order (0 = first admitted).
        ``spec_depth`` > 0 makes the runner speculative: a cycle drafts ``spec_depth`` tokens, each draft matches the
        true continuation with probability ``spec_accept_rate`` (a deterministic draw per request and position), and
        the accepted prefix plus one token is emitted -- always the tokens plain decoding would have produced, so a
        speculative run must equal a plain one (the reference's ``SpeculativeCycleSimulator`` plays this role)."""
        self.config = config
        self.vocab = vocab
        self.eos_token_id = eos_token_id
        self.max_slots = config.scheduler.max_active_requests
        self.max_context = config.max_sequence_length
        self.kv = SimulatedKVBackend(kv_capacity_tokens, config.kv.page_tokens,
                                     prefix_cache=config.kv.prefix_cache != "off")
        self.now_us = 0.0
        self.c_prefill, self.c_base, self.c_row = prefill_us_per_token, decode_us_base, decode_us_per_row
        self.fail_decode_for = set(fail_decode_for)
        self.fail_decode_admission = set(fail_decode_admission)
        self.admitted = 0
        self.free_slots = list(range(self.max_slots - 1, -1, -1))
        self.trace: List[Tuple[str, float, int]] = []
        self.spec_depth, self.spec_accept_rate = int(spec_depth), float(spec_accept_rate)
        self.spec_max_requests = int(spec_max_requests)
        self.supports_mtp = self.spec_depth > 0
        self.spec_stats = {"cycles": 0, "drafted": 0, "accepted": 0, "fallback_steps": 0}

    def admit(self, rs: RequestState) -> bool:
        if rs.total_budget_tokens > self.max_context:
            raise GenerationAdmissionRejected("context_overflow: request exceeds the context window")
        if not self.free_slots:
            return False
        lease = self.kv.admit(rs.rid, rs.req.prompt_token_ids, rs.req.max_tokens)
        if lease is None:
            return False
        rs.slot = self.free_slots.pop()
        rs.runner_data = lease
        if self.admitted in self.fail_decode_admission:
            self.fail_decode_for.add(rs.rid)
        self.admitted += 1
        cached = min(lease.cached_tokens, rs.prompt_len - 1)
        rs.prefilled = rs.cached_tokens = cached
        return True

    def prefill(self, work):
        out: Dict[int, Tuple[int, Optional[TokenLogprob]]] = {}
        n = sum(k for _, k in work)
        self.now_us += n * self.c_prefill
        self.trace.append(("prefill", self.now_us, n))
        for rs, k in work:
            if rs.prefilled + k >= rs.prompt_len:
                self.kv.publish_prefix(rs.req.prompt_token_ids, rs.runner_data)
                out[rs.rid] = (_tok(rs.req.prompt_token_ids, 0, self.vocab), None)
        return out

    def decode(self, rows: List[RequestState]):
        bad = [rs.rid for rs in rows if rs.rid in self.fail_decode_for]
        if bad:
            self.fail_decode_for -= set(bad)
            raise ExecutionFailure(bad, "decode", "injected decode failure", "none")
        self.now_us += self.c_base + self.c_row * len(rows)
        self.trace.append(("decode", self.now_us, len(rows)))
        return [(_tok(rs.req.prompt_token_ids, len(rs.generated), self.vocab), None) for rs in rows]

    # ------------------------------------------------------------------ speculative cycles
    def speculative_eligible(self, rs: RequestState) -> bool:
        from ..speculative.serving import resolve_mtp_serving_plan
        return resolve_mtp_serving_plan("on", self.supports_mtp, rs.req.temperature, self._needs_processing(rs),
                                        bool(rs.forced), bool(rs.req.logprobs), depth=self.spec_depth).use_mtp

    def _draft_matches(self, rs: RequestState, index: int) -> bool:
        h = hashlib.blake2b(repr(("draft", rs.rid, index)).encode(), digest_size=8).digest()
        return int.from_bytes(h, "little") / 2.0 ** 64 < self.spec_accept_rate

    def speculative_cycle(self, rows: List[RequestState]):
        from ..speculative.contracts import SpecCycleResult
        from ..speculative.policy import cycle_cost, plan_draft_depth
        bad = [rs.rid for rs in rows if rs.rid in self.fail_decode_for]
        if bad:
            self.fail_decode_for -= set(bad)
            raise ExecutionFailure(bad, "verify", "injected verify failure", "partial")
        depth = self.spec_depth
        for rs in rows:
            depth = min(depth, plan_draft_depth(self.spec_depth, rs.remaining(), rs.total_budget_tokens - rs.position,
                                                rs.telemetry.speculative_drafted, rs.telemetry.speculative_accepted,
                                                adaptive=self.config.speculative.adaptive_depth))
        if depth < 1 or len(rows) > self.spec_max_requests:
            self.spec_stats["fallback_steps"] += 1
            return [SpecCycleResult([t], 0, 0) for t, _ in self.decode(rows)]
        self.now_us += (self.c_base + self.c_row * len(rows)) * cycle_cost(depth)
        self.trace.append(("spec_cycle", self.now_us, len(rows)))
        out = []
        for rs in rows:
            base = len(rs.generated)
            n = 0
            while n < depth and self._draft_matches(rs, base + n):
                n += 1
            toks = [_tok(rs.req.prompt_token_ids, base + i, self.vocab) for i in range(n + 1)]
            out.append(SpecCycleResult(toks, depth, n))
            self.spec_stats["drafted"] += depth
            self.spec_stats["accepted"] += n
        self.spec_stats["cycles"] += 1
        return out

    def release(self, rs: RequestState) -> None:
        if rs.runner_data is not None:
            self.kv.release(rs.rid)
            rs.runner_data = None
        if rs.slot is not None and rs.slot not in self.free_slots:
            self.free_slots.append(rs.slot)

    def capacity(self) -> Dict[str, Any]:
        return {"backend": "simulated", "max_slots": self.max_slots, "max_context": self.max_context,
                **self.kv.capacity()}


def poisson_arrivals(n: int, rate_per_s: float, seed: int = 0) -> List[float]:
    """Arrival times (seconds) of a Poisson process with the given rate."""
    rng = random.Random(seed)
    t, out = 0.0, []
    for _ in range(n):
        t += -math.log(1.0 - rng.random()) / rate_per_s
        out.append(t)
    return out


@dataclass
class LoadResult:
    completed: int = 0
    failed: int = 0
    ttft_ms: List[float] = field(default_factory=list)
    itl_ms: List[float] = field(default_factory=list)
    total_tokens: int = 0
    makespan_s: float = 0.0
    cached_prompt_tokens: int = 0

    def summary(self) -> Dict[str, float]:
        def pct(xs, p):
            if not xs:
                return 0.0
            s = sorted(xs)
            return s[min(len(s) - 1, int(p * len(s)))]
        return {"completed": self.completed, "failed": self.failed, "tokens": self.total_tokens,
                "tok_per_s": self.total_tokens / self.makespan_s if self.makespan_s else 0.0,
                "ttft_p50_ms": pct(self.ttft_ms, 0.5), "ttft_p99_ms": pct(self.ttft_ms, 0.99),
                "itl_p50_ms": pct(self.itl_ms, 0.5), "itl_p99_ms": pct(self.itl_ms, 0.99),
                "cached_prompt_tokens": self.cached_prompt_tokens}


def run_load_scenario(config: EngineConfig, requests: Sequence[GenerationRequest], arrivals_s: Sequence[float],
                      max_concurrent: int = 64, runner: Optional[SimulatedRunner] = None) -> LoadResult:
    """Drive an ``EngineLoop`` over a simulated runner in virtual time: requests are submitted when the virtual
    clock passes their arrival time (at most ``max_concurrent`` in flight), the loop ticks until all are done."""
    from .engine_loop import EngineLoop
    runner = runner or SimulatedRunner(config)
    loop = EngineLoop(runner, config)
    order = sorted(range(len(requests)), key=lambda i: arrivals_s[i])
    nxt = 0
    arrival_us: Dict[int, float] = {}
    first_us: Dict[int, float] = {}
    last_us: Dict[int, float] = {}
    seen_tokens: Dict[int, int] = {}
    res = LoadResult()
    in_flight = 0

    def on_event(rs: RequestState) -> None:
        n = len(rs.generated)
        prev = seen_tokens.get(rs.rid, 0)
        if n > prev:
            if prev == 0:
                first_us[rs.rid] = runner.now_us
                res.ttft_ms.append((runner.now_us - arrival_us[rs.rid]) / 1e3)
            else:
                res.itl_ms.append((runner.now_us - last_us[rs.rid]) / 1e3 / (n - prev))
            last_us[rs.rid] = runner.now_us
            seen_tokens[rs.rid] = n

    loop.on_event = on_event
    done = set()
    guard = 0
    while len(done) < len(requests):
        while nxt < len(order) and in_flight < max_concurrent and arrivals_s[order[nxt]] * 1e6 <= runner.now_us:
            i = order[nxt]
            rid = loop.submit(requests[i]).rid
            arrival_us[rid] = arrivals_s[i] * 1e6
            nxt += 1
            in_flight += 1
        if loop.idle():
            if nxt < len(order):
                runner.now_us = max(runner.now_us, arrivals_s[order[nxt]] * 1e6)   # jump to the next arrival
                continue
            break
        loop.tick()
        for rid, rs in list(loop.sched.finished.items()):
            if rid in done:
                continue
            done.add(rid)
            in_flight -= 1
            if rs.error:
                res.failed += 1
            else:
                res.completed += 1
                res.total_tokens += len(rs.generated)
                res.cached_prompt_tokens += rs.cached_tokens
        guard += 1
        if guard > 10_000_000:
            raise RuntimeError("load scenario did not converge")
    res.makespan_s = runner.now_us / 1e6
    return res
