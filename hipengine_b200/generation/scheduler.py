"""Host-only continuous-batching scheduler state.

Roles of the reference's ``ResidentBatchScheduler`` (``hipengine/generation/batch_scheduler.py:982-2456``):
pending deque, active slots, per-request ``RequestState``, work producers for prefill chunks / decode rows /
speculative verify rows, commit of generated tokens with stop / EOS / length checks, stream chunk assembly with
stop-sequence hold-back, latency percentiles and graph-bucket statistics.  Nothing here touches the device.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

from .constraints import (ForcedTokenQueue, JsonObjectConstraintState, ThinkingBudgetState,
                          TokenSequenceDFAState, ToolCallConstraintState)
from .sampling import mix_seed
from .types import (FinishDetails, GenerationOutput, GenerationRequest, GenerationStreamChunk,
                    GenerationTelemetry, TokenLogprob, WorkKind)

PENDING, PREFILL, DECODE, FINISHED = "pending", "prefill", "decode", "finished"


class GenerationAdmissionRejected(RuntimeError):
    """The request can never be admitted (too long for the configured context / pool)."""


@dataclass
class RequestState:
    req: GenerationRequest
    status: str = PENDING
    slot: Optional[int] = None
    prefilled: int = 0                 # prompt tokens already in the cache (prefix hits included)
    cached_tokens: int = 0
    generated: List[int] = field(default_factory=list)
    logprobs: List[TokenLogprob] = field(default_factory=list)
    emitted: int = 0                   # generated tokens already handed to the stream
    finish: Optional[FinishDetails] = None
    error: Optional[str] = None
    telemetry: GenerationTelemetry = field(default_factory=GenerationTelemetry)
    seed: int = 0
    sample_counter: int = 0
    stop: Optional[TokenSequenceDFAState] = None
    forced: ForcedTokenQueue = field(default_factory=ForcedTokenQueue)
    json_state: Optional[JsonObjectConstraintState] = None
    thinking: Optional[ThinkingBudgetState] = None
    tool_state: Optional[ToolCallConstraintState] = None
    grammar: Any = None          # token-mask matcher of the tool-call grammar (generation/grammar.py), when enforced
    t_submit: float = field(default_factory=time.perf_counter)
    t_admit: float = 0.0
    t_first: float = 0.0
    t_last: float = 0.0
    runner_data: Any = None            # lease / draft state owned by the model runner
    spec: Any = None                   # speculative decoding state

    @property
    def rid(self) -> int:
        return self.req.request_id

    @property
    def prompt_len(self) -> int:
        return len(self.req.prompt_token_ids)

    @property
    def position(self) -> int:
        """Number of tokens in the sequence so far (next token is written at this position)."""
        return self.prompt_len + len(self.generated)

    @property
    def last_token(self) -> int:
        return self.generated[-1] if self.generated else self.req.prompt_token_ids[-1]

    @property
    def total_budget_tokens(self) -> int:
        return self.prompt_len + self.req.max_tokens

    def remaining(self) -> int:
        return self.req.max_tokens - len(self.generated)


class LatencyStats:
    def __init__(self, cap: int = 4096):
        self.ttft: Deque[float] = deque(maxlen=cap)
        self.itl: Deque[float] = deque(maxlen=cap)

    @staticmethod
    def _pct(xs: Sequence[float], p: float) -> float:
        if not xs:
            return 0.0
        s = sorted(xs)
        return s[min(len(s) - 1, int(p * len(s)))]

    def snapshot(self) -> Dict[str, float]:
        return {"ttft_p50_ms": 1e3 * self._pct(self.ttft, 0.5), "ttft_p99_ms": 1e3 * self._pct(self.ttft, 0.99),
                "itl_p50_ms": 1e3 * self._pct(self.itl, 0.5), "itl_p99_ms": 1e3 * self._pct(self.itl, 0.99),
                "samples": len(self.itl)}


class Scheduler:
    def __init__(self, max_active: int, max_pending: int, eos_token_id: Optional[int],
                 decode: Optional[Callable[[Sequence[int]], str]] = None,
                 encode: Optional[Callable[[str], List[int]]] = None):
        self.max_active = max_active
        self.max_pending = max_pending
        self.eos_token_id = eos_token_id
        self.decode_text = decode
        self.tokenizer = None        # set by the engine loop: the grammar matcher needs the whole vocabulary
        self.encode_text = encode
        self.pending: Deque[RequestState] = deque()
        self.active: Dict[int, RequestState] = {}
        self.finished: Dict[int, RequestState] = {}
        self.latency = LatencyStats()
        self.counters = {"submitted": 0, "admitted": 0, "finished": 0, "cancelled": 0, "failed": 0,
                         "prefill_tokens": 0, "decode_tokens": 0, "prefill_chunks": 0, "decode_steps": 0,
                         "cached_prompt_tokens": 0, "spec_cycles": 0, "spec_drafted": 0, "spec_accepted": 0}
        self._rr = 0
        self._rejected: List[RequestState] = []

    def drain_rejected(self) -> List[RequestState]:
        out, self._rejected = self._rejected, []
        return out

    # ------------------------------------------------------------------ submission
    def submit(self, req: GenerationRequest) -> RequestState:
        if len(self.pending) >= self.max_pending:
            raise GenerationAdmissionRejected("engine_busy: pending queue is full")
        if not req.prompt_token_ids:
            raise GenerationAdmissionRejected("empty prompt")
        rs = RequestState(req)
        # an explicit seed makes a request repeatable: its rows are told apart by their index alone; without one the
        # engine-wide request id keeps concurrent requests apart
        rs.seed = mix_seed(req.seed, req.row_index, req.request_id if req.seed is None else 0)
        rs.telemetry.prompt_tokens = len(req.prompt_token_ids)
        rs.telemetry.sampler_mode = req.sampler_mode
        if req.stop_token_sequences:
            rs.stop = TokenSequenceDFAState(req.stop_token_sequences)
        if req.forced_tokens_pending:
            rs.forced = ForcedTokenQueue(req.forced_tokens_pending, "forced_tokens")
        if req.thinking_close_token_ids:
            rs.thinking = ThinkingBudgetState(tuple(req.thinking_close_token_ids), req.thinking_hard_token_cap,
                                              req.thinking_soft_close_window)
        if req.json_object_close_forcing and self.decode_text and self.encode_text:
            rs.json_state = JsonObjectConstraintState(self.decode_text, self.encode_text)
        if req.tool_call_constraint is not None and self.decode_text:
            rs.tool_state = ToolCallConstraintState(req.tool_call_constraint, self.decode_text)
            spec = req.tool_call_constraint
            if getattr(spec, "tools_json", None) and self.tokenizer is not None:
                import json as _json
                from .grammar import tool_call_matcher
                try:
                    rs.grammar = tool_call_matcher(
                        _json.loads(spec.tools_json), self.tokenizer,
                        req.eos_token_id if req.eos_token_id is not None else self.eos_token_id,
                        # the definitions travel only when the tool choice demands a call (required / a named
                        # function): then nothing but calls is admitted -- free text first would let a model that
                        # does not want to call talk forever
                        allow_text_before=False, parallel=True,
                        only=spec.specific if spec.mode == "specific" else None)
                except ValueError:
                    rs.grammar = None        # names the grammar cannot express: post-validation still applies
        self.pending.append(rs)
        self.counters["submitted"] += 1
        return rs

    def find(self, rid: int) -> Optional[RequestState]:
        if rid in self.active:
            return self.active[rid]
        for rs in self.pending:
            if rs.rid == rid:
                return rs
        return self.finished.get(rid)

    # ------------------------------------------------------------------ admission
    def admit_pending(self, try_admit: Callable[[RequestState], bool]) -> List[RequestState]:
        """Move pending requests into active slots while ``try_admit`` (the runner's reservation) succeeds."""
        admitted: List[RequestState] = []
        while self.pending and len(self.active) < self.max_active:
            rs = self.pending[0]
            try:
                ok = try_admit(rs)
            except GenerationAdmissionRejected as exc:
                self.pending.popleft()
                self._finish(rs, FinishDetails("error", message=str(exc)), error=str(exc))
                self._rejected.append(rs)
                continue
            if not ok:
                break                      # head-of-line: keep arrival order, retry next tick
            self.pending.popleft()
            rs.status = PREFILL
            rs.t_admit = time.perf_counter()
            rs.telemetry.queue_seconds = rs.t_admit - rs.t_submit
            rs.telemetry.cached_prompt_tokens = rs.cached_tokens
            self.counters["cached_prompt_tokens"] += rs.cached_tokens
            self.active[rs.rid] = rs
            self.counters["admitted"] += 1
            admitted.append(rs)
        return admitted

    # ------------------------------------------------------------------ work producers
    def prefill_rows(self) -> List[RequestState]:
        return [rs for rs in self.active.values() if rs.status == PREFILL]

    def decode_rows(self) -> List[RequestState]:
        return [rs for rs in self.active.values() if rs.status == DECODE]

    def next_prefill_work(self, chunk_tokens: int, budget_tokens: int, round_robin: bool = False
                          ) -> List[Tuple[RequestState, int]]:
        """(request, n_tokens) chunks for this tick, at most ``budget_tokens`` prompt tokens in total."""
        rows = self.prefill_rows()
        if not rows:
            return []
        if round_robin and len(rows) > 1:
            self._rr = (self._rr + 1) % len(rows)
            rows = rows[self._rr:] + rows[:self._rr]
        work: List[Tuple[RequestState, int]] = []
        left = budget_tokens
        for rs in rows:
            if left <= 0:
                break
            n = min(chunk_tokens, rs.prompt_len - rs.prefilled, left)
            if n > 0:
                work.append((rs, n))
                left -= n
        return work

    def next_decode_work(self, row_budget: int) -> List[RequestState]:
        rows = self.decode_rows()
        return rows[:row_budget]

    # ------------------------------------------------------------------ commits
    def record_prefill(self, rs: RequestState, n_tokens: int) -> None:
        rs.prefilled += n_tokens
        self.counters["prefill_tokens"] += n_tokens
        self.counters["prefill_chunks"] += 1

    def record_token(self, rs: RequestState, token: int, logprob: Optional[TokenLogprob] = None) -> bool:
        """Append one generated token; returns True when the request finished with it."""
        now = time.perf_counter()
        if not rs.generated:
            rs.t_first = now
            rs.telemetry.ttft_seconds = now - rs.t_submit
            rs.telemetry.prefill_seconds = now - rs.t_admit
            self.latency.ttft.append(rs.telemetry.ttft_seconds)
            rs.status = DECODE
        else:
            self.latency.itl.append(now - rs.t_last)
        rs.t_last = now
        rs.generated.append(int(token))
        rs.sample_counter += 1
        if logprob is not None:
            rs.logprobs.append(logprob)
        self.counters["decode_tokens"] += 1
        req = rs.req
        was_thinking = rs.thinking is not None and rs.thinking.thinking
        if rs.thinking is not None:
            rs.thinking.push(token)
            if rs.thinking.must_force_close():
                rs.forced.extend(rs.thinking.forced_close(), "thinking_hard_cap")
        if rs.json_state is not None:
            rs.json_state.push(token)
        if rs.tool_state is not None:
            rs.tool_state.push(token)
        if rs.grammar is not None and not was_thinking:
            rs.grammar.accept(token)          # the thinking block (and the token that closes it) is outside the grammar
        n = len(rs.generated)
        eos = req.eos_token_id if req.eos_token_id is not None else self.eos_token_id
        if n >= req.min_tokens:
            if not req.ignore_eos and eos is not None and token == eos and not (rs.thinking and rs.thinking.thinking):
                return self._finish(rs, FinishDetails("stop_eos", stop_token_id=token), trim=1)
            if token in req.stop_token_ids:
                return self._finish(rs, FinishDetails("stop", stop_token_id=token), trim=1)
            if rs.stop is not None and rs.stop.push(token):
                return self._finish(rs, FinishDetails("stop", stop_sequence=rs.stop.matched),
                                    trim=len(rs.stop.matched))
        elif rs.stop is not None:
            rs.stop.push(token)
        if rs.json_state is not None and rs.json_state.complete:
            return self._finish(rs, FinishDetails("stop", message="json_object_closed"))
        if rs.json_state is not None and not rs.forced and not rs.json_state.complete and rs.remaining() <= 64:
            # close while the closing suffix still fits: it grows by at most a few tokens per generated token (a new
            # key adds `": null`), so eight tokens of slack are kept between its length and the room that is left
            close = rs.json_state.forced_close_tokens()
            if close and len(close) <= rs.remaining() <= len(close) + 8:
                rs.forced.extend(close, "json_close_forcing")
        if n >= req.max_tokens:
            return self._finish(rs, FinishDetails("length"))
        return False

    def _finish(self, rs: RequestState, details: FinishDetails, trim: int = 0, error: Optional[str] = None) -> bool:
        if rs.status == FINISHED:
            return True
        if trim and details.reason in ("stop", "stop_eos"):
            rs.generated = rs.generated[:len(rs.generated) - trim]
            if rs.logprobs:
                rs.logprobs = rs.logprobs[:len(rs.generated)]
        rs.finish = details
        rs.error = error
        rs.status = FINISHED
        rs.telemetry.generated_tokens = len(rs.generated)
        if rs.t_first:
            rs.telemetry.decode_seconds = max(time.perf_counter() - rs.t_first, 1e-9)
        self.active.pop(rs.rid, None)
        self.finished[rs.rid] = rs
        self.counters["finished"] += 1
        if details.reason == "cancelled":
            self.counters["cancelled"] += 1
        if details.reason == "error":
            self.counters["failed"] += 1
        return True

    def cancel(self, rid: int, reason: str = "cancelled", message: Optional[str] = None) -> Optional[RequestState]:
        rs = self.active.get(rid)
        if rs is None:
            for cand in list(self.pending):
                if cand.rid == rid:
                    self.pending.remove(cand)
                    rs = cand
                    break
        if rs is None:
            return None
        self._finish(rs, FinishDetails(reason, message=message), error=message if reason == "error" else None)
        return rs

    def fail(self, rid: int, message: str) -> Optional[RequestState]:
        return self.cancel(rid, "error", message)

    # ------------------------------------------------------------------ streaming
    def take_stream_tokens(self, rs: RequestState) -> List[int]:
        """Newly generated tokens safe to emit (tokens that may still turn into a stop sequence are held back)."""
        hold = 0 if rs.status == FINISHED or rs.stop is None else rs.stop.holdback()
        upto = max(rs.emitted, len(rs.generated) - hold)
        out = rs.generated[rs.emitted:upto]
        rs.emitted = upto
        return out

    def make_output(self, rs: RequestState) -> GenerationOutput:
        return GenerationOutput(rs.rid, list(rs.req.prompt_token_ids), list(rs.generated), None,
                                rs.finish or FinishDetails("length"),
                                list(rs.logprobs) if rs.req.logprobs else None, rs.telemetry, rs.error)

    def pop_finished(self, rid: int) -> Optional[RequestState]:
        return self.finished.pop(rid, None)

    def snapshot(self) -> Dict[str, Any]:
        return {"pending": len(self.pending), "active": len(self.active),
                "prefill_rows": len(self.prefill_rows()), "decode_rows": len(self.decode_rows()),
                "counters": dict(self.counters), "latency": self.latency.snapshot()}
