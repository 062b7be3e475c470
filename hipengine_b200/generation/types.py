"""Request / output value types shared by the API, the engine and the server.

Field inventory follows the reference's generator registry types
(``hipengine/generation/registry.py``: ``GenerationRequest :97-255``, ``TokenLogprob :257``,
``GenerationTelemetry :610``, ``FinishDetails :806``, ``GenerationOutput :938``,
``GenerationStreamChunk :991``) and the dispatch value types
(``hipengine/dispatch/batch.py:16-172``: ``WorkKind``, ``RequestState``, ``WorkItem``).
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

_REQ_COUNTER = itertools.count(1)


def normalize_logit_bias(v: Any) -> Tuple[Tuple[int, float], ...]:
    if not v:
        return ()
    if isinstance(v, Mapping):
        items = v.items()
    else:
        items = v
    out = []
    for k, b in items:
        b = float(b)
        if not (-100.0 <= b <= 100.0):
            raise ValueError("logit_bias values must be in [-100, 100]")
        out.append((int(k), b))
    return tuple(sorted(out))


def normalize_stop_sequences(v: Any) -> Tuple[Tuple[int, ...], ...]:
    if not v:
        return ()
    out = []
    for seq in v:
        t = tuple(int(x) for x in seq)
        if t:
            out.append(t)
    return tuple(out)


class WorkKind(str, Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    VERIFY_CHAIN = "verify_chain"
    VERIFY_TREE = "verify_tree"


class FinishReason(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    EOS = "stop_eos"
    CANCELLED = "cancelled"
    DEADLINE = "deadline_exceeded"
    ERROR = "error"
    TOOL_CALLS = "tool_calls"


@dataclass
class FinishDetails:
    reason: str = "length"
    stop_token_id: Optional[int] = None
    stop_sequence: Optional[Tuple[int, ...]] = None
    message: Optional[str] = None

    @property
    def openai_reason(self) -> str:
        if self.reason in ("stop", "stop_eos"):
            return "stop"
        if self.reason == "tool_calls":
            return "tool_calls"
        return "length" if self.reason == "length" else self.reason


@dataclass
class TokenLogprob:
    token_id: int
    logprob: float
    top: Tuple[Tuple[int, float], ...] = ()


@dataclass
class GenerationTelemetry:
    prompt_tokens: int = 0
    cached_prompt_tokens: int = 0
    generated_tokens: int = 0
    sampler_mode: str = "greedy"
    execution_path: str = ""
    d2h_bytes: int = 0
    h2d_bytes: int = 0
    queue_seconds: float = 0.0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    ttft_seconds: float = 0.0
    speculative_cycles: int = 0
    speculative_drafted: int = 0
    speculative_accepted: int = 0
    fallbacks: List[str] = field(default_factory=list)

    @property
    def decode_tokens_per_second(self) -> float:
        return self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0

    def as_dict(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d["decode_tokens_per_second"] = self.decode_tokens_per_second
        return d


@dataclass
class GenerationRequest:
    prompt_token_ids: List[int]
    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Tuple[Tuple[int, float], ...] = ()
    suppress_token_ids: Tuple[int, ...] = ()
    min_tokens: int = 0
    eos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    stop_token_sequences: Tuple[Tuple[int, ...], ...] = ()
    forced_tokens_pending: Tuple[int, ...] = ()
    json_object_close_forcing: bool = False
    tool_call_constraint: Any = None
    thinking_close_token_ids: Tuple[int, ...] = ()
    thinking_hard_token_cap: Optional[int] = None
    thinking_soft_close_window: int = 0
    ignore_eos: bool = False
    seed: Optional[int] = None
    deadline_at: Optional[float] = None
    cancellation_token: Any = None
    session_key: Optional[str] = None
    speculative_mtp: bool = False
    logprobs: bool = False
    top_logprobs: int = 0
    prompt_text: Optional[str] = None
    row_index: int = 0
    request_id: int = field(default_factory=lambda: next(_REQ_COUNTER))
    created_at: float = field(default_factory=time.time)

    @classmethod
    def from_sampling(cls, ids: Sequence[int], sp: Any, prompt_text: Optional[str] = None,
                      row_index: int = 0) -> "GenerationRequest":
        seed = sp.seed
        if sp.row_seeds and row_index < len(sp.row_seeds):
            seed = sp.row_seeds[row_index]
        return cls(
            prompt_token_ids=list(ids), max_tokens=sp.max_tokens, temperature=sp.temperature, top_p=sp.top_p,
            top_k=sp.top_k, min_p=sp.min_p, repetition_penalty=sp.repetition_penalty,
            presence_penalty=sp.presence_penalty, frequency_penalty=sp.frequency_penalty,
            logit_bias=sp.logit_bias, suppress_token_ids=sp.suppress_token_ids, min_tokens=sp.min_tokens,
            eos_token_id=sp.eos_token_id, stop_token_ids=sp.stop_token_ids,
            stop_token_sequences=sp.stop_token_sequences, forced_tokens_pending=sp.forced_tokens_pending,
            json_object_close_forcing=sp.json_object_close_forcing, tool_call_constraint=sp.tool_call_constraint,
            thinking_close_token_ids=sp.thinking_close_token_ids, thinking_hard_token_cap=sp.thinking_hard_token_cap,
            thinking_soft_close_window=sp.thinking_soft_close_window, ignore_eos=sp.ignore_eos, seed=seed,
            deadline_at=sp.deadline_at, cancellation_token=sp.cancellation_token,
            session_key=sp.resident_session_key, speculative_mtp=sp.speculative_mtp, logprobs=sp.logprobs,
            top_logprobs=sp.top_logprobs, prompt_text=prompt_text, row_index=row_index)

    @property
    def sampler_mode(self) -> str:
        """greedy | sampled | processed (processors or constraints touch the logits)."""
        processed = (self.logit_bias or self.suppress_token_ids or self.repetition_penalty != 1.0
                     or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.min_tokens > 0
                     or self.json_object_close_forcing or self.tool_call_constraint is not None
                     or self.thinking_hard_token_cap is not None or self.forced_tokens_pending)
        if processed:
            return "processed"
        return "greedy" if self.temperature == 0.0 else "sampled"


@dataclass
class GenerationOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    text: Optional[str] = None
    finish: FinishDetails = field(default_factory=FinishDetails)
    logprobs: Optional[List[TokenLogprob]] = None
    telemetry: GenerationTelemetry = field(default_factory=GenerationTelemetry)
    error: Optional[str] = None

    @property
    def finish_reason(self) -> str:
        return self.finish.openai_reason


@dataclass
class GenerationStreamChunk:
    request_id: int
    token_ids: List[int]
    text: Optional[str] = None
    finished: bool = False
    finish: Optional[FinishDetails] = None
    logprobs: Optional[List[TokenLogprob]] = None
    telemetry: Optional[GenerationTelemetry] = None
    error: Optional[str] = None
