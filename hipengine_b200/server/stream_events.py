"""Pure SSE frame construction and token / timing accounting for streamed responses.

Shapes follow the reference's stream projection (``hipengine/server/stream_events.py``;
``docs/API.md:885-960``): ``data: {chunk}\\n\\n`` ... ``data: [DONE]``; with ``stream_options.include_usage``
a final chunk with ``choices: []`` and ``usage``; with ``include_hipengine`` a per-event block carrying
elapsed_ms, ttft_ms, decode tokens/s and the per-choice phase (think | answer | tool_call | done).
"""
from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


def sse(data: Any) -> str:
    if isinstance(data, str):
        return f"data: {data}\n\n"
    return "data: " + json.dumps(data, ensure_ascii=False, separators=(",", ":")) + "\n\n"


SSE_DONE = "data: [DONE]\n\n"


@dataclass
class StreamTimingTracker:
    started: float = field(default_factory=time.perf_counter)
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    tokens: int = 0
    itl: List[float] = field(default_factory=list)

    def on_tokens(self, n: int) -> None:
        if n <= 0:
            return
        now = time.perf_counter()
        if self.first_token_at is None:
            self.first_token_at = now
        elif self.last_token_at is not None:
            self.itl.append((now - self.last_token_at) / n)
        self.last_token_at = now
        self.tokens += n

    def block(self) -> Dict[str, Any]:
        now = time.perf_counter()
        ttft = None if self.first_token_at is None else 1e3 * (self.first_token_at - self.started)
        tps = None
        if self.first_token_at is not None and self.tokens > 1 and self.last_token_at > self.first_token_at:
            tps = (self.tokens - 1) / (self.last_token_at - self.first_token_at)
        return {"timing": {"elapsed_ms": 1e3 * (now - self.started), "ttft_ms": ttft,
                           "decode_tokens_per_second": tps}}


@dataclass
class StreamTokenAccounting:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0
    reasoning_tokens: int = 0

    def usage(self) -> Dict[str, Any]:
        return {"prompt_tokens": self.prompt_tokens, "completion_tokens": self.completion_tokens,
                "total_tokens": self.prompt_tokens + self.completion_tokens,
                "prompt_tokens_details": {"cached_tokens": self.cached_tokens},
                "completion_tokens_details": {"reasoning_tokens": self.reasoning_tokens}}


def new_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


def chat_chunk(cid: str, model: str, created: int, delta: Dict[str, Any], index: int = 0,
               finish_reason: Optional[str] = None, logprobs: Any = None, extra: Optional[Dict[str, Any]] = None
               ) -> Dict[str, Any]:
    choice: Dict[str, Any] = {"index": index, "delta": delta, "finish_reason": finish_reason}
    if logprobs is not None:
        choice["logprobs"] = logprobs
    out = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model, "choices": [choice]}
    if extra:
        out["hipengine"] = extra
    return out


def completion_chunk(cid: str, model: str, created: int, text: str, index: int = 0,
                     finish_reason: Optional[str] = None, logprobs: Any = None,
                     extra: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    choice: Dict[str, Any] = {"index": index, "text": text, "finish_reason": finish_reason, "logprobs": logprobs}
    out = {"id": cid, "object": "text_completion", "created": created, "model": model, "choices": [choice]}
    if extra:
        out["hipengine"] = extra
    return out


def usage_chunk(cid: str, model: str, created: int, obj: str, usage: Dict[str, Any]) -> Dict[str, Any]:
    return {"id": cid, "object": obj, "created": created, "model": model, "choices": [], "usage": usage}
