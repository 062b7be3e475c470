"""Parsing of model output into reasoning / content / tool calls, batch and incremental.

Behaviour of the reference's ``chat_output.py`` + ``tool_stream.py`` (``hipengine/server/chat_output.py``,
``hipengine/server/tool_stream.py``): ``<think>...</think>`` is split into ``reasoning_content``; tool calls
are ``<tool_call><function=NAME><parameter=K>V</parameter></function></tool_call>`` blocks (the legacy JSON
body ``{"name":..., "arguments":...}`` is also accepted); when streaming, the first delta of a call carries
the name and later deltas append argument JSON text, all with the same id and index.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"

_FUNC_RE = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


@dataclass
class ToolCall:
    name: str
    arguments: Dict[str, Any]
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])
    raw: str = ""
    error: Optional[str] = None

    def to_openai(self, index: Optional[int] = None) -> Dict[str, Any]:
        d = {"id": self.id, "type": "function",
             "function": {"name": self.name, "arguments": json.dumps(self.arguments, ensure_ascii=False)}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ParsedOutput:
    content: str = ""
    reasoning: Optional[str] = None
    tool_calls: List[ToolCall] = field(default_factory=list)
    thinking_closed: bool = True


def _coerce(v: str) -> Any:
    s = v.strip()
    try:
        return json.loads(s)
    except Exception:
        return v


def parse_tool_body(body: str) -> ToolCall:
    body = body.strip()
    m = _FUNC_RE.search(body)
    if m:
        args = {k: _coerce(v) for k, v in _PARAM_RE.findall(m.group(2))}
        return ToolCall(m.group(1), args, raw=body)
    try:
        obj = json.loads(body)
        args = obj.get("arguments", {})
        if isinstance(args, str):
            args = json.loads(args)
        return ToolCall(str(obj.get("name", "")), args if isinstance(args, dict) else {"value": args}, raw=body)
    except Exception as exc:
        return ToolCall("", {}, raw=body, error=f"unparseable tool call: {exc}")


def split_reasoning(text: str, starts_in_think: bool = False) -> Tuple[Optional[str], str, bool]:
    """Returns (reasoning, rest, closed).  ``starts_in_think``: the prompt already opened ``<think>``."""
    t = text
    if t.lstrip().startswith(THINK_OPEN):
        t = t.lstrip()[len(THINK_OPEN):]
        starts_in_think = True
    if not starts_in_think:
        return None, text, True
    i = t.find(THINK_CLOSE)
    if i < 0:
        return t.strip("\n"), "", False
    return t[:i].strip("\n"), t[i + len(THINK_CLOSE):].lstrip("\n"), True


def parse_chat_output(text: str, starts_in_think: bool = False, parse_tools: bool = True) -> ParsedOutput:
    reasoning, rest, closed = split_reasoning(text, starts_in_think)
    calls: List[ToolCall] = []
    content = rest
    if parse_tools and TOOL_OPEN in rest:
        parts = []
        pos = 0
        while True:
            i = rest.find(TOOL_OPEN, pos)
            if i < 0:
                parts.append(rest[pos:])
                break
            parts.append(rest[pos:i])
            j = rest.find(TOOL_CLOSE, i)
            body = rest[i + len(TOOL_OPEN):j if j >= 0 else len(rest)]
            calls.append(parse_tool_body(body))
            if j < 0:
                break
            pos = j + len(TOOL_CLOSE)
        content = "".join(parts).strip()
    return ParsedOutput(content, reasoning, calls, closed)


class ChatStreamParser:
    """Incremental splitter: feed text pieces, get (phase, delta) events.

    Phases: ``think`` (reasoning delta), ``answer`` (content delta), ``tool_call`` (dict delta in OpenAI shape).
    Text that could be the start of a tag is held back until it is disambiguated.
    """

    TAGS = (THINK_OPEN, THINK_CLOSE, TOOL_OPEN, TOOL_CLOSE)

    def __init__(self, starts_in_think: bool = False, parse_tools: bool = True):
        self.phase = "think" if starts_in_think else "answer"
        self.parse_tools = parse_tools
        self.buf = ""
        self.tool_buf = ""
        self.calls: List[ToolCall] = []
        self.seen_answer = False

    def _holdback(self, s: str) -> int:
        for k in range(min(len(s), max(len(t) for t in self.TAGS) - 1), 0, -1):
            tail = s[-k:]
            if any(t.startswith(tail) for t in self.TAGS):
                return k
        return 0

    def feed(self, piece: str, final: bool = False) -> List[Tuple[str, Any]]:
        self.buf += piece
        events: List[Tuple[str, Any]] = []
        while True:
            if self.phase == "tool_call":
                j = self.buf.find(TOOL_CLOSE)
                if j < 0:
                    if final:
                        self.tool_buf += self.buf
                        self.buf = ""
                        events += self._finish_call()
                    else:
                        hb = self._holdback(self.buf)
                        self.tool_buf += self.buf[:len(self.buf) - hb]
                        self.buf = self.buf[len(self.buf) - hb:]
                    break
                self.tool_buf += self.buf[:j]
                self.buf = self.buf[j + len(TOOL_CLOSE):]
                events += self._finish_call()
                self.phase = "answer"
                continue
            # think / answer
            nxt, tag = len(self.buf), None
            for t in self.TAGS:
                if t in (TOOL_OPEN, TOOL_CLOSE) and not self.parse_tools:
                    continue
                i = self.buf.find(t)
                if 0 <= i < nxt:
                    nxt, tag = i, t
            if tag is None:
                hb = 0 if final else self._holdback(self.buf)
                out = self.buf[:len(self.buf) - hb]
                self.buf = self.buf[len(self.buf) - hb:]
                if out:
                    events.append(self._text_event(out))
                break
            if nxt:
                events.append(self._text_event(self.buf[:nxt]))
            self.buf = self.buf[nxt + len(tag):]
            if tag == THINK_OPEN:
                self.phase = "think"
            elif tag == THINK_CLOSE:
                self.phase = "answer"
                self.buf = self.buf.lstrip("\n")
            elif tag == TOOL_OPEN:
                self.phase = "tool_call"
                self.tool_buf = ""
        return [e for e in events if e is not None]

    def _text_event(self, s: str):
        if self.phase == "answer":
            if not self.seen_answer:
                s = s.lstrip("\n")
            if not s:
                return None
            self.seen_answer = True
        return (self.phase, s)

    def _finish_call(self) -> List[Tuple[str, Any]]:
        call = parse_tool_body(self.tool_buf)
        self.tool_buf = ""
        idx = len(self.calls)
        self.calls.append(call)
        first = {"index": idx, "id": call.id, "type": "function", "function": {"name": call.name, "arguments": ""}}
        args = {"index": idx, "id": call.id, "function": {"arguments": json.dumps(call.arguments, ensure_ascii=False)}}
        return [("tool_call", first), ("tool_call", args)]
