"""Request-owned decoding constraints evaluated on the host between steps.

Parity with the reference's constraint states (``hipengine/generation/constraints.py:20-923``):
``TokenSequenceDFAState`` (stop sequences with stream hold-back), ``ForcedTokenQueue``,
``JsonObjectConstraintState`` (root-object prefix masking + parse-validated close forcing),
``ThinkingBudgetState`` (soft-close bias ramp, EOS suppression while thinking, forced close sequence at the
hard cap) and ``ToolCallConstraintState`` (allowed-function envelope check).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple


class TokenSequenceDFAState:
    """Matches any of several stop token sequences; reports how many trailing tokens must be held back
    from the stream because they might still become part of a stop sequence."""

    def __init__(self, sequences: Sequence[Sequence[int]]):
        self.seqs = [tuple(s) for s in sequences if len(s) > 0]
        self.max_len = max((len(s) for s in self.seqs), default=0)
        self.tail: List[int] = []
        self.matched: Optional[Tuple[int, ...]] = None

    def push(self, token: int) -> bool:
        """Feed one generated token.  True when a stop sequence just completed."""
        if not self.seqs:
            return False
        self.tail.append(int(token))
        if len(self.tail) > self.max_len:
            self.tail = self.tail[-self.max_len:]
        for s in self.seqs:
            if len(self.tail) >= len(s) and tuple(self.tail[-len(s):]) == s:
                self.matched = s
                return True
        return False

    def holdback(self) -> int:
        """Number of most recent tokens that are a proper prefix of some stop sequence."""
        best = 0
        for s in self.seqs:
            for k in range(min(len(s) - 1, len(self.tail)), 0, -1):
                if tuple(self.tail[-k:]) == s[:k]:
                    best = max(best, k)
                    break
        return best


class ForcedTokenQueue:
    def __init__(self, tokens: Sequence[int] = (), reason: Optional[str] = None):
        self.pending = list(tokens)
        self.reason = reason

    def __bool__(self) -> bool:
        return bool(self.pending)

    def pop(self) -> int:
        return self.pending.pop(0)

    def extend(self, tokens: Sequence[int], reason: Optional[str] = None) -> None:
        self.pending.extend(tokens)
        if reason:
            self.reason = reason


_LITERALS = ("true", "false", "null")


def json_closing_suffix(text: str) -> str:
    """Suffix that completes ``text``, a prefix of a JSON document, into a parseable one.

    One pass over the characters keeps, per open container, what is expected next (object: key / colon / value /
    comma-or-end; array: value / comma-or-end) and whether a string, a literal or a number is in progress."""
    stack: List[List[str]] = []            # [kind "{" or "[", state]
    in_str = esc = False
    str_is_key = False
    scalar = ""                            # literal or number in progress

    def value_done() -> None:
        if stack:
            stack[-1][1] = "comma"

    for ch in text:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
                if str_is_key:
                    stack[-1][1] = "colon"
                else:
                    value_done()
            continue
        if scalar:
            if ch in "+-.0123456789eEtrufalsn" and not ch.isspace():
                scalar += ch
                continue
            scalar = ""
            value_done()
        if ch.isspace():
            continue
        if ch == '"':
            in_str = True
            str_is_key = bool(stack) and stack[-1][0] == "{" and stack[-1][1] in ("key", "key_or_end")
        elif ch == "{":
            stack.append(["{", "key_or_end"])
        elif ch == "[":
            stack.append(["[", "value_or_end"])
        elif ch in "}]":
            if stack:
                stack.pop()
            value_done()
        elif ch == ":":
            if stack:
                stack[-1][1] = "value"
        elif ch == ",":
            if stack:
                stack[-1][1] = "key" if stack[-1][0] == "{" else "value"
        else:
            scalar = ch
    out = ""
    if in_str:
        if esc:
            out += "\\"                   # a lone backslash would escape the closing quote
        out += '"'
        if str_is_key:
            out += ": null"
    elif scalar:
        lit = next((l for l in _LITERALS if l.startswith(scalar)), None)
        if lit is not None:
            out += lit[len(scalar):]
        elif scalar[-1] in "+-.eE":
            out += "0"
    for depth in range(len(stack) - 1, -1, -1):
        kind, state = stack[depth]
        if depth == len(stack) - 1 and not in_str and not scalar:
            if state == "colon":
                out += ": null"
            elif state == "value":
                out += " null"
            elif state == "key":
                out += ' "_": null'        # after a trailing comma an object needs one more member
        out += "}" if kind == "{" else "]"
    return out


class JsonObjectConstraintState:
    """Tracks whether the decoded text so far is a prefix of one JSON object and when it is complete.

    The engine masks nothing for arbitrary vocabularies (no token->text table is assumed); it uses the state
    to (a) stop as soon as the root object closes and validates, and (b) near the token budget, force the
    shortest closing suffix that makes the text parse.
    """

    def __init__(self, decode: Callable[[Sequence[int]], str], encode: Callable[[str], List[int]]):
        self.decode = decode
        self.encode = encode
        self.ids: List[int] = []
        self.complete = False

    def push(self, token: int) -> None:
        self.ids.append(int(token))
        text = self.decode(self.ids).strip()
        if text.startswith("{") and text.endswith("}"):
            try:
                if isinstance(json.loads(text), dict):
                    self.complete = True
            except Exception:
                pass

    def closing_suffix(self) -> str:
        """Shortest suffix that makes the current text (a prefix of one JSON object) parse: closes an open string,
        completes a cut literal or number, supplies the value a key or a colon is waiting for, drops into ``null``
        after a trailing comma, and closes the open arrays / objects."""
        return json_closing_suffix(self.decode(self.ids))

    def forced_close_tokens(self) -> List[int]:
        if not self.decode(self.ids).strip():
            return self.encode("{}")
        return self.encode(self.closing_suffix())


@dataclass
class ThinkingBudgetState:
    """Thinking runs from the start of generation until ``close_ids`` has been emitted."""
    close_ids: Tuple[int, ...] = ()
    hard_cap: Optional[int] = None
    soft_window: int = 0
    thinking: bool = True
    n_think: int = 0
    _tail: List[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if not self.close_ids:
            self.thinking = False

    def push(self, token: int) -> None:
        if not self.thinking:
            return
        self.n_think += 1
        self._tail.append(int(token))
        n = len(self.close_ids)
        if len(self._tail) > n:
            self._tail = self._tail[-n:]
        if tuple(self._tail) == tuple(self.close_ids):
            self.thinking = False

    def suppress_eos(self) -> bool:
        return self.thinking

    def close_bias(self) -> float:
        """Additive logit bias on the first close token inside the soft-close window (linear ramp to +10)."""
        if not self.thinking or self.hard_cap is None or self.soft_window <= 0:
            return 0.0
        start = self.hard_cap - self.soft_window
        if self.n_think < start:
            return 0.0
        return 10.0 * min(1.0, (self.n_think - start + 1) / self.soft_window)

    def must_force_close(self) -> bool:
        return self.thinking and self.hard_cap is not None and self.n_think >= self.hard_cap

    def forced_close(self) -> List[int]:
        self.thinking = False
        return list(self.close_ids)


@dataclass(frozen=True)
class ToolCallConstraintSpec:
    allowed_functions: Tuple[str, ...] = ()
    mode: str = "auto"            # auto | required | specific
    specific: Optional[str] = None
    allow_think_prefix: bool = True
    # tool definitions (JSON text of the OpenAI "tools" list): when present and the mode demands a call (required /
    # specific), token masks from the in-tree grammar matcher enforce the call format while it is generated
    tools_json: Optional[str] = None


class ToolCallConstraintState:
    """Envelope-level check of ``<tool_call><function=NAME>`` openings against the allowed function names."""

    def __init__(self, spec: ToolCallConstraintSpec, decode: Callable[[Sequence[int]], str]):
        self.spec = spec
        self.decode = decode
        self.ids: List[int] = []
        self.violation: Optional[str] = None

    def push(self, token: int) -> None:
        self.ids.append(int(token))
        text = self.decode(self.ids)
        pos = 0
        while True:
            i = text.find("<function=", pos)
            if i < 0:
                break
            j = text.find(">", i)
            if j < 0:
                break
            name = text[i + len("<function="):j]
            allowed = (self.spec.specific,) if self.spec.mode == "specific" and self.spec.specific else \
                self.spec.allowed_functions
            if allowed and name not in allowed:
                self.violation = f"function {name!r} is not one of {list(allowed)}"
            pos = j + 1

    def satisfied(self) -> bool:
        text = self.decode(self.ids)
        if self.spec.mode in ("required", "specific"):
            return "<tool_call>" in text and self.violation is None
        return self.violation is None
