"""App-local chat sessions: transcript store, continuations, fork / rollback, snapshot export / restore.

Same scope as the reference (``hipengine/server/chat_sessions.py``, ``session_snapshots.py``): a session is a
transcript plus tokenizer metadata -- *not* KV; the radix prefix cache is what makes resending a transcript
cheap.  Snapshots are JSON documents with schema id ``he.chat_session_snapshot.v1``.
"""
from __future__ import annotations

import copy
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

SNAPSHOT_SCHEMA = "he.chat_session_snapshot.v1"


class SessionError(ValueError):
    def __init__(self, code: str, message: str):
        super().__init__(message)
        self.code = code


_ROLES = ("system", "developer", "user", "assistant", "tool")


def _check_transcript(msgs: Any) -> None:
    """A restored transcript must be what a chat request could have stored: a list of ``{role, content, ...}``
    objects with a known role and text (or parts, or nothing beside tool calls) as content.  Refusing it at restore
    time keeps a malformed document from becoming a session that fails on every later use."""
    if not isinstance(msgs, list):
        raise SessionError("invalid_continuation", "snapshot 'messages' must be a list")
    for i, m in enumerate(msgs):
        if not isinstance(m, dict) or m.get("role") not in _ROLES:
            raise SessionError("invalid_continuation", f"snapshot messages[{i}] has no supported role")
        c = m.get("content")
        if not (c is None or isinstance(c, str) or (isinstance(c, list) and all(isinstance(x, dict) for x in c))):
            raise SessionError("invalid_continuation", f"snapshot messages[{i}].content must be text or a list of parts")
        if "tool_calls" in m and not isinstance(m["tool_calls"], list):
            raise SessionError("invalid_continuation", f"snapshot messages[{i}].tool_calls must be a list")


@dataclass
class ChatSession:
    id: str
    messages: List[Dict[str, Any]] = field(default_factory=list)
    created: float = field(default_factory=time.time)
    updated: float = field(default_factory=time.time)
    turns: int = 0
    parent: Optional[str] = None


class ChatSessionStore:
    def __init__(self, max_sessions: int = 256, ttl_seconds: float = 3600.0):
        self.max_sessions = max_sessions
        self.ttl = ttl_seconds
        self.sessions: Dict[str, ChatSession] = {}
        self.lock = threading.Lock()

    def _expire(self) -> None:
        now = time.time()
        for sid in [s for s, v in self.sessions.items() if now - v.updated > self.ttl]:
            del self.sessions[sid]

    def get(self, sid: str) -> ChatSession:
        with self.lock:
            self._expire()
            if sid not in self.sessions:
                raise SessionError("continuation_expired" if sid.startswith("sess_") else "invalid_continuation",
                                   f"unknown or expired session {sid!r}")
            return self.sessions[sid]

    def create(self, messages: Optional[List[Dict[str, Any]]] = None, sid: Optional[str] = None) -> ChatSession:
        with self.lock:
            self._expire()
            if len(self.sessions) >= self.max_sessions:
                oldest = min(self.sessions.values(), key=lambda s: s.updated)
                del self.sessions[oldest.id]
            s = ChatSession(sid or "sess_" + uuid.uuid4().hex[:20], copy.deepcopy(messages or []))
            s.turns = sum(1 for m in s.messages if m.get("role") == "assistant")
            self.sessions[s.id] = s
            return s

    def append(self, sid: str, new_messages: List[Dict[str, Any]], assistant: Optional[Dict[str, Any]] = None) -> ChatSession:
        s = self.get(sid)
        with self.lock:
            s.messages.extend(copy.deepcopy(new_messages))
            if assistant is not None:
                s.messages.append(copy.deepcopy(assistant))
                s.turns += 1
            s.updated = time.time()
        return s

    def fork(self, sid: str) -> ChatSession:
        src = self.get(sid)
        child = self.create(src.messages)
        child.parent = sid
        child.turns = src.turns
        return child

    def rollback(self, sid: str, turns: int = 1) -> ChatSession:
        s = self.get(sid)
        with self.lock:
            for _ in range(max(0, turns)):
                while s.messages and s.messages[-1].get("role") != "assistant":
                    s.messages.pop()
                if s.messages:
                    s.messages.pop()
                while s.messages and s.messages[-1].get("role") in ("user", "tool"):
                    s.messages.pop()
                s.turns = max(0, s.turns - 1)
            s.updated = time.time()
        return s

    def delete(self, sid: str) -> bool:
        with self.lock:
            return self.sessions.pop(sid, None) is not None

    def list(self) -> List[Dict[str, Any]]:
        with self.lock:
            self._expire()
            return [{"id": s.id, "messages": len(s.messages), "turns": s.turns, "created": s.created,
                     "updated": s.updated, "parent": s.parent} for s in self.sessions.values()]

    def export(self, sid: str, tokenizer_meta: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        s = self.get(sid)
        return {"schema": SNAPSHOT_SCHEMA, "session": {"id": s.id, "messages": copy.deepcopy(s.messages),
                                                       "turns": s.turns, "created": s.created, "parent": s.parent},
                "tokenizer": tokenizer_meta or {}, "exported_at": time.time()}

    def restore(self, doc: Dict[str, Any], tokenizer_meta: Optional[Dict[str, Any]] = None) -> ChatSession:
        if doc.get("schema") != SNAPSHOT_SCHEMA:
            raise SessionError("invalid_continuation", f"unsupported snapshot schema {doc.get('schema')!r}")
        if tokenizer_meta and doc.get("tokenizer") and doc["tokenizer"].get("vocab_size") not in (
                None, tokenizer_meta.get("vocab_size")):
            raise SessionError("invalid_continuation", "snapshot was taken with a different tokenizer")
        body = doc.get("session")
        if not isinstance(body, dict):
            raise SessionError("invalid_continuation", "snapshot has no 'session' object")
        msgs = body.get("messages") or []
        _check_transcript(msgs)
        turns = body.get("turns", 0)
        if isinstance(turns, bool) or not isinstance(turns, int) or turns < 0:
            raise SessionError("invalid_continuation", "snapshot 'turns' must be a non-negative integer")
        s = self.create(msgs)
        s.turns = turns
        return s
