"""Request replay log: every admitted API request as one JSON line, so that a production incident can be reproduced
offline with the same sampling parameters.

``--replay-dir DIR`` turns it on; ``--replay-redaction {none,hash,drop}`` controls what is kept of the prompt text:
``none`` keeps it, ``hash`` (default) replaces every string of the prompt / messages by its SHA-256 and length (enough
to see repeats and sizes, not content), ``drop`` removes the fields.  Sampling parameters, model name, route, stream
flag, arrival time and the request id are always kept; the outcome (finish reason, token counts, latency) is appended
as a second line when the request ends.  Files rotate by day.  The reference's server has the same switch pair
(``--replay-dir`` / ``--replay-redaction``, ``hipengine/server/__main__.py``).
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
import time
from typing import Any, Dict, Optional

PROMPT_FIELDS = ("prompt", "messages", "tools", "suffix")


def _redact(value: Any, mode: str) -> Any:
    if mode == "none":
        return value
    if isinstance(value, str):
        return {"sha256": hashlib.sha256(value.encode()).hexdigest(), "chars": len(value)}
    if isinstance(value, list):
        if value and all(isinstance(x, int) for x in value):
            raw = ",".join(str(x) for x in value)
            return {"sha256": hashlib.sha256(raw.encode()).hexdigest(), "tokens": len(value)}
        return [_redact(v, mode) for v in value]
    if isinstance(value, dict):
        return {k: (_redact(v, mode) if k in ("content", "text", "arguments", "description") or isinstance(v, (dict, list))
                    else v) for k, v in value.items()}
    return value


class ReplayLog:
    def __init__(self, directory: str, redaction: str = "hash"):
        if redaction not in ("none", "hash", "drop"):
            raise ValueError("replay redaction must be none, hash or drop")
        self.dir, self.redaction = directory, redaction
        os.makedirs(directory, exist_ok=True)
        self._lock = threading.Lock()
        self.written = 0

    def _path(self) -> str:
        return os.path.join(self.dir, time.strftime("requests-%Y%m%d.jsonl", time.gmtime()))

    def _write(self, rec: Dict[str, Any]) -> None:
        line = json.dumps(rec, default=str, separators=(",", ":"))
        with self._lock:
            with open(self._path(), "a", encoding="utf-8") as f:
                f.write(line + "\n")
            self.written += 1

    def request(self, request_id: str, route: str, body: Dict[str, Any]) -> None:
        rec: Dict[str, Any] = {"kind": "request", "id": request_id, "route": route, "t": time.time()}
        kept = {}
        for k, v in body.items():
            if k in PROMPT_FIELDS:
                if self.redaction == "drop":
                    continue
                kept[k] = _redact(v, self.redaction)
            else:
                kept[k] = v
        rec["body"] = kept
        self._write(rec)

    def outcome(self, request_id: str, finish_reason: Optional[str], prompt_tokens: int, completion_tokens: int,
                seconds: float, error: Optional[str] = None) -> None:
        self._write({"kind": "outcome", "id": request_id, "t": time.time(), "finish_reason": finish_reason,
                     "prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
                     "seconds": round(seconds, 4), "error": error})
