"""Terminal chat client of a *running server* (plain stdlib HTTP + SSE; rich rendering when available).

Commands mirror the reference client (``hipengine/chat_cli.py``; ``README.md:259-279``): ``/status /usage
/bench /think /retry /clear /quit``.  Per turn it prints TTFT and decode tokens/s from the stream timing.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
import urllib.request
from typing import Any, Dict, Iterator, List, Optional


class ChatClient:
    def __init__(self, base_url: str, api_key: Optional[str] = None, model: Optional[str] = None):
        self.base = base_url.rstrip("/")
        self.key = api_key
        self.model = model
        self.messages: List[Dict[str, Any]] = []
        self.think = True
        self.usage = {"prompt_tokens": 0, "completion_tokens": 0, "turns": 0}

    def _req(self, path: str, body: Optional[Dict[str, Any]] = None):
        headers = {"Content-Type": "application/json"}
        if self.key:
            headers["Authorization"] = f"Bearer {self.key}"
        data = None if body is None else json.dumps(body).encode()
        return urllib.request.urlopen(urllib.request.Request(self.base + path, data=data, headers=headers), timeout=600)

    def discover_model(self) -> str:
        if self.model is None:
            self.model = json.load(self._req("/v1/models"))["data"][0]["id"]
        return self.model

    def status(self) -> Dict[str, Any]:
        return json.load(self._req("/ready"))

    def stream_turn(self, text: str, max_tokens: int = 512) -> Iterator[Dict[str, Any]]:
        self.messages.append({"role": "user", "content": text})
        body = {"model": self.discover_model(), "messages": self.messages, "stream": True, "max_tokens": max_tokens,
                "enable_thinking": self.think, "stream_options": {"include_usage": True, "include_hipengine": True}}
        resp = self._req("/v1/chat/completions", body)
        answer = ""
        for raw in resp:
            line = raw.decode().strip()
            if not line.startswith("data: "):
                continue
            d = line[6:]
            if d == "[DONE]":
                break
            ev = json.loads(d)
            if ev.get("usage"):
                self.usage["prompt_tokens"] += ev["usage"]["prompt_tokens"]
                self.usage["completion_tokens"] += ev["usage"]["completion_tokens"]
            for ch in ev.get("choices", []):
                answer += ch.get("delta", {}).get("content") or ""
            yield ev
        self.messages.append({"role": "assistant", "content": answer})
        self.usage["turns"] += 1

    def retry(self) -> Optional[str]:
        while self.messages and self.messages[-1]["role"] == "assistant":
            self.messages.pop()
        if self.messages and self.messages[-1]["role"] == "user":
            return self.messages.pop()["content"]
        return None


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="hipengine-b200 chat")
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--model", default=None)
    ap.add_argument("--max-tokens", type=int, default=512)
    a = ap.parse_args(argv)
    c = ChatClient(a.url, a.api_key, a.model)
    try:
        print(f"connected to {a.url}, model {c.discover_model()}  (/status /usage /bench /think /retry /clear /quit)")
    except Exception as exc:
        print(f"cannot reach server: {exc}", file=sys.stderr)
        return 1
    pending: Optional[str] = None
    while True:
        try:
            line = pending if pending is not None else input("> ")
        except (EOFError, KeyboardInterrupt):
            print()
            return 0
        pending = None
        if not line.strip():
            continue
        if line.startswith("/"):
            cmd = line.split()[0]
            if cmd == "/quit":
                return 0
            if cmd == "/clear":
                c.messages.clear()
            elif cmd == "/think":
                c.think = not c.think
                print(f"thinking {'on' if c.think else 'off'}")
            elif cmd == "/usage":
                print(c.usage)
            elif cmd == "/status":
                print(json.dumps(c.status(), indent=1)[:2000])
            elif cmd == "/retry":
                pending = c.retry()
            elif cmd == "/bench":
                t0 = time.time()
                n = sum(1 for _ in c.stream_turn("Count from 1 to 50.", a.max_tokens))
                print(f"{n} events in {time.time() - t0:.2f}s")
            else:
                print("unknown command")
            continue
        last = {}
        for ev in c.stream_turn(line, a.max_tokens):
            for ch in ev.get("choices", []):
                d = ch.get("delta", {})
                sys.stdout.write(d.get("content") or "")
                sys.stdout.flush()
            last = ev.get("hipengine", last)
        t = (last or {}).get("timing", {})
        print(f"\n[ttft {t.get('ttft_ms')} ms, {t.get('decode_tokens_per_second')} tok/s]")


if __name__ == "__main__":
    sys.exit(main())
