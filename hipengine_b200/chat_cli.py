"""Terminal chat client of a *running server* (plain stdlib HTTP + SSE).

What the reference client does (``hipengine/chat_cli.py``: ``_Settings, _Usage, _Conversation, _Turn, _Bench``;
``README.md:259-279``) and this one follows: discover the served model, stream the answer as it arrives with the
reasoning part set apart, and after every turn show what the server measured -- time to first token, decode rate,
prompt / cached-prompt / completion / reasoning token counts.  Commands: ``/status /usage /bench [N] /think /system
TEXT /max N /temp T /retry /undo /clear /save FILE /help /quit``.

The transport is a small callable so that the client can be driven against an in-process app in tests.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
import urllib.request
from dataclasses import dataclass
from typing import Any, Dict, Iterable, Iterator, List, Optional, TextIO

HELP = ("/status  readiness document      /usage  token totals           /bench [N]  N timed turns (default 3)\n"
        "/think   toggle thinking          /system TEXT  system prompt    /max N      max tokens per turn\n"
        "/temp T  sampling temperature     /retry  resend the last turn   /undo       drop the last turn\n"
        "/clear   forget the conversation  /save FILE  write transcript   /quit")

BENCH_PROMPT = "Count from 1 to 50, one number per line."


class HttpTransport:
    """``get(path) -> dict`` and ``stream(path, body) -> iterator of SSE data payloads`` over urllib."""

    def __init__(self, base_url: str, api_key: Optional[str] = None, timeout: float = 600.0):
        self.base, self.key, self.timeout = base_url.rstrip("/"), api_key, timeout

    def _open(self, path: str, body: Optional[Dict[str, Any]] = None):
        headers = {"Content-Type": "application/json"}
        if self.key:
            headers["Authorization"] = f"Bearer {self.key}"
        data = None if body is None else json.dumps(body).encode()
        return urllib.request.urlopen(urllib.request.Request(self.base + path, data=data, headers=headers),
                                      timeout=self.timeout)

    def get(self, path: str) -> Dict[str, Any]:
        return json.load(self._open(path))

    def stream(self, path: str, body: Dict[str, Any]) -> Iterator[str]:
        for raw in self._open(path, body):
            line = raw.decode().strip()
            if line.startswith("data: "):
                yield line[6:]


@dataclass
class Settings:
    max_tokens: int = 512
    temperature: Optional[float] = None
    think: bool = True
    system: Optional[str] = None


@dataclass
class TurnStats:
    """What one turn cost, from the server's own accounting (usage chunk + per-event timing block)."""
    ttft_ms: Optional[float] = None
    decode_tok_s: Optional[float] = None
    elapsed_ms: Optional[float] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    completion_tokens: int = 0
    reasoning_tokens: int = 0
    finish_reason: Optional[str] = None
    wall_s: float = 0.0

    def line(self) -> str:
        f = lambda v, spec: "-" if v is None else format(v, spec)
        cached = f" ({self.cached_tokens} cached)" if self.cached_tokens else ""
        think = f" ({self.reasoning_tokens} reasoning)" if self.reasoning_tokens else ""
        return (f"[ttft {f(self.ttft_ms, '.0f')} ms | {f(self.decode_tok_s, '.1f')} tok/s | prompt "
                f"{self.prompt_tokens}{cached} | completion {self.completion_tokens}{think} | {self.finish_reason}]")


@dataclass
class Usage:
    turns: int = 0
    prompt_tokens: int = 0
    cached_tokens: int = 0
    completion_tokens: int = 0
    reasoning_tokens: int = 0

    def add(self, t: TurnStats) -> None:
        self.turns += 1
        self.prompt_tokens += t.prompt_tokens
        self.cached_tokens += t.cached_tokens
        self.completion_tokens += t.completion_tokens
        self.reasoning_tokens += t.reasoning_tokens


@dataclass
class Delta:
    """One piece of a streamed turn: answer text, reasoning text, or the start of a tool call."""
    kind: str            # "content" | "reasoning" | "tool_call"
    text: str


class ChatClient:
    def __init__(self, transport, model: Optional[str] = None, settings: Optional[Settings] = None):
        self.t = transport
        self.model = model
        self.settings = settings or Settings()
        self.messages: List[Dict[str, Any]] = []
        self.usage = Usage()
        self.last: Optional[TurnStats] = None

    # ------------------------------------------------------------------ server
    def discover_model(self) -> str:
        if self.model is None:
            self.model = self.t.get("/v1/models")["data"][0]["id"]
        return self.model

    def status(self) -> Dict[str, Any]:
        return self.t.get("/ready")

    # ------------------------------------------------------------------ one turn
    def _body(self, messages: List[Dict[str, Any]]) -> Dict[str, Any]:
        s = self.settings
        msgs = ([{"role": "system", "content": s.system}] if s.system else []) + messages
        body = {"model": self.discover_model(), "messages": msgs, "stream": True, "max_tokens": s.max_tokens,
                "enable_thinking": s.think, "stream_options": {"include_usage": True, "include_hipengine": True}}
        if s.temperature is not None:
            body["temperature"] = s.temperature
        return body

    def stream_turn(self, text: str, remember: bool = True) -> Iterator[Delta]:
        """Send ``text`` as the next user turn and yield the pieces as they arrive; afterwards ``self.last`` holds the
        turn's statistics and (with ``remember``) the transcript has grown by the user and assistant messages."""
        messages = self.messages + [{"role": "user", "content": text}]
        st = TurnStats()
        answer, t0 = "", time.time()
        for payload in self.t.stream("/v1/chat/completions", self._body(messages)):
            if payload == "[DONE]":
                break
            ev = json.loads(payload)
            if "error" in ev:
                raise RuntimeError(ev["error"].get("message", "server error"))
            u = ev.get("usage")
            if u:
                st.prompt_tokens, st.completion_tokens = u.get("prompt_tokens", 0), u.get("completion_tokens", 0)
                st.cached_tokens = (u.get("prompt_tokens_details") or {}).get("cached_tokens", 0)
                st.reasoning_tokens = (u.get("completion_tokens_details") or {}).get("reasoning_tokens", 0)
            timing = (ev.get("hipengine") or {}).get("timing") or {}
            if timing:
                st.ttft_ms = timing.get("ttft_ms", st.ttft_ms)
                st.decode_tok_s = timing.get("decode_tokens_per_second", st.decode_tok_s)
                st.elapsed_ms = timing.get("elapsed_ms", st.elapsed_ms)
            for ch in ev.get("choices", []):
                d = ch.get("delta", {})
                if ch.get("finish_reason"):
                    st.finish_reason = ch["finish_reason"]
                if d.get("reasoning_content"):
                    yield Delta("reasoning", d["reasoning_content"])
                if d.get("content"):
                    answer += d["content"]
                    yield Delta("content", d["content"])
                for tc in d.get("tool_calls") or []:
                    name = (tc.get("function") or {}).get("name")
                    if name:
                        yield Delta("tool_call", name)
        st.wall_s = time.time() - t0
        self.last = st
        self.usage.add(st)
        if remember:
            self.messages = messages + [{"role": "assistant", "content": answer}]

    def ask(self, text: str, remember: bool = True) -> str:
        return "".join(d.text for d in self.stream_turn(text, remember) if d.kind == "content")

    # ------------------------------------------------------------------ transcript edits
    def undo(self) -> bool:
        """Drop the last user turn and its answer."""
        while self.messages and self.messages[-1]["role"] != "user":
            self.messages.pop()
        if self.messages:
            self.messages.pop()
            return True
        return False

    def retry(self) -> Optional[str]:
        """Remove the last exchange and return its user text for resending."""
        while self.messages and self.messages[-1]["role"] != "user":
            self.messages.pop()
        return self.messages.pop()["content"] if self.messages else None

    def bench(self, turns: int = 3, prompt: str = BENCH_PROMPT) -> Dict[str, Any]:
        """``turns`` independent single-turn requests (not added to the transcript): medians of what the server
        measured."""
        rows: List[TurnStats] = []
        for _ in range(max(1, turns)):
            saved = self.messages
            self.messages = []
            try:
                for _d in self.stream_turn(prompt, remember=False):
                    pass
            finally:
                self.messages = saved
            rows.append(self.last)
        med = lambda xs: statistics.median(xs) if xs else None
        return {"turns": len(rows),
                "ttft_ms_median": med([r.ttft_ms for r in rows if r.ttft_ms is not None]),
                "decode_tok_s_median": med([r.decode_tok_s for r in rows if r.decode_tok_s is not None]),
                "completion_tokens": sum(r.completion_tokens for r in rows),
                "cached_prompt_tokens": sum(r.cached_tokens for r in rows),
                "wall_s": round(sum(r.wall_s for r in rows), 3)}

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8") as f:
            json.dump({"model": self.model, "system": self.settings.system, "messages": self.messages}, f, indent=1)


def run_repl(c: ChatClient, lines: Iterable[str], out: TextIO, color: bool = False) -> int:
    """The command loop over an iterable of input lines (``sys.stdin`` interactively, a list in tests)."""
    dim, reset = ("\033[2m", "\033[0m") if color else ("", "")
    pending: Optional[str] = None
    it = iter(lines)
    while True:
        if pending is not None:
            line, pending = pending, None
        else:
            try:
                line = next(it)
            except (StopIteration, EOFError, KeyboardInterrupt):
                return 0
        line = line.rstrip("\n")
        if not line.strip():
            continue
        if line.startswith("/"):
            cmd, _, arg = line.partition(" ")
            arg = arg.strip()
            s = c.settings
            try:
                if cmd == "/quit":
                    return 0
                elif cmd == "/help":
                    print(HELP, file=out)
                elif cmd == "/clear":
                    c.messages = []
                elif cmd == "/think":
                    s.think = not s.think
                    print(f"thinking {'on' if s.think else 'off'}", file=out)
                elif cmd == "/system":
                    s.system = arg or None
                elif cmd == "/max":
                    s.max_tokens = max(1, int(arg))
                elif cmd == "/temp":
                    s.temperature = None if arg in ("", "default") else float(arg)
                elif cmd == "/usage":
                    print(json.dumps(c.usage.__dict__), file=out)
                elif cmd == "/status":
                    print(json.dumps(c.status(), indent=1)[:4000], file=out)
                elif cmd == "/retry":
                    pending = c.retry()
                elif cmd == "/undo":
                    print("dropped the last turn" if c.undo() else "nothing to drop", file=out)
                elif cmd == "/save":
                    c.save(arg or "chat.json")
                    print(f"saved {len(c.messages)} messages", file=out)
                elif cmd == "/bench":
                    print(json.dumps(c.bench(int(arg) if arg else 3)), file=out)
                else:
                    print("unknown command (/help)", file=out)
            except (ValueError, OSError, RuntimeError) as exc:
                print(f"error: {exc}", file=out)
            continue
        try:
            mode = None
            for d in c.stream_turn(line):
                if d.kind != mode:
                    if mode == "reasoning":
                        out.write(reset + "\n")
                    if d.kind == "reasoning":
                        out.write(dim)
                    mode = d.kind
                out.write(f"[tool call: {d.text}]" if d.kind == "tool_call" else d.text)
                out.flush()
            if mode == "reasoning":
                out.write(reset)
            print("\n" + c.last.line(), file=out)
        except Exception as exc:                      # noqa: BLE001 - a failed turn must not end the session
            print(f"\nerror: {exc}", file=out)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="hipengine-b200 chat")
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--model", default=None)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--system", default=None)
    ap.add_argument("--no-think", action="store_true")
    a = ap.parse_args(argv)
    c = ChatClient(HttpTransport(a.url, a.api_key), a.model,
                   Settings(max_tokens=a.max_tokens, temperature=a.temperature, think=not a.no_think, system=a.system))
    try:
        print(f"connected to {a.url}, model {c.discover_model()}  (/help for commands)")
    except Exception as exc:                          # noqa: BLE001
        print(f"cannot reach server: {exc}", file=sys.stderr)
        return 1

    def prompt_lines() -> Iterator[str]:
        while True:
            try:
                yield input("> ")
            except (EOFError, KeyboardInterrupt):
                print()
                return

    return run_repl(c, prompt_lines(), sys.stdout, color=sys.stdout.isatty())


if __name__ == "__main__":
    sys.exit(main())
