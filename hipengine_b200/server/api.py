"""OpenAI-compatible HTTP server (FastAPI).

Routes and observable behaviour follow the reference's contract (``hipengine/server/api.py:7133-8069``,
``docs/API.md:473-496``): ``/health`` (unauthenticated liveness), ``/ready`` (200/503 + capacity and unhealthy
reason), ``/v1/models``, ``/metrics`` (opt-in), ``/v1/completions`` and ``/v1/chat/completions`` (SSE token
streaming, logprobs, tools, structured output, thinking controls, deadlines, cancel on disconnect),
tokenize / detokenize / count_tokens / fit_context, chat sessions (list / delete / fork / rollback / snapshot
export + restore) and the ``/v1/hipengine/*`` introspection routes.  The asyncio side never touches the
device: requests go to the engine service, whose single driver thread owns the model; a bounded in-process
queue applies back-pressure (429 + Retry-After).
"""
from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from fastapi.exceptions import RequestValidationError
from fastapi import Depends, FastAPI, Request
from starlette.exceptions import HTTPException as StarletteHTTPException
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..generation.types import GenerationOutput, GenerationRequest, TokenLogprob
from ..llm import LLM, SamplingParams
from . import stream_events as SE
from .chat_output import ChatStreamParser, parse_chat_output
from .chat_sessions import ChatSessionStore, SessionError
from .errors import APIError, classify_engine_error
from .metrics import ServerMetrics
from .request_build import ResultPlan, apply_result_policy, build_chat, build_completion_params
from .schemas import ChatCompletionRequest, CompletionRequest, DetokenizeRequest, TokenizeRequest


@dataclass
class ServerConfig:
    served_model_name: str = "he-b200"
    api_key: Optional[str] = None
    chat_default_max_tokens: int = 4096
    completion_default_max_tokens: int = 16
    max_queued_requests: int = 256
    request_timeout_ms: Optional[int] = None
    stream_queue_max_chunks: int = 16
    metrics: Optional[str] = None            # "prometheus" enables /metrics
    max_chat_sessions: int = 256
    mtp_breaker_threshold: int = 3
    shutdown_grace_seconds: float = 5.0
    batch_window_ms: float = 0.0             # hold compatible requests this long so they are released together
    max_batch_size: int = 64                 # ... or until this many are waiting
    replay_dir: Optional[str] = None         # request replay log (server/replay.py)
    replay_redaction: str = "hash"           # none | hash | drop

    def validate(self) -> None:
        if self.max_queued_requests < 1:
            raise ValueError("max_queued_requests must be >= 1")
        if self.stream_queue_max_chunks < 1:
            raise ValueError("stream_queue_max_chunks must be >= 1")
        if self.metrics not in (None, "prometheus"):
            raise ValueError("metrics must be None or 'prometheus'")
        if self.replay_redaction not in ("none", "hash", "drop"):
            raise ValueError("replay_redaction must be none, hash or drop")


class MTPCircuitBreaker:
    """Per (model, profile, context bucket of 256) failure counter; an open scope falls back to plain decoding
    until an operator rolls it back (``hipengine/server/api.py:3398-3490``)."""

    def __init__(self, threshold: int = 3):
        self.threshold = threshold
        self.failures: Dict[Tuple[str, int], int] = {}
        self.open: Dict[Tuple[str, int], float] = {}

    @staticmethod
    def scope(model: str, ctx_tokens: int) -> Tuple[str, int]:
        return (model, ctx_tokens // 256)

    def allow(self, model: str, ctx_tokens: int) -> bool:
        return self.scope(model, ctx_tokens) not in self.open

    def record(self, model: str, ctx_tokens: int, ok: bool) -> None:
        k = self.scope(model, ctx_tokens)
        if ok:
            self.failures.pop(k, None)
            return
        self.failures[k] = self.failures.get(k, 0) + 1
        if self.failures[k] >= self.threshold:
            self.open[k] = time.time()

    def rollback(self) -> int:
        n = len(self.open)
        self.open.clear()
        self.failures.clear()
        return n

    def snapshot(self) -> Dict[str, Any]:
        return {"open_scopes": [{"model": m, "ctx_bucket": b, "since": t} for (m, b), t in self.open.items()],
                "threshold": self.threshold}


from .batcher import GenerationBatcher  # noqa: E402


def _lp_chat(lps: Optional[List[TokenLogprob]], tok) -> Optional[Dict[str, Any]]:
    if lps is None:
        return None
    content = []
    for lp in lps:
        s = tok.decode([lp.token_id])
        content.append({"token": s, "logprob": lp.logprob, "bytes": list(s.encode("utf-8")),
                        "top_logprobs": [{"token": tok.decode([t]), "logprob": v,
                                          "bytes": list(tok.decode([t]).encode("utf-8"))} for t, v in lp.top]})
    return {"content": content}


def _lp_completion(lps: Optional[List[TokenLogprob]], tok, offset0: int = 0) -> Optional[Dict[str, Any]]:
    if lps is None:
        return None
    tokens, tlp, top, offs = [], [], [], []
    off = offset0
    for lp in lps:
        s = tok.decode([lp.token_id])
        tokens.append(s)
        tlp.append(lp.logprob)
        top.append({tok.decode([t]): v for t, v in lp.top})
        offs.append(off)
        off += len(s)
    return {"tokens": tokens, "token_logprobs": tlp, "top_logprobs": top, "text_offset": offs}


class _Bridge:
    """Runs a blocking chunk iterator on a worker thread and exposes it as an async iterator through a
    bounded queue (``StreamBridgePool`` in the reference, ``hipengine/server/stream_bridge.py``)."""

    def __init__(self, make_iter, maxsize: int):
        self.loop = asyncio.get_running_loop()
        self.q: asyncio.Queue = asyncio.Queue(maxsize=maxsize)
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._run, args=(make_iter,), daemon=True)
        self.thread.start()

    def _put(self, item) -> None:
        fut = asyncio.run_coroutine_threadsafe(self.q.put(item), self.loop)
        while not self.stop.is_set():
            try:
                fut.result(timeout=0.25)
                return
            except Exception as exc:  # timeout -> retry unless the consumer is gone
                if not isinstance(exc, (TimeoutError, asyncio.TimeoutError)) and not fut.running():
                    return
        fut.cancel()

    def _run(self, make_iter) -> None:
        try:
            for ch in make_iter():
                if self.stop.is_set():
                    break
                self._put(("chunk", ch))
            self._put(("end", None))
        except BaseException as exc:
            self._put(("error", exc))

    async def __aiter__(self):
        while True:
            kind, val = await self.q.get()
            if kind == "end":
                return
            if kind == "error":
                raise val
            yield val

    def close(self) -> None:
        self.stop.set()


def create_app(llm: LLM, config: Optional[ServerConfig] = None) -> FastAPI:
    cfg = config or ServerConfig()
    cfg.validate()
    metrics = ServerMetrics()
    gate = GenerationBatcher(cfg.max_queued_requests, cfg.batch_window_ms, cfg.max_batch_size)

    from contextlib import asynccontextmanager

    @asynccontextmanager
    async def lifespan(_app):
        yield
        # drain: refuse new work, give requests in flight a grace period, then close the engine
        gate.drain()
        deadline = time.time() + cfg.shutdown_grace_seconds
        while gate.in_flight > 0 and time.time() < deadline:
            await asyncio.sleep(0.05)
        await asyncio.get_running_loop().run_in_executor(None, llm.close)

    app = FastAPI(title="hipengine_b200", version="0.1.0", lifespan=lifespan)
    sessions = ChatSessionStore(cfg.max_chat_sessions)
    replay = None
    if cfg.replay_dir:
        from .replay import ReplayLog
        replay = ReplayLog(cfg.replay_dir, cfg.replay_redaction)

    def replay_request(cid: str, route: str, req_model) -> float:
        if replay is not None:
            replay.request(cid, route, req_model.model_dump(exclude_none=True))
        return time.time()

    def replay_outcome(cid: str, t0: float, reason, prompt_tokens: int, completion_tokens: int, error=None) -> None:
        if replay is not None:
            replay.outcome(cid, reason, prompt_tokens, completion_tokens, time.time() - t0, error)
    breaker = MTPCircuitBreaker(cfg.mtp_breaker_threshold)
    state = {"started": time.time(), "ready": False, "startup": []}
    app.state.llm, app.state.cfg, app.state.metrics, app.state.sessions, app.state.breaker = llm, cfg, metrics, sessions, breaker

    def tok():
        return llm._get_tokenizer()

    def arch() -> str:
        w = getattr(llm, "_weights", None)
        if w is not None:
            return w.config.arch
        ex = getattr(llm, "model", None)
        return getattr(getattr(ex, "cfg", None), "arch", "qwen35")

    # ------------------------------------------------------------------ plumbing
    @app.exception_handler(APIError)
    async def _api_error(_: Request, exc: APIError):
        headers = {"Retry-After": str(int(max(1, exc.retry_after)))} if exc.retry_after else None
        metrics.inc("hipengine_http_errors_total", code=exc.code)
        return JSONResponse(exc.body(), status_code=exc.status, headers=headers)

    @app.exception_handler(SessionError)
    async def _session_error(_: Request, exc: SessionError):
        return JSONResponse(APIError(exc.code, str(exc)).body(), status_code=APIError(exc.code, "").status)

    @app.exception_handler(ValueError)
    async def _bad_value(_: Request, exc: ValueError):
        """``LLM`` refuses malformed requests (empty prompt, token ids outside the vocabulary, a bad sampler value)
        with ``ValueError`` before anything reaches the engine: the client's error."""
        metrics.inc("hipengine_http_errors_total", code="invalid_request")
        e = APIError("invalid_request", str(exc))
        return JSONResponse(e.body(), status_code=e.status)

    @app.exception_handler(Exception)
    async def _unexpected(_: Request, exc: Exception):
        """Anything a route did not turn into an API error still answers in the envelope (500, not retryable)."""
        import logging
        logging.getLogger("hipengine_b200.server").exception("unhandled error in a route")
        metrics.inc("hipengine_http_errors_total", code="internal_error")
        e = APIError("internal_error", f"{type(exc).__name__}: {exc}")
        return JSONResponse(e.body(), status_code=e.status)

    @app.exception_handler(StarletteHTTPException)
    async def _http_error(request: Request, exc: StarletteHTTPException):
        """An unknown path or a wrong method answers in the envelope too (the framework's default is ``{"detail": ..}``)."""
        code = {404: "not_found", 405: "method_not_allowed"}.get(exc.status_code, "invalid_request")
        metrics.inc("hipengine_http_errors_total", code=code)
        body = APIError(code, f"{request.method} {request.url.path}: {exc.detail}").body()
        return JSONResponse(body, status_code=exc.status_code, headers=getattr(exc, "headers", None))

    @app.exception_handler(RequestValidationError)
    async def _validation_error(_: Request, exc: RequestValidationError):
        """A body that does not fit the request schema answers in the same envelope as every other client error (the
        framework's default is a bare 422 list)."""
        errs = exc.errors()
        first = errs[0] if errs else {}
        loc = [str(x) for x in first.get("loc", ()) if x != "body"]
        param = ".".join(loc) or None
        msg = "; ".join(f"{'.'.join(str(x) for x in e.get('loc', ()) if x != 'body')}: {e.get('msg')}" for e in errs[:3])
        metrics.inc("hipengine_http_errors_total", code="invalid_request")
        e = APIError("invalid_request", f"request body does not match the schema: {msg}", param)
        return JSONResponse(e.body(), status_code=e.status)

    async def auth(request: Request) -> None:
        if cfg.api_key:
            h = request.headers.get("authorization", "")
            if h != f"Bearer {cfg.api_key}":
                raise APIError("unauthorized", "missing or invalid bearer token")

    def check_model(name: Optional[str]) -> None:
        if name and name != cfg.served_model_name:
            raise APIError("model_unavailable", f"model {name!r} is not served here (serving {cfg.served_model_name!r})",
                           "model")

    def engine():
        try:
            return llm._get_engine()
        except Exception as exc:
            raise APIError("engine_unavailable", f"engine is not available: {exc}") from None

    def with_timeout(sp: SamplingParams) -> SamplingParams:
        if sp.deadline_at is None and cfg.request_timeout_ms:
            from dataclasses import replace
            return replace(sp, deadline_at=time.time() + cfg.request_timeout_ms / 1e3)
        return sp

    def raise_for_output(out: GenerationOutput) -> None:
        if out.error:
            code = classify_engine_error(out.error)
            extra = {}
            if code == "context_overflow":
                extra = {"fit_context": {"prompt_tokens": len(out.prompt_token_ids),
                                         "max_context": engine().capacity().get("max_context")}}
            raise APIError(code, out.error, extra=extra)
        if out.finish.reason == "deadline_exceeded":
            raise APIError("deadline_exceeded", "the request deadline passed before generation finished")

    async def run_blocking(fn, *a):
        return await asyncio.get_running_loop().run_in_executor(None, fn, *a)

    # ------------------------------------------------------------------ liveness / readiness / introspection
    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/ready")
    async def ready():
        from .readiness import build_readiness
        h = llm.engine_service_health()
        cap = live = None
        err = None
        if llm._engine is not None and h.get("healthy"):
            try:
                cap = await run_blocking(llm.resident_capacity_estimate)
                live = await run_blocking(llm.live_loop_snapshot)
            except Exception as exc:
                err = str(exc)
        mcfg = getattr(llm._weights, "config", None) if getattr(llm, "_weights", None) is not None else \
            getattr(getattr(llm, "model", None), "cfg", None)
        body = build_readiness(model_id=cfg.served_model_name, health=h, startup=llm.startup, capacity=cap, live=live,
                               config=llm.config, server_cfg=cfg, gate=gate,
                               sessions={"count": len(sessions.sessions), "max": cfg.max_chat_sessions}, started=state["started"],
                               model_cfg=mcfg, error=err)
        return JSONResponse(body, status_code=200 if body["ready"] else 503)

    @app.get("/v1/models", dependencies=[Depends(auth)])
    async def models():
        return {"object": "list", "data": [{"id": cfg.served_model_name, "object": "model",
                                            "created": int(state["started"]), "owned_by": "hipengine_b200"}]}

    @app.get("/metrics")
    async def metrics_route():
        if cfg.metrics != "prometheus":
            raise APIError("unsupported_feature", "metrics are disabled (start with --metrics prometheus)")
        snap, cap = {}, {}
        if llm._engine is not None:
            try:
                snap = await run_blocking(llm.live_loop_snapshot)
                cap = await run_blocking(llm.resident_capacity_estimate)
            except Exception:
                pass
        return PlainTextResponse(metrics.render(snap, cap, gate.in_flight, gate.snapshot()), media_type="text/plain; version=0.0.4")

    @app.get("/v1/hipengine/capabilities", dependencies=[Depends(auth)])
    async def capabilities():
        return {"model": cfg.served_model_name, "backend": llm.backend, "profile": llm.profile.value,
                "features": {"streaming": True, "logprobs": True, "tools": True, "structured_output": True,
                             "thinking_controls": True, "prefix_cache": llm.config.kv.prefix_cache,
                             "speculative_mtp": llm.config.speculative.mode, "sessions": True},
                "limits": {"max_queued_requests": cfg.max_queued_requests, "top_logprobs": 20, "n": 16},
                "mtp_circuit_breaker": breaker.snapshot(), "model_family": _family()}

    def _family() -> Optional[Dict[str, Any]]:
        """The served family's declaration (layer schedule, block types read in place, providers, KV storage)."""
        from ..models.registry import plugin_for
        w = getattr(llm, "_weights", None)
        mcfg = getattr(w, "config", None) or getattr(getattr(llm, "model", None), "cfg", None)
        try:
            return plugin_for(arch()).describe(mcfg)
        except KeyError:
            return None

    @app.get("/v1/hipengine/decode", dependencies=[Depends(auth)])
    async def decode_state():
        return await run_blocking(llm.live_loop_snapshot)

    @app.post("/v1/hipengine/speculative_mtp/rollback", dependencies=[Depends(auth)])
    async def mtp_rollback():
        return {"closed_scopes": breaker.rollback()}

    @app.post("/v1/hipengine/tokenize", dependencies=[Depends(auth)])
    async def tokenize(req: TokenizeRequest):
        text = req.text if req.text is not None else (req.prompt or "")
        if req.messages:
            from ..chat.templates import render_chat
            text = render_chat([m.model_dump(exclude_none=True) for m in req.messages], arch=arch())
        ids = tok().encode(text)
        return {"tokens": ids, "count": len(ids)}

    @app.post("/v1/hipengine/detokenize", dependencies=[Depends(auth)])
    async def detokenize(req: DetokenizeRequest):
        return {"text": tok().decode(req.tokens)}

    @app.post("/v1/hipengine/count_tokens", dependencies=[Depends(auth)])
    async def count_tokens(req: TokenizeRequest):
        r = await tokenize(req)
        return {"count": r["count"]}

    @app.post("/v1/hipengine/fit_context", dependencies=[Depends(auth)])
    async def fit_context(req: TokenizeRequest):
        """Does this input fit the served context, how many tokens may follow it, and (with ``max_tokens``) would a
        request asking for that many be admitted.  The reference's route of the same name
        (``hipengine/server/api.py:7664``) answers the same question from its own tokenizer count."""
        if req.max_tokens is not None and req.max_tokens < 1:
            raise APIError("unsupported_parameter", "max_tokens must be >= 1", "max_tokens")
        r = await tokenize(req)
        fit = await run_blocking(llm.fit_context, r["tokens"], req.max_tokens)
        kind = "chat" if req.messages else "text"
        out = {"object": "hipengine.fit_context", "input_type": kind, "requested_max_tokens": req.max_tokens, **fit}
        if kind == "chat":
            out["chat_default_max_tokens"] = cfg.chat_default_max_tokens
            out["fits_with_default_max_tokens"] = fit["prompt_tokens"] + cfg.chat_default_max_tokens <= fit["max_context"]
        return out

    # ------------------------------------------------------------------ completions
    def _prompts(req: CompletionRequest) -> List[Any]:
        p = req.prompt
        if isinstance(p, str):
            return [p]
        if isinstance(p, list) and p and all(isinstance(x, int) for x in p):
            return [p]
        if isinstance(p, list) and p:
            return list(p)
        raise APIError("invalid_request", "prompt must not be empty", "prompt")

    def _usage(outs: List[GenerationOutput]) -> Dict[str, Any]:
        acc = SE.StreamTokenAccounting()
        for o in outs:
            acc.prompt_tokens += o.telemetry.prompt_tokens
            acc.completion_tokens += len(o.token_ids)
            acc.cached_tokens += o.telemetry.cached_prompt_tokens
        return acc.usage()

    @app.post("/v1/audio/songs", dependencies=[Depends(auth)])
    async def audio_songs(request: Request):
        """Song generation (lyrics + style -> audio) is a separate diffusion / codec pipeline in the reference
        (``hipengine/server/api.py:7732``); this engine serves text models only and says so with 501."""
        raise APIError("unsupported_feature", "song generation is not served by this engine (text generation only: "
                                              "/v1/completions, /v1/chat/completions)")

    def stream_request(prompt_ids, sp):
        """The engine request of a live stream, checked BEFORE the response starts: a malformed prompt or one that
        cannot fit the served context answers with its HTTP status instead of an error event inside a 200 stream.  The
        caller holds a place in the admission gate; it is given back when the check refuses."""
        try:
            greq = llm._request(prompt_ids, sp, 0)
            fit = llm.fit_context(greq.prompt_token_ids, greq.max_tokens)
            if not fit.get("fits_with_max_tokens", True):
                raise APIError("context_overflow", f"context_overflow: prompt {fit['prompt_tokens']} + max_tokens "
                                                   f"{greq.max_tokens} exceeds max context {fit['max_context']}")
            return greq, engine()
        except BaseException:
            gate.leave()
            raise

    @app.post("/v1/completions", dependencies=[Depends(auth)])
    async def completions(req: CompletionRequest, request: Request):
        check_model(req.model)
        t = tok()
        sp = with_timeout(build_completion_params(req, t, cfg.completion_default_max_tokens))
        prompts = _prompts(req)
        cid, created = SE.new_id("cmpl"), int(time.time())
        t_req = replay_request(cid, "completions", req)
        gate.enter()
        try:
            await gate.admit(gate.compat_key("completions", bool(req.stream), sp.temperature == 0.0, bool(sp.logprobs),
                                             bool(getattr(sp, "json_schema", None) or getattr(sp, "grammar", None))))
        except BaseException:
            gate.leave()
            raise
        metrics.inc("hipengine_requests_total", route="completions")
        live = req.stream and len(prompts) == 1 and req.n == 1 and not req.echo
        if live:
            greq, eng = stream_request(prompts[0], sp)
            opts = req.stream_options
            timing = SE.StreamTimingTracker()

            async def gen():
                bridge = _Bridge(lambda: eng.stream(greq), cfg.stream_queue_max_chunks)
                dec = t.stream_decoder()
                n_out, cached = 0, 0
                try:
                    async for ch in bridge:
                        if await request.is_disconnected():
                            eng.cancel(greq.request_id, wait=False)
                            break
                        if ch.error:
                            yield SE.sse(APIError(classify_engine_error(ch.error), ch.error).body())
                            break
                        text = dec.feed(ch.token_ids) + (dec.flush() if ch.finished else "")
                        n_out += len(ch.token_ids)
                        timing.on_tokens(len(ch.token_ids))
                        fr = ch.finish.openai_reason if ch.finished else None
                        extra = timing.block() if opts and opts.include_hipengine else None
                        if text or ch.finished:
                            yield SE.sse(SE.completion_chunk(cid, cfg.served_model_name, created, text, 0, fr,
                                                             _lp_completion(ch.logprobs, t), extra))
                        if ch.finished and ch.telemetry is not None:
                            cached = ch.telemetry.cached_prompt_tokens
                    if opts and opts.include_usage:
                        acc = SE.StreamTokenAccounting(len(greq.prompt_token_ids), n_out, cached)
                        yield SE.sse(SE.usage_chunk(cid, cfg.served_model_name, created, "text_completion", acc.usage()))
                    yield SE.SSE_DONE
                finally:
                    bridge.close()
                    gate.leave()
                    metrics.inc("hipengine_generated_tokens_total", n_out)
                    replay_outcome(cid, t_req, "stream", len(greq.prompt_token_ids), n_out)
            return StreamingResponse(gen(), media_type="text/event-stream")
        try:
            plist = [p for p in prompts for _ in range(req.n)]
            sps = [sp] * len(plist)
            outs = await run_blocking(llm.generate_detailed, plist, sps)
        finally:
            gate.leave()
        for o in outs:
            raise_for_output(o)
        choices = []
        for i, (p, o) in enumerate(zip(plist, outs)):
            text = o.text or ""
            if req.echo:
                text = (p if isinstance(p, str) else t.decode(p)) + text
            choices.append({"index": i, "text": text, "finish_reason": o.finish_reason,
                            "logprobs": _lp_completion(o.logprobs, t)})
        metrics.inc("hipengine_generated_tokens_total", sum(len(o.token_ids) for o in outs))
        body = {"id": cid, "object": "text_completion", "created": created, "model": cfg.served_model_name,
                "choices": choices, "usage": _usage(outs)}
        replay_outcome(cid, t_req, choices[0]["finish_reason"] if choices else None, body["usage"]["prompt_tokens"],
                       body["usage"]["completion_tokens"])
        if req.stream:   # buffered SSE for multi-prompt / n>1 / echo
            async def buffered():
                for c in choices:
                    yield SE.sse(SE.completion_chunk(cid, cfg.served_model_name, created, c["text"], c["index"],
                                                     c["finish_reason"], c["logprobs"]))
                if req.stream_options and req.stream_options.include_usage:
                    yield SE.sse(SE.usage_chunk(cid, cfg.served_model_name, created, "text_completion", body["usage"]))
                yield SE.SSE_DONE
            return StreamingResponse(buffered(), media_type="text/event-stream")
        return body

    # ------------------------------------------------------------------ chat completions
    def _session_messages(req: ChatCompletionRequest):
        """Continuation / session handling: prepend the stored transcript, remember where to append."""
        sid = req.continuation_id or (req.session if isinstance(req.session, str) else
                                      (req.session or {}).get("id") if isinstance(req.session, dict) else None)
        if sid is None:
            return None, req
        from .schemas import ChatMessage
        s = sessions.get(sid)
        merged = [ChatMessage(**m) for m in s.messages] + list(req.messages)
        return sid, req.model_copy(update={"messages": merged})

    def _assistant_message(parsed, details) -> Dict[str, Any]:
        msg: Dict[str, Any] = {"role": "assistant", "content": parsed.content or None}
        if parsed.reasoning is not None:
            msg["reasoning_content"] = parsed.reasoning
        if parsed.tool_calls and not (details and details["reason"].startswith("invalid")):
            msg["tool_calls"] = [c.to_openai() for c in parsed.tool_calls]
            if not parsed.content:
                msg["content"] = None
        return msg

    @app.post("/v1/chat/completions", dependencies=[Depends(auth)])
    async def chat_completions(req: ChatCompletionRequest, request: Request):
        check_model(req.model)
        t = tok()
        new_msgs = [m.model_dump(exclude_none=True) for m in req.messages]
        sid, full_req = _session_messages(req)
        prompt, sp, plan = build_chat(full_req, t, arch(), cfg.chat_default_max_tokens)
        sp = with_timeout(sp)
        prompt_ids = t.encode(prompt)
        if sp.speculative_mtp and not breaker.allow(cfg.served_model_name, len(prompt_ids)):
            from dataclasses import replace
            sp = replace(sp, speculative_mtp=False)
        cid, created = SE.new_id("chatcmpl"), int(time.time())
        t_req = replay_request(cid, "chat", req)
        gate.enter()
        try:
            await gate.admit(gate.compat_key("chat", bool(req.stream), sp.temperature == 0.0, bool(sp.logprobs),
                                             bool(getattr(sp, "json_schema", None) or getattr(sp, "grammar", None))))
        except BaseException:
            gate.leave()
            raise
        metrics.inc("hipengine_requests_total", route="chat")

        def finish_session(msg: Dict[str, Any]) -> Optional[str]:
            if sid is not None:
                sessions.append(sid, new_msgs, msg)
                return sid
            if isinstance(req.session, dict) and req.session.get("create"):
                s = sessions.create(new_msgs + [msg])
                return s.id
            return None

        if req.stream and req.n == 1:
            greq, eng = stream_request(prompt_ids, sp)
            opts = req.stream_options
            timing = SE.StreamTimingTracker()

            async def gen():
                bridge = _Bridge(lambda: eng.stream(greq), cfg.stream_queue_max_chunks)
                dec = t.stream_decoder()
                parser = ChatStreamParser(plan.starts_in_think, parse_tools=bool(plan.tools))
                n_out = cached = think_tokens = 0
                full_text = ""
                final_reason = None
                sent_role = False
                try:
                    async for ch in bridge:
                        if await request.is_disconnected():
                            eng.cancel(greq.request_id, wait=False)
                            break
                        if ch.error:
                            yield SE.sse(APIError(classify_engine_error(ch.error), ch.error).body())
                            break
                        piece = dec.feed(ch.token_ids) + (dec.flush() if ch.finished else "")
                        full_text += piece
                        n_out += len(ch.token_ids)
                        timing.on_tokens(len(ch.token_ids))
                        if not sent_role:
                            sent_role = True
                            yield SE.sse(SE.chat_chunk(cid, cfg.served_model_name, created, {"role": "assistant", "content": ""}))
                        for phase, delta in parser.feed(piece, final=ch.finished):
                            if phase == "think":
                                d = {"reasoning_content": delta}
                                think_tokens += len(ch.token_ids)
                            elif phase == "answer":
                                d = {"content": delta}
                            else:
                                d = {"tool_calls": [delta]}
                            extra = None
                            if opts and opts.include_hipengine:
                                extra = dict(timing.block(), phase=phase, tokens=n_out)
                            lp = _lp_chat(ch.logprobs, t) if phase == "answer" else None
                            yield SE.sse(SE.chat_chunk(cid, cfg.served_model_name, created, d, 0, None, lp, extra))
                        if ch.finished:
                            final_reason = ch.finish.openai_reason
                            if ch.telemetry is not None:
                                cached = ch.telemetry.cached_prompt_tokens
                    if final_reason is not None:
                        parsed = parse_chat_output(full_text, plan.starts_in_think, bool(plan.tools))
                        try:
                            parsed, details = apply_result_policy(parsed, plan)
                        except APIError as exc:
                            yield SE.sse(exc.body())
                            details = {"reason": exc.code}
                        if parser.calls and not details:
                            final_reason = "tool_calls"
                        last = SE.chat_chunk(cid, cfg.served_model_name, created, {}, 0, final_reason, None,
                                             dict(timing.block(), phase="done", tokens=n_out)
                                             if opts and opts.include_hipengine else None)
                        if details:
                            last["choices"][0]["finish_details"] = details
                        new_sid = finish_session(_assistant_message(parsed, details))
                        if new_sid:
                            last["session"] = {"id": new_sid}
                        yield SE.sse(last)
                    if opts and opts.include_usage:
                        acc = SE.StreamTokenAccounting(len(prompt_ids), n_out, cached, think_tokens)
                        yield SE.sse(SE.usage_chunk(cid, cfg.served_model_name, created, "chat.completion.chunk", acc.usage()))
                    yield SE.SSE_DONE
                finally:
                    bridge.close()
                    gate.leave()
                    metrics.inc("hipengine_generated_tokens_total", n_out)
                    replay_outcome(cid, t_req, final_reason, len(prompt_ids), n_out)
            return StreamingResponse(gen(), media_type="text/event-stream")

        try:
            outs = await run_blocking(llm.generate_detailed, [prompt_ids] * req.n, [sp] * req.n)
        finally:
            gate.leave()
        choices = []
        for i, o in enumerate(outs):
            raise_for_output(o)
            parsed = parse_chat_output(o.text or "", plan.starts_in_think, bool(plan.tools))
            parsed, details = apply_result_policy(parsed, plan)
            msg = _assistant_message(parsed, details)
            reason = "tool_calls" if msg.get("tool_calls") else o.finish_reason
            choice: Dict[str, Any] = {"index": i, "message": msg, "finish_reason": reason}
            if req.logprobs:
                choice["logprobs"] = _lp_chat(o.logprobs, t)
            if details:
                choice["finish_details"] = details
            choices.append(choice)
            if sp.speculative_mtp:
                breaker.record(cfg.served_model_name, len(prompt_ids), ok=True)
        metrics.inc("hipengine_generated_tokens_total", sum(len(o.token_ids) for o in outs))
        body = {"id": cid, "object": "chat.completion", "created": created, "model": cfg.served_model_name,
                "choices": choices, "usage": _usage(outs)}
        replay_outcome(cid, t_req, choices[0]["finish_reason"] if choices else None, body["usage"]["prompt_tokens"],
                       body["usage"]["completion_tokens"])
        new_sid = finish_session(choices[0]["message"])
        if new_sid:
            body["session"] = {"id": new_sid}
        if req.stream:   # buffered SSE for n > 1
            async def buffered():
                for c in choices:
                    yield SE.sse(SE.chat_chunk(cid, cfg.served_model_name, created, c["message"], c["index"],
                                               c["finish_reason"]))
                yield SE.SSE_DONE
            return StreamingResponse(buffered(), media_type="text/event-stream")
        return body

    # ------------------------------------------------------------------ sessions
    @app.get("/v1/hipengine/sessions", dependencies=[Depends(auth)])
    async def list_sessions():
        return {"sessions": sessions.list()}

    @app.post("/v1/hipengine/sessions", dependencies=[Depends(auth)])
    async def create_session(body: Dict[str, Any]):
        s = sessions.create(body.get("messages") or [])
        return {"id": s.id}

    @app.delete("/v1/hipengine/sessions/{sid}", dependencies=[Depends(auth)])
    async def delete_session(sid: str):
        return {"deleted": sessions.delete(sid)}

    @app.post("/v1/hipengine/sessions/{sid}/fork", dependencies=[Depends(auth)])
    async def fork_session(sid: str):
        return {"id": sessions.fork(sid).id, "parent": sid}

    @app.post("/v1/hipengine/sessions/{sid}/rollback", dependencies=[Depends(auth)])
    async def rollback_session(sid: str, body: Optional[Dict[str, Any]] = None):
        turns = (body or {}).get("turns", 1)
        if isinstance(turns, bool) or not isinstance(turns, int) or turns < 0:
            raise APIError("unsupported_parameter", "turns must be a non-negative integer", "turns")
        s = sessions.rollback(sid, turns)
        return {"id": s.id, "turns": s.turns, "messages": len(s.messages)}

    @app.get("/v1/hipengine/sessions/{sid}/snapshot", dependencies=[Depends(auth)])
    async def export_session(sid: str):
        return sessions.export(sid, {"vocab_size": getattr(tok(), "vocab_size", None)})

    @app.post("/v1/hipengine/sessions/restore", dependencies=[Depends(auth)])
    async def restore_session(doc: Dict[str, Any]):
        s = sessions.restore(doc, {"vocab_size": getattr(tok(), "vocab_size", None)})
        return {"id": s.id, "turns": s.turns}

    return app
