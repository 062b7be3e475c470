"""Data-parallel serving: one HTTP front in front of N replica servers (one engine per GPU, or one tensor-parallel
group per replica).

    python -m hipengine_b200.server --model M --port 8001 &      # replica on GPU 0 (CUDA_VISIBLE_DEVICES=0)
    python -m hipengine_b200.server --model M --port 8002 &      # replica on GPU 1 ...
    python -m hipengine_b200.server.router --backends http://127.0.0.1:8001,http://127.0.0.1:8002 --port 8000

Routing: a request whose prompt starts like an earlier one goes to the replica that served that prefix (so the
replica's radix prefix cache hits); otherwise to the replica with the fewest requests in flight.  Replicas that fail a
request or their `/ready` probe are taken out of rotation and probed again after a back-off.  Responses are streamed
through unchanged (SSE included).  `/health`, `/ready`, `/v1/models` and `/metrics` of the router aggregate the
replicas'.  The reference serves one model per process and leaves replication to an external balancer; this is that
balancer, prefix-aware, in-tree.

Chat sessions are transcripts held by ONE replica, so the router pins them: it learns a session's owner from the
response that created it (``"id": "sess_..."`` in a chat response asked to create one, or in the answer of the
session routes), sends every later request that names the session (``session``, ``continuation_id``, the session
routes) to that replica, and merges the replicas' session lists.  A replica that answers 5xx is not what the request
asked for: 500 / 502 / 504 are retried on another replica (nothing was streamed yet) without taking the replica out of
rotation, 501 and 503 pass through (an unserved feature or a busy queue is the answer); a replica that cannot be
reached, or whose ``/ready`` fails, is taken out until the back-off ends.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import re
import time
from collections import OrderedDict
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

PREFIX_CHARS = 512           # how much of the prompt identifies "the same prefix"
AFFINITY_ENTRIES = 4096
SESSION_ENTRIES = 65536
_SESSION_ID = re.compile(rb'"id":\s*"(sess_[0-9a-f]{8,64})"')
_SESSION_PATH = re.compile(r"^/v1/hipengine/sessions/(sess_[0-9a-f]+)")
RETRY_ELSEWHERE = (500, 502, 504)


def session_of(path: str, body: Any) -> Optional[str]:
    """The chat session a request names (in its path or its body), or None."""
    m = _SESSION_PATH.match(path)
    if m:
        return m.group(1)
    if isinstance(body, dict):
        if isinstance(body.get("continuation_id"), str):
            return body["continuation_id"]
        sess = body.get("session")
        if isinstance(sess, str):
            return sess
        if isinstance(sess, dict) and isinstance(sess.get("id"), str):
            return sess["id"]
    return None


def may_name_a_new_session(path: str, body: Any) -> bool:
    """Will the response carry the id of a session this replica now owns (created, forked, restored, continued)?"""
    return path.startswith("/v1/hipengine/sessions") or (isinstance(body, dict) and body.get("session") is not None)


class Replica:
    def __init__(self, url: str):
        self.url = url.rstrip("/")
        self.in_flight = 0
        self.served = 0
        self.failed = 0
        self.down_until = 0.0

    def available(self, now: float) -> bool:
        return now >= self.down_until

    def snapshot(self) -> Dict[str, Any]:
        return {"url": self.url, "in_flight": self.in_flight, "served": self.served, "failed": self.failed,
                "down": self.down_until > time.time()}


def prompt_key(body: Dict[str, Any]) -> Optional[str]:
    """Stable key of the leading part of a request's prompt (chat messages, text or token ids)."""
    if "messages" in body:
        text = json.dumps(body["messages"], sort_keys=True)[:PREFIX_CHARS * 2]
    elif "prompt" in body:
        p = body["prompt"]
        text = (p if isinstance(p, str) else json.dumps(p))[:PREFIX_CHARS * 2]
    else:
        return None
    if len(text) < 64:
        return None
    return hashlib.sha1(text[:PREFIX_CHARS].encode()).hexdigest()


class Router:
    def __init__(self, backends: List[str], backoff_s: float = 5.0):
        if not backends:
            raise ValueError("at least one backend")
        self.replicas = [Replica(u) for u in backends]
        self.affinity: "OrderedDict[str, int]" = OrderedDict()
        self.session_owner: "OrderedDict[str, int]" = OrderedDict()
        self.backoff_s = backoff_s
        self.stats = {"routed": 0, "affinity_hits": 0, "session_pins": 0, "retries": 0, "no_replica": 0}

    def own(self, sid: str, i: int) -> None:
        self.session_owner[sid] = i
        self.session_owner.move_to_end(sid)
        while len(self.session_owner) > SESSION_ENTRIES:
            self.session_owner.popitem(last=False)

    def learn_sessions(self, data: bytes, i: int) -> None:
        for m in _SESSION_ID.finditer(data):
            self.own(m.group(1).decode(), i)

    def pick(self, key: Optional[str], exclude: Optional[set] = None, session: Optional[str] = None) -> Optional[int]:
        now = time.time()
        ok = [i for i, r in enumerate(self.replicas) if r.available(now) and not (exclude and i in exclude)]
        if not ok:
            return None
        if session is not None and self.session_owner.get(session) in ok:
            self.stats["session_pins"] += 1
            return self.session_owner[session]
        if key is not None and key in self.affinity and self.affinity[key] in ok:
            self.affinity.move_to_end(key)
            self.stats["affinity_hits"] += 1
            return self.affinity[key]
        i = min(ok, key=lambda j: (self.replicas[j].in_flight, self.replicas[j].served))
        if key is not None:
            self.affinity[key] = i
            while len(self.affinity) > AFFINITY_ENTRIES:
                self.affinity.popitem(last=False)
        return i

    def mark_down(self, i: int) -> None:
        r = self.replicas[i]
        r.failed += 1
        r.down_until = time.time() + self.backoff_s
        for k in [k for k, v in self.affinity.items() if v == i]:
            self.affinity.pop(k, None)

    def snapshot(self) -> Dict[str, Any]:
        return {"replicas": [r.snapshot() for r in self.replicas], **self.stats,
                "affinity_entries": len(self.affinity), "pinned_sessions": len(self.session_owner)}


def create_router_app(router: Router):
    import aiohttp

    app = FastAPI(title="hipengine_b200 replica router")
    state: Dict[str, Any] = {"session": None}

    async def session() -> "aiohttp.ClientSession":
        if state["session"] is None:
            state["session"] = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None, sock_connect=5))
        return state["session"]

    async def _close() -> None:
        if state["session"] is not None:
            await state["session"].close()

    app.router.on_shutdown.append(_close)

    async def fan_out(path: str) -> List[Any]:
        s = await session()
        out: List[Any] = []
        for r in router.replicas:
            try:
                async with s.get(r.url + path) as resp:
                    ctype = resp.headers.get("content-type", "")
                    out.append((resp.status, await (resp.json() if "json" in ctype else resp.text())))
            except Exception as exc:
                out.append((599, {"error": str(exc)}))
        return out

    @app.get("/health")
    async def health():
        return {"status": "ok", "object": "hipengine.router.health", "replicas": len(router.replicas)}

    @app.get("/ready")
    async def ready():
        res = await fan_out("/ready")
        now = time.time()
        for i, (st, _b) in enumerate(res):
            if st != 200 and router.replicas[i].available(now):
                router.mark_down(i)
        n_ready = sum(1 for st, _ in res if st == 200)
        body = {"object": "hipengine.router.readiness", "ready": n_ready > 0, "ready_replicas": n_ready,
                "router": router.snapshot(), "replicas": [b for _, b in res]}
        return JSONResponse(body, status_code=200 if n_ready else 503)

    @app.get("/v1/models")
    async def models():
        for st, body in await fan_out("/v1/models"):
            if st == 200:
                return body
        return refusal("engine_unavailable", "no replica available")

    @app.get("/metrics")
    async def metrics():
        parts = [f"# replica {r.url}\n{b if isinstance(b, str) else ''}" for r, (st, b) in
                 zip(router.replicas, await fan_out("/metrics"))]
        snap = router.snapshot()
        head = "".join(f"hipengine_router_{k} {snap[k]}\n" for k in ("routed", "affinity_hits", "session_pins", "retries", "no_replica"))
        return PlainTextResponse(head + "\n".join(parts), media_type="text/plain; version=0.0.4")

    def refusal(code: str, message: str) -> JSONResponse:
        from .errors import APIError
        e = APIError(code, message)
        return JSONResponse(e.body(), status_code=e.status)

    async def forward(request: Request, path: str):
        raw = await request.body()
        try:
            body = json.loads(raw) if raw else {}
        except Exception:
            body = {}
        key = prompt_key(body) if isinstance(body, dict) else None
        sid = session_of(path, body)
        learn = may_name_a_new_session(path, body)
        headers = {k: v for k, v in request.headers.items() if k.lower() in ("authorization", "content-type")}
        tried: set = set()
        last_failure: Optional[tuple] = None
        s = await session()
        while True:
            i = router.pick(key, exclude=tried, session=sid)
            if i is None:
                if last_failure is not None:                  # every replica answered 5xx: the last answer stands
                    st, data, ctype = last_failure
                    return Response(content=data, status_code=st, media_type=ctype)
                router.stats["no_replica"] += 1
                return refusal("routing_failed", "no replica available")
            rep = router.replicas[i]
            rep.in_flight += 1
            try:
                resp = await s.request(request.method, rep.url + path, data=raw, headers=headers)
            except Exception:
                rep.in_flight -= 1
                router.mark_down(i)
                tried.add(i)
                router.stats["retries"] += 1
                continue
            if resp.status in RETRY_ELSEWHERE:
                # this replica failed the request (an engine failure, not "busy" and not "unserved"): nothing was
                # streamed yet, so another replica may serve it; the replica stays in rotation (its /ready decides)
                last_failure = (resp.status, await resp.read(), resp.headers.get("content-type", "application/json"))
                await resp.release()
                rep.in_flight -= 1
                rep.failed += 1
                tried.add(i)
                router.stats["retries"] += 1
                continue
            router.stats["routed"] += 1

            async def stream(resp=resp, rep=rep, i=i):
                tail = b""
                try:
                    async for chunk in resp.content.iter_any():
                        if learn and resp.status == 200:
                            router.learn_sessions(tail + chunk, i)        # an id may straddle two chunks
                            tail = chunk[-96:]
                        yield chunk
                    rep.served += 1
                finally:
                    rep.in_flight -= 1
                    await resp.release()

            return StreamingResponse(stream(), status_code=resp.status,
                                     media_type=resp.headers.get("content-type", "application/json"))

    @app.get("/v1/hipengine/sessions")
    async def list_sessions(request: Request):
        """Every replica's sessions in one list (each entry names its replica); owners are learned on the way."""
        hdr = {k: v for k, v in request.headers.items() if k.lower() == "authorization"}
        s = await session()
        merged: List[Any] = []
        for i, rep in enumerate(router.replicas):
            if not rep.available(time.time()):
                continue
            try:
                async with s.get(rep.url + "/v1/hipengine/sessions", headers=hdr) as resp:
                    if resp.status != 200:
                        continue
                    for ent in (await resp.json()).get("sessions", []):
                        router.own(str(ent.get("id")), i)
                        merged.append(dict(ent, replica=rep.url))
            except Exception:
                router.mark_down(i)
        return {"sessions": merged}

    @app.api_route("/v1/{rest:path}", methods=["POST", "GET", "DELETE"])
    async def v1(rest: str, request: Request):
        return await forward(request, "/v1/" + rest)

    return app


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="hipengine-b200 router", description=__doc__.split("\n\n")[0])
    ap.add_argument("--backends", required=True, help="comma-separated replica base URLs")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--backoff-seconds", type=float, default=5.0)
    a = ap.parse_args(argv)
    import uvicorn
    uvicorn.run(create_router_app(Router([u for u in a.backends.split(",") if u], a.backoff_seconds)), host=a.host,
                port=a.port, log_level="info")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
