"""FastAPI TestClient over the real engine on the CPU reference backend (tiny random-init model)."""
import json

import pytest

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402

from hipengine_b200 import LLM  # noqa: E402
from hipengine_b200.loading.synth import build_random_model  # noqa: E402
from hipengine_b200.models.config import TINY_DENSE  # noqa: E402
from hipengine_b200.server.api import ServerConfig, create_app  # noqa: E402


@pytest.fixture(scope="module")
def client():
    w = build_random_model(TINY_DENSE, seed=0)
    llm = LLM(w, backend="cpu_reference", max_active_requests=4, max_sequence_length=512)
    app = create_app(llm, ServerConfig(served_model_name="tiny", api_key="k", metrics="prometheus",
                                       chat_default_max_tokens=12))
    with TestClient(app) as c:
        c.headers.update({"Authorization": "Bearer k"})
        yield c


def _sse(resp):
    out = []
    for line in resp.iter_lines():
        if line.startswith("data: "):
            d = line[6:]
            out.append(d if d == "[DONE]" else json.loads(d))
    return out


def test_health_ready_models_auth(client):
    assert client.get("/health").json() == {"status": "ok"}
    r = client.get("/ready")
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "hipengine.readiness" and body["ready"] is True and body["status"] == "ready"
    for key in ("engine_service", "model", "startup", "context", "kv_capacity", "prefix_cache", "graph_cache",
                "queue", "batcher", "sessions", "parallelism", "diagnostics"):
        assert key in body, key
    assert "kv_capability" in body["model"] and "stages" in body["startup"]
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    r = client.get("/v1/models", headers={"Authorization": "Bearer wrong"})
    assert r.status_code == 401 and r.json()["error"]["code"] == "unauthorized"
    r = client.post("/v1/completions", json={"model": "other", "prompt": "hi"})
    assert r.status_code == 404 and r.json()["error"]["hipengine"]["code"] == "model_unavailable"


def test_completions_shapes_and_logprobs(client):
    r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0, "logprobs": 2,
                                             "ignore_eos": True})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "text_completion"
    ch = body["choices"][0]
    assert ch["finish_reason"] == "length" and len(ch["logprobs"]["tokens"]) == 5
    assert body["usage"]["completion_tokens"] == 5 and body["usage"]["prompt_tokens"] == 5
    r = client.post("/v1/completions", json={"prompt": ["a", "b"], "n": 2, "max_tokens": 2, "temperature": 0})
    assert len(r.json()["choices"]) == 4
    r = client.post("/v1/completions", json={"prompt": [1, 2, 3], "max_tokens": 2, "echo": True, "temperature": 0})
    assert r.status_code == 200


def test_completion_streaming_matches_blocking(client):
    req = {"prompt": "stream me", "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    full = client.post("/v1/completions", json=req).json()["choices"][0]["text"]
    with client.stream("POST", "/v1/completions", json=dict(req, stream=True,
                                                            stream_options={"include_usage": True})) as r:
        ev = _sse(r)
    assert ev[-1] == "[DONE]"
    text = "".join(e["choices"][0]["text"] for e in ev[:-1] if e.get("choices"))
    assert text == full
    assert ev[-2]["choices"] == [] and ev[-2]["usage"]["completion_tokens"] == 6


def test_chat_completion_and_stream(client):
    req = {"messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "hi"}], "max_tokens": 8,
           "temperature": 0, "enable_thinking": False, "ignore_eos": True}
    r = client.post("/v1/chat/completions", json=req)
    body = r.json()
    assert r.status_code == 200 and body["choices"][0]["message"]["role"] == "assistant"
    with client.stream("POST", "/v1/chat/completions", json=dict(req, stream=True,
                       stream_options={"include_usage": True, "include_hipengine": True})) as r2:
        ev = _sse(r2)
    assert ev[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(e["choices"][0]["delta"].get("content", "") for e in ev if isinstance(e, dict) and e.get("choices"))
    assert text.strip() == (body["choices"][0]["message"]["content"] or "").strip()
    finals = [e for e in ev if isinstance(e, dict) and e.get("choices") and e["choices"][0]["finish_reason"]]
    assert finals and finals[-1]["choices"][0]["finish_reason"] == "length"
    assert finals[-1]["hipengine"]["phase"] == "done"


def test_chat_validation_errors(client):
    r = client.post("/v1/chat/completions", json={"messages": []})
    assert r.status_code == 400
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "grammar": "root ::= x"})
    assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported_parameter"
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "tool", "content": "x"}]})
    assert r.status_code == 400
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "top_logprobs": 3})
    assert r.status_code == 400
    r = client.post("/v1/completions", json={"prompt": "x" * 600, "max_tokens": 50})
    assert r.status_code == 400 and r.json()["error"]["code"] == "context_overflow"


def test_structured_output_violation_is_reported(client):
    r = client.post("/v1/chat/completions", json={
        "messages": [{"role": "user", "content": "json please"}], "max_tokens": 6, "temperature": 0,
        "enable_thinking": False,
        "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "object", "required": ["a"]}}}})
    ch = r.json()["choices"][0]
    assert r.status_code == 200
    # a random-init model does not emit valid JSON: the server must say so instead of returning garbage
    assert ch["finish_details"]["reason"] == "schema_violation" and not ch["message"]["content"]


def test_tools_required_not_satisfied(client):
    tools = [{"type": "function", "function": {"name": "get_time", "parameters": {"type": "object"}}}]
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "time?"}], "tools": tools,
                                                  "tool_choice": "required", "max_tokens": 4, "temperature": 0,
                                                  "enable_thinking": False})
    # four tokens cannot hold a call: the grammar-forced opening is cut off by the length limit, which is reported as
    # an unsatisfied requirement or as an invalid (unterminated) call, never as a successful one
    ch = r.json()["choices"][0]
    assert ch["finish_details"]["reason"] in ("tool_required_not_satisfied", "invalid_tool_call")
    assert ch["finish_reason"] == "length" and not ch["message"].get("tool_calls")
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "tools": tools,
                                                  "tool_choice": {"type": "function", "function": {"name": "nope"}}})
    assert r.status_code == 400


def test_sessions_and_tokenize_and_metrics(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "a"}], "max_tokens": 3,
                                                  "temperature": 0, "session": {"create": True},
                                                  "enable_thinking": False})
    sid = r.json()["session"]["id"]
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "b"}], "max_tokens": 3,
                                                  "temperature": 0, "continuation_id": sid, "enable_thinking": False})
    assert r.status_code == 200
    lst = client.get("/v1/hipengine/sessions").json()["sessions"]
    assert any(s["id"] == sid and s["turns"] == 2 for s in lst)
    fork = client.post(f"/v1/hipengine/sessions/{sid}/fork").json()["id"]
    rb = client.post(f"/v1/hipengine/sessions/{fork}/rollback", json={"turns": 1}).json()
    assert rb["turns"] == 1
    snap = client.get(f"/v1/hipengine/sessions/{sid}/snapshot").json()
    assert snap["schema"].endswith("v1")
    assert client.post("/v1/hipengine/sessions/restore", json=snap).status_code == 200
    assert client.delete(f"/v1/hipengine/sessions/{sid}").json()["deleted"]
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "b"}], "continuation_id": sid})
    assert r.status_code in (400, 410)
    t = client.post("/v1/hipengine/tokenize", json={"text": "abc"}).json()
    assert client.post("/v1/hipengine/detokenize", json={"tokens": t["tokens"]}).json()["text"] == "abc"
    fit = client.post("/v1/hipengine/fit_context", json={"text": "abc"}).json()
    assert fit["fits"] and fit["object"] == "hipengine.fit_context" and fit["input_type"] == "text"
    mx = fit["max_context"]
    fit = client.post("/v1/hipengine/fit_context", json={"text": "abc", "max_tokens": mx - 3}).json()
    assert fit["fits_with_max_tokens"] and fit["prompt_tokens"] == 3 and fit["max_new_tokens"] == mx - 3
    assert not client.post("/v1/hipengine/fit_context", json={"text": "abc", "max_tokens": mx - 2}).json()["fits_with_max_tokens"]
    fit = client.post("/v1/hipengine/fit_context", json={"messages": [{"role": "user", "content": "hi"}]}).json()
    assert fit["input_type"] == "chat" and fit["chat_default_max_tokens"] > 0 and "fits_with_default_max_tokens" in fit
    assert client.post("/v1/hipengine/fit_context", json={"text": "abc", "max_tokens": 0}).status_code == 400
    m = client.get("/metrics").text
    assert "hipengine_completion_tokens_total" in m and "hipengine_requests_total" in m
    assert "hipengine_generation_queue_depth" in m and "hipengine_request_completed_total" in m
    caps = client.get("/v1/hipengine/capabilities").json()
    assert caps["features"]["tools"] and caps["limits"]["top_logprobs"] == 20


def test_generation_batcher_groups_compatible_requests_within_the_window():
    """Requests of one compatibility class that arrive inside the batch window are released together; another class
    gets its own release; a full group is released at once; drain releases what is held."""
    import asyncio
    from hipengine_b200.server.batcher import GenerationBatcher
    from hipengine_b200.server.errors import APIError

    async def run():
        b = GenerationBatcher(limit=8, window_ms=80.0, max_batch=3)
        k_greedy = b.compat_key("chat", False, True, False, False)
        k_sampled = b.compat_key("chat", False, False, False, False)
        released = []

        async def one(name, key, delay):
            await asyncio.sleep(delay)
            b.enter()
            await b.admit(key)
            released.append((name, round(asyncio.get_running_loop().time(), 2)))
            b.leave()

        t0 = asyncio.get_running_loop().time()
        await asyncio.gather(one("a", k_greedy, 0.0), one("b", k_greedy, 0.02), one("s", k_sampled, 0.03))
        times = dict(released)
        assert abs(times["a"] - times["b"]) < 0.02 and times["a"] - t0 >= 0.07        # held, released together
        assert times["s"] - t0 >= 0.10                                                  # its own window
        snap = b.snapshot()
        assert snap["batches"] == 2 and snap["max_batch_seen"] == 2 and snap["flush_window"] == 2
        # a full group does not wait for the window
        t1 = asyncio.get_running_loop().time()
        await asyncio.gather(*[one(f"f{i}", k_greedy, 0.0) for i in range(3)])
        assert asyncio.get_running_loop().time() - t1 < 0.05 and b.snapshot()["flush_full"] == 1
        # bound + drain
        for _ in range(8):
            b.enter()
        try:
            b.enter()
            raise AssertionError("expected engine_busy")
        except APIError as exc:
            assert exc.code == "engine_busy"
        held = asyncio.ensure_future(b.admit(k_greedy))
        await asyncio.sleep(0.01)
        b.drain()
        await asyncio.wait_for(held, 0.5)
        assert b.snapshot()["flush_drain"] == 1 and b.closing

    asyncio.run(run())


def test_replica_router_balances_sticks_to_prefixes_and_fails_over():
    """Two in-process replica servers (CPU reference backend) behind the router: requests with the same prompt prefix
    land on the same replica, others spread by load, a dead replica is taken out of rotation."""
    import threading
    import time

    import requests
    import uvicorn

    from hipengine_b200.llm import LLM
    from hipengine_b200.server.api import ServerConfig, create_app
    from hipengine_b200.server.router import Router, create_router_app, prompt_key

    assert prompt_key({"prompt": "x" * 10}) is None and prompt_key({"prompt": "y" * 600}) == prompt_key({"prompt": "y" * 700})
    servers, llms = [], []

    def serve(app, port):
        srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
        threading.Thread(target=srv.run, daemon=True).start()
        for _ in range(200):
            if srv.started:
                break
            time.sleep(0.05)
        servers.append(srv)
        return srv

    try:
        for port in (8061, 8062):
            llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=1024)
            llms.append(llm)
            serve(create_app(llm, ServerConfig(served_model_name="tiny-dense")), port)
        router = Router(["http://127.0.0.1:8061", "http://127.0.0.1:8062", "http://127.0.0.1:8069"], backoff_s=60.0)
        serve(create_router_app(router), 8060)
        base = "http://127.0.0.1:8060"
        assert requests.get(base + "/health").json()["replicas"] == 3
        shared = "p" * 600
        for i in range(4):                                   # same prefix -> same replica
            r = requests.post(base + "/v1/completions", json={"model": "tiny-dense", "prompt": shared + str(i),
                                                              "max_tokens": 2, "temperature": 0.0})
            assert r.status_code == 200 and r.json()["choices"][0]["text"] is not None
        served = [rep.served for rep in router.replicas]
        assert sorted(served)[-1] == 4 and router.stats["affinity_hits"] == 3
        for i in range(4):                                   # distinct prompts spread; the dead replica is skipped
            r = requests.post(base + "/v1/completions", json={"model": "tiny-dense", "prompt": chr(65 + i) * 700,
                                                              "max_tokens": 2, "temperature": 0.0})
            assert r.status_code == 200
        assert router.replicas[2].served == 0 and router.replicas[2].failed >= 1
        assert min(router.replicas[0].served, router.replicas[1].served) >= 2
        # streaming passes through
        with requests.post(base + "/v1/completions", json={"model": "tiny-dense", "prompt": "z" * 100, "max_tokens": 3,
                                                            "stream": True}, stream=True) as r:
            lines = [l for l in r.iter_lines() if l.startswith(b"data: ")]
        assert lines[-1] == b"data: [DONE]" and len(lines) >= 2
        ready = requests.get(base + "/ready")
        assert ready.status_code == 200 and ready.json()["ready_replicas"] == 2
        # a chat session lives in ONE replica: the router learns its owner from the creating response (blocking and
        # streamed) and pins every later request that names it, whatever the load says
        chat = {"model": "tiny-dense", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 2,
                "enable_thinking": False}
        sids = [requests.post(base + "/v1/chat/completions", json=dict(chat, session={"create": True})).json()["session"]["id"]]
        with requests.post(base + "/v1/chat/completions", json=dict(chat, session={"create": True}, stream=True),
                           stream=True) as r:
            text = b"".join(r.iter_content(None)).decode()
        sids.append(text.split('"session":{"id":"')[1].split('"')[0])
        sids.append(requests.post(base + f"/v1/hipengine/sessions/{sids[0]}/fork").json()["id"])
        assert all(s in router.session_owner for s in sids)
        assert router.session_owner[sids[2]] == router.session_owner[sids[0]]
        for s in sids * 3:
            r = requests.post(base + "/v1/chat/completions", json=dict(chat, session=s))
            assert r.status_code == 200 and r.json()["session"]["id"] == s, r.text
        assert router.stats["session_pins"] >= 9
        listed = requests.get(base + "/v1/hipengine/sessions").json()["sessions"]
        assert {e["id"] for e in listed} >= set(sids) and all(e["replica"].startswith("http://127.0.0.1:806") for e in listed)
        assert requests.delete(base + f"/v1/hipengine/sessions/{sids[1]}").json()["deleted"]
        # an unserved feature is the replica's ANSWER: passed through, the replica stays in rotation
        failed = [rep.failed for rep in router.replicas]
        r = requests.post(base + "/v1/audio/songs", json={"model": "tiny-dense", "lyrics": "la"})
        assert r.status_code == 501 and r.json()["error"]["code"] == "unsupported_feature"
        assert [rep.failed for rep in router.replicas] == failed
        assert requests.post(base + "/v1/completions", json={"model": "tiny-dense", "prompt": "ok", "max_tokens": 1}).status_code == 200
        # nothing left to route to: the envelope, not a bare message
        for rep in router.replicas:
            rep.down_until = time.time() + 60
        r = requests.post(base + "/v1/completions", json={"model": "tiny-dense", "prompt": "ok", "max_tokens": 1})
        assert r.status_code == 502 and r.json()["error"]["code"] == "routing_failed" and r.json()["error"]["hipengine"]["retryable"]
    finally:
        for s in servers:
            s.should_exit = True
        for l in llms:
            l.close()


def test_replay_log_records_requests_with_redaction(tmp_path):
    """--replay-dir writes one JSON line per admitted request and one per outcome; with the default redaction the
    prompt text is replaced by a hash and its length."""
    import json
    from fastapi.testclient import TestClient
    from hipengine_b200.llm import LLM
    from hipengine_b200.server.api import ServerConfig, create_app
    from hipengine_b200.server.__main__ import build_parser, configs_from_args
    a = build_parser().parse_args(["--model", "tiny-dense", "--replay-dir", str(tmp_path), "--generation-batch-window-ms", "2",
                                   "--kv-pool-memory-budget-mib", "64", "--startup-min-free-mib", "128", "--quant", "Q4_K"])
    eng_cfg, srv_cfg = configs_from_args(a)
    assert srv_cfg.replay_dir == str(tmp_path) and srv_cfg.batch_window_ms == 2.0
    assert eng_cfg.kv.pool_budget_mib == 64 and eng_cfg.kv.memory_reserve_mib == 128
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=256)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="tiny-dense", replay_dir=str(tmp_path)))) as c:
            r = c.post("/v1/completions", json={"model": "tiny-dense", "prompt": "a secret prompt", "max_tokens": 3,
                                                "temperature": 0.0})
            assert r.status_code == 200
            r = c.post("/v1/chat/completions", json={"model": "tiny-dense", "max_tokens": 3,
                                                     "messages": [{"role": "user", "content": "another secret"}]})
            assert r.status_code == 200
        lines = []
        for f in tmp_path.iterdir():
            lines += [json.loads(l) for l in f.read_text().splitlines()]
        kinds = [l["kind"] for l in lines]
        assert kinds.count("request") == 2 and kinds.count("outcome") == 2
        text = json.dumps(lines)
        assert "secret" not in text and "sha256" in text
        out = [l for l in lines if l["kind"] == "outcome"][0]
        assert out["completion_tokens"] == 3 and out["prompt_tokens"] > 0
    finally:
        llm.close()


def test_pool_budget_and_expected_quant_in_admission():
    from hipengine_b200.config import EngineConfig, KVConfig, resolve_pool_pages
    from dataclasses import replace
    kv = KVConfig(pool_budget_mib=64)
    assert resolve_pool_pages(kv, kv_bytes_per_token=4096, n_slots=4, pages_per_slot=64) == 64 * (1 << 20) // (16 * 4096) + 1
    assert resolve_pool_pages(replace(kv, pool_pages=77), 4096, 4, 64) == 77
    import pytest
    from hipengine_b200.loading.admission import ArtifactRejected, admit
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_DENSE
    w = build_random_model(TINY_DENSE, seed=0)
    rep = admit(w, EngineConfig.from_env(), free_bytes=10 ** 12, expected_quant=None)
    with pytest.raises(ArtifactRejected, match="expected"):
        admit(w, EngineConfig.from_env(), free_bytes=10 ** 12, expected_quant="Q2_K")
    assert admit(w, EngineConfig.from_env(), free_bytes=10 ** 12, expected_quant=rep["dominant_block_type"])["admitted"]


class _InProcessTransport:
    """The chat client's transport over a FastAPI TestClient (no sockets)."""

    def __init__(self, client):
        self.c = client

    def get(self, path):
        return self.c.get(path).json()

    def stream(self, path, body):
        with self.c.stream("POST", path, json=body) as r:
            assert r.status_code == 200, r.read()
            for line in r.iter_lines():
                if line.startswith("data: "):
                    yield line[6:]


def test_chat_client_streams_turns_keeps_the_transcript_and_reports_server_side_stats(tmp_path):
    import io
    import json
    from fastapi.testclient import TestClient
    from hipengine_b200.chat_cli import ChatClient, Settings, run_repl
    from hipengine_b200.llm import LLM
    from hipengine_b200.server.api import ServerConfig, create_app
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=512)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="tiny-dense"))) as tc:
            c = ChatClient(_InProcessTransport(tc), settings=Settings(max_tokens=6, temperature=0.0, think=False))
            assert c.discover_model() == "tiny-dense"
            pieces = list(c.stream_turn("hello there"))
            assert pieces and all(p.kind in ("content", "reasoning", "tool_call") for p in pieces)
            st = c.last
            assert st.completion_tokens == 6 and st.prompt_tokens > 0 and st.finish_reason == "length"
            assert st.ttft_ms is not None and st.decode_tok_s is not None and "tok/s" in st.line()
            assert [m["role"] for m in c.messages] == ["user", "assistant"]
            b = c.bench(2)
            assert b["turns"] == 2 and b["completion_tokens"] == 12 and b["ttft_ms_median"] is not None
            assert [m["role"] for m in c.messages] == ["user", "assistant"]          # bench leaves the transcript
            assert c.usage.turns == 3
            # the command loop: settings, a turn, retry, undo, save, status, unknown command
            out = io.StringIO()
            f = tmp_path / "t.json"
            rc = run_repl(c, ["/max 4", "/system be brief", "second question", "/retry", "/undo", "/usage",
                              f"/save {f}", "/status", "/nope", "/max x", "/quit", "never reached"], out)
            text = out.getvalue()
            assert rc == 0 and text.count("tok/s") == 2                                # the turn and its retry
            assert "unknown command" in text and "error:" in text and "never reached" not in text
            assert c.settings.max_tokens == 4 and c.settings.system == "be brief" and c.last.completion_tokens == 4
            saved = json.loads(f.read_text())
            assert saved["system"] == "be brief" and [m["role"] for m in saved["messages"]] == ["user", "assistant"]
            assert '"status"' in text or '"ready"' in text or '"engine"' in text
    finally:
        llm.close()


def _png(w, h):
    import struct
    import zlib
    ihdr = struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)
    chunk = lambda t, d: struct.pack(">I", len(d)) + t + d + struct.pack(">I", zlib.crc32(t + d))
    return b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", ihdr) + chunk(b"IDAT", zlib.compress(b"\0" * 4)) + chunk(b"IEND", b"")


def test_media_parts_are_parsed_under_limits_and_refused_by_the_text_only_server():
    import base64
    import struct
    from fastapi.testclient import TestClient
    from hipengine_b200.llm import LLM
    from hipengine_b200.server.api import ServerConfig, create_app
    from hipengine_b200.server.multimodal import MediaError, MediaLimits, extract_media, sniff_image
    url = lambda raw, mime="image/png": f"data:{mime};base64," + base64.b64encode(raw).decode()
    msg = lambda *parts: [{"role": "user", "content": list(parts)}]
    img = lambda u: {"type": "image_url", "image_url": {"url": u}}
    got = extract_media(msg({"type": "text", "text": "what is this"}, img(url(_png(640, 480)))))
    assert [(m.kind, m.mime, m.width, m.height, m.part_index) for m in got] == [("image", "image/png", 640, 480, 1)]
    gif = b"GIF89a" + struct.pack("<HH", 12, 7) + b"\0" * 8
    jpg = b"\xff\xd8\xff\xe0\x00\x10JFIF\0" + b"\0" * 9 + b"\xff\xc0\x00\x11\x08" + struct.pack(">HH", 30, 40) + b"\0" * 12
    assert sniff_image(gif) == ("image/gif", 12, 7) and sniff_image(jpg) == ("image/jpeg", 40, 30)
    assert sniff_image(b"not an image at all") == (None, None, None)
    for bad, needle in [
        (img("https://example.com/cat.png"), "not fetched"),
        (img(url(_png(640, 480), "image/jpeg")), "does not match"),
        (img("data:image/png;base64,@@@@"), "not valid base64"),
        (img(url(_png(70000, 10))), "exceeds the limit"),
        (img(url(b"plain text", "image/png")), "unrecognised image"),
        ({"type": "image_url"}, "no URL"),
    ]:
        with pytest.raises(MediaError, match=needle) as ei:
            extract_media(msg(bad))
        assert ei.value.param == "messages[0].content[0]"
    with pytest.raises(MediaError, match="more than 2 media parts"):
        extract_media(msg(*[img(url(_png(8, 8)))] * 3), MediaLimits(max_parts=2))
    with pytest.raises(MediaError, match="exceeds 64 bytes"):
        extract_media(msg(img(url(_png(8, 8) + b"\0" * 100))), MediaLimits(max_image_bytes=64))
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=256)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="tiny-dense"))) as c:
            body = {"model": "tiny-dense", "max_tokens": 3, "messages": msg({"type": "text", "text": "hi"},
                                                                           img(url(_png(32, 32))))}
            r = c.post("/v1/chat/completions", json=body)
            assert r.status_code == 501, r.text
            e = r.json()["error"]
            assert e["code"] == "unsupported_feature" and e["param"] == "messages[0].content[1]"
            assert e["hipengine"]["media"][0]["width"] == 32
            body["messages"] = msg(img("http://10.0.0.1/x.png"))
            r = c.post("/v1/chat/completions", json=body)
            assert r.status_code == 400 and "not fetched" in r.json()["error"]["message"]
            body["messages"] = msg({"type": "text", "text": "text parts alone are fine"})
            assert c.post("/v1/chat/completions", json=body).status_code == 200
    finally:
        llm.close()


def test_router_retries_a_failed_request_elsewhere_and_lets_the_last_failure_stand():
    """Stand-in replicas: one answers 500 to every generation request, one answers 200.  The router retries the 500 on
    the other replica and keeps the failing one in rotation (its /ready decides, not one failed request); when every
    replica fails, the client gets the last replica's own error body, not a routing error."""
    import threading
    import time

    import requests
    import uvicorn
    from fastapi import FastAPI
    from fastapi.responses import JSONResponse

    from hipengine_b200.server.errors import APIError
    from hipengine_b200.server.router import Router, create_router_app, session_of

    assert session_of("/v1/hipengine/sessions/sess_ab12/fork", {}) == "sess_ab12"
    assert session_of("/v1/chat/completions", {"session": {"id": "sess_1"}}) == "sess_1"
    assert session_of("/v1/chat/completions", {"continuation_id": "sess_2"}) == "sess_2"
    assert session_of("/v1/chat/completions", {"session": {"create": True}}) is None
    mode = {"good_fails": False}
    bad, good = FastAPI(), FastAPI()

    @bad.post("/v1/completions")
    async def _bad():
        return JSONResponse(APIError("execution_failed", "device fault on replica A").body(), status_code=500)

    @good.post("/v1/completions")
    async def _good():
        if mode["good_fails"]:
            return JSONResponse(APIError("execution_failed", "device fault on replica B").body(), status_code=500)
        return {"choices": [{"text": "fine"}]}

    servers = []
    try:
        for app, port in ((bad, 8071), (good, 8072)):
            srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
            threading.Thread(target=srv.run, daemon=True).start()
            servers.append(srv)
        router = Router(["http://127.0.0.1:8071", "http://127.0.0.1:8072"], backoff_s=60.0)
        srv = uvicorn.Server(uvicorn.Config(create_router_app(router), host="127.0.0.1", port=8070, log_level="warning"))
        threading.Thread(target=srv.run, daemon=True).start()
        servers.append(srv)
        for _ in range(200):
            if all(s.started for s in servers):
                break
            time.sleep(0.05)
        for _ in range(4):
            r = requests.post("http://127.0.0.1:8070/v1/completions", json={"prompt": "x"})
            assert r.status_code == 200 and r.json()["choices"][0]["text"] == "fine"
        assert router.stats["retries"] >= 1 and router.replicas[0].failed >= 1
        assert router.replicas[0].available(time.time())                   # still in rotation
        mode["good_fails"] = True
        r = requests.post("http://127.0.0.1:8070/v1/completions", json={"prompt": "x"})
        assert r.status_code == 500 and r.json()["error"]["code"] == "execution_failed"
        assert "device fault on replica" in r.json()["error"]["message"]
    finally:
        for s in servers:
            s.should_exit = True
