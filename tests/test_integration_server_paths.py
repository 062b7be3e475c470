"""More HTTP paths over the real engine on the CPU reference backend: speculative decoding and its circuit breaker,
thinking budgets, several choices, echo, deadlines, per-event timing blocks."""
import json

import pytest

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402

from hipengine_b200 import LLM  # noqa: E402
from hipengine_b200.server.api import ServerConfig, create_app  # noqa: E402


def _sse(resp):
    out = []
    for line in resp.iter_lines():
        if line.startswith("data: "):
            d = line[6:]
            out.append(d if d == "[DONE]" else json.loads(d))
    return out


def test_speculative_decoding_over_http_equals_plain_and_is_counted():
    """A hybrid model with its NextN block behind the server on the host backend: `speculative_mtp: true` yields the
    same greedy text as a plain request, the cycles show in /metrics and in the live snapshot, and the operator
    endpoint of the circuit breaker answers."""
    llm = LLM("tiny-hybrid-mtp", backend="cpu_reference", max_active_requests=2, max_sequence_length=256,
              prefix_cache="off", speculative_mtp_serving="on", speculative_candidate_budget=3)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="hy", metrics="prometheus"))) as c:
            body = {"model": "hy", "prompt": list(range(9, 30)), "max_tokens": 9, "temperature": 0, "ignore_eos": True}
            plain = c.post("/v1/completions", json=body).json()
            spec = c.post("/v1/completions", json=dict(body, speculative_mtp=True)).json()
            assert plain["choices"][0]["text"] == spec["choices"][0]["text"]
            assert spec["usage"]["completion_tokens"] == 9
            chat = {"model": "hy", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0,
                    "enable_thinking": False, "speculative_mtp": True, "stream": True,
                    "stream_options": {"include_usage": True, "include_hipengine": True}}
            with c.stream("POST", "/v1/chat/completions", json=chat) as r:
                ev = _sse(r)
            assert ev[-1] == "[DONE]" and ev[-2]["usage"]["completion_tokens"] == 6
            blocks = [e["hipengine"] for e in ev[:-1] if isinstance(e, dict) and "hipengine" in e]
            assert blocks and blocks[-1]["phase"] == "done" and blocks[-1]["timing"]["ttft_ms"] is not None
            assert blocks[-1]["tokens"] == 6
            m = c.get("/metrics").text
            assert "hipengine_mtp_requests_total" in m and "hipengine_mtp_draft_tokens_rejected_total" in m
            runner = llm._get_engine().loop.runner
            assert runner.spec_stats["cycles"] >= 2
            caps = c.get("/v1/hipengine/capabilities").json()
            assert caps["features"]["speculative_mtp"] == "mtp" and "mtp_circuit_breaker" in caps
            assert "closed_scopes" in c.post("/v1/hipengine/speculative_mtp/rollback").json()
            snap = c.get("/v1/hipengine/decode").json()
            assert snap["counters"]["spec_cycles"] >= 2
    finally:
        llm.close()


@pytest.fixture(scope="module")
def client():
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=4, max_sequence_length=512)
    with TestClient(create_app(llm, ServerConfig(served_model_name="tiny", chat_default_max_tokens=10))) as c:
        yield c
    llm.close()


def test_thinking_budget_forces_the_close_sequence_and_splits_reasoning(client):
    """A random model never closes its thinking block by itself: the budget must force `</think>`; the reasoning part
    is reported apart from the answer and counted as reasoning tokens."""
    body = {"model": "tiny", "messages": [{"role": "user", "content": "why"}], "max_tokens": 40, "temperature": 0,
            "enable_thinking": True, "thinking_token_budget": 5, "ignore_eos": True}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    msg = r.json()["choices"][0]["message"]
    assert msg.get("reasoning_content") and "</think>" not in (msg.get("content") or "")
    assert "</think>" not in msg["reasoning_content"]
    with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True,
                                                                stream_options={"include_usage": True})) as r:
        ev = _sse(r)
    deltas = [e["choices"][0]["delta"] for e in ev if isinstance(e, dict) and e.get("choices")]
    assert any(d.get("reasoning_content") for d in deltas) and any(d.get("content") for d in deltas)
    first_answer = next(i for i, d in enumerate(deltas) if d.get("content"))
    assert not any(d.get("reasoning_content") for d in deltas[first_answer:])      # reasoning first, then the answer
    usage = ev[-2]["usage"]
    assert 0 < usage["completion_tokens_details"]["reasoning_tokens"] < usage["completion_tokens"] == 40
    off = client.post("/v1/chat/completions", json=dict(body, enable_thinking=False)).json()["choices"][0]["message"]
    assert not off.get("reasoning_content")
    none = client.post("/v1/chat/completions", json=dict(body, reasoning_effort="none")).json()["choices"][0]["message"]
    assert not none.get("reasoning_content")
    bad = client.post("/v1/chat/completions", json=dict(body, reasoning_effort="extreme"))
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "reasoning_effort"


def test_several_choices_echo_and_buffered_streams(client):
    r = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "x"}],
                                                  "max_tokens": 4, "n": 3, "temperature": 0.9, "seed": 1,
                                                  "enable_thinking": False})
    ch = r.json()["choices"]
    assert [c["index"] for c in ch] == [0, 1, 2] and r.json()["usage"]["completion_tokens"] == 12
    assert len({c["message"]["content"] for c in ch}) >= 2                      # rows are seeded apart
    again = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "x"}],
                                                      "max_tokens": 4, "n": 3, "temperature": 0.9, "seed": 1,
                                                      "enable_thinking": False}).json()["choices"]
    assert [c["message"]["content"] for c in again] == [c["message"]["content"] for c in ch]
    with client.stream("POST", "/v1/chat/completions",
                       json={"model": "tiny", "messages": [{"role": "user", "content": "x"}], "max_tokens": 3, "n": 2,
                             "stream": True, "enable_thinking": False}) as r:
        ev = _sse(r)
    assert ev[-1] == "[DONE]" and sorted(e["choices"][0]["index"] for e in ev[:-1]) == [0, 1]
    e = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 2, "echo": True,
                                             "temperature": 0}).json()
    assert e["choices"][0]["text"].startswith("abc") and e["usage"]["completion_tokens"] == 2
    r = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "n": 17})
    assert r.status_code == 400 and r.json()["error"]["code"] == "unsupported_parameter"
    many = client.post("/v1/completions", json={"model": "tiny", "prompt": ["a", "bb", [5, 6, 7]], "max_tokens": 2,
                                                "temperature": 0})
    assert many.status_code == 400                                  # strings and token rows cannot be mixed
    err = many.json()["error"]
    assert err["code"] == "invalid_request" and err["param"].startswith("prompt") and err["hipengine"]["status"] == 400
    rows = client.post("/v1/completions", json={"model": "tiny", "prompt": [[5, 6, 7], [8, 9]], "max_tokens": 2,
                                                "temperature": 0})
    assert rows.status_code == 200 and len(rows.json()["choices"]) == 2
    texts = client.post("/v1/completions", json={"model": "tiny", "prompt": ["a", "bb"], "max_tokens": 2, "temperature": 0})
    assert texts.status_code == 200 and [c["index"] for c in texts.json()["choices"]] == [0, 1]
    bad = client.post("/v1/chat/completions", json={"model": "tiny", "messages": "not a list"})
    assert bad.status_code == 400 and bad.json()["error"]["param"] == "messages"


def test_request_deadline_is_reported(client):
    r = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 400, "timeout_ms": 1,
                                             "ignore_eos": True})
    assert r.status_code in (200, 408)
    if r.status_code == 408:
        assert r.json()["error"]["code"] == "deadline_exceeded" and r.json()["error"]["hipengine"]["retryable"]
    else:                                                       # finished inside a millisecond: a complete answer
        assert r.json()["usage"]["completion_tokens"] == 400
    ok = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 3, "timeout_ms": 60000})
    assert ok.status_code == 200


@pytest.fixture(scope="module")
def wide_client():
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=1024)
    with TestClient(create_app(llm, ServerConfig(served_model_name="tiny"))) as c:
        yield c
    llm.close()


def test_required_tool_call_over_http_is_parsed_and_streamed(wide_client):
    """A parameterless tool under `tool_choice: required`: the grammar leaves one possible text, which a random model
    then has to produce; the server parses it into `tool_calls` (blocking) and `delta.tool_calls` (streaming)."""
    client = wide_client
    tools = [{"type": "function", "function": {"name": "get_time", "parameters": {"type": "object"}}}]
    body = {"model": "tiny", "messages": [{"role": "user", "content": "time?"}], "tools": tools,
            "tool_choice": "required", "max_tokens": 120, "temperature": 0.7, "seed": 3, "enable_thinking": False}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    ch = r.json()["choices"][0]
    assert ch["finish_reason"] == "tool_calls", ch
    call = ch["message"]["tool_calls"][0]
    assert call["type"] == "function" and call["function"]["name"] == "get_time" and call["id"]
    assert json.loads(call["function"]["arguments"]) == {} and ch["message"]["content"] is None
    with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as resp:
        ev = _sse(resp)
    deltas = [e["choices"][0] for e in ev if isinstance(e, dict) and e.get("choices")]
    calls = [tc for d in deltas for tc in (d["delta"].get("tool_calls") or [])]
    by_index = {}
    for tc in calls:
        by_index.setdefault(tc["index"], []).append(tc)
    assert sorted(by_index) == list(range(len(by_index))) and by_index       # parallel calls get consecutive indices
    for parts in by_index.values():
        assert parts[0]["function"]["name"] == "get_time" and parts[0]["type"] == "function"   # the name comes first
        assert len({p["id"] for p in parts}) == 1                             # one id for all chunks of a call
        assert json.loads("".join(p["function"].get("arguments", "") for p in parts)) == {}
    assert deltas[-1]["finish_reason"] == "tool_calls"
    named = dict(body, tool_choice={"type": "function", "function": {"name": "get_time"}})
    assert client.post("/v1/chat/completions", json=named).json()["choices"][0]["finish_reason"] == "tool_calls"
    none = client.post("/v1/chat/completions", json=dict(body, tool_choice="none", max_tokens=5)).json()["choices"][0]
    assert none["finish_reason"] in ("length", "stop") and not none["message"].get("tool_calls")


def test_stop_strings_logit_bias_choice_and_refused_parameters(client):
    base = {"model": "tiny", "prompt": "abc", "max_tokens": 12, "temperature": 0, "ignore_eos": True}
    full = client.post("/v1/completions", json=base).json()["choices"][0]
    assert full["finish_reason"] == "length"
    # stop strings are lowered to token sequences: one made of forced byte tokens ends the text before it
    z = client.post("/v1/hipengine/tokenize", json={"text": "Z"}).json()["tokens"][0]
    r = client.post("/v1/completions", json=dict(base, logit_bias={str(z): 100}, stop=["ZZZ"])).json()["choices"][0]
    assert r["finish_reason"] == "stop" and r["text"] == ""
    # a large bias on one token makes the greedy continuation that token
    tok = client.post("/v1/hipengine/tokenize", json={"text": "Z"}).json()["tokens"][0]
    biased = client.post("/v1/completions", json=dict(base, max_tokens=4, logit_bias={str(tok): 100})).json()
    assert biased["choices"][0]["text"] == "ZZZZ"
    bad = client.post("/v1/completions", json=dict(base, logit_bias={"not-a-token": 1}))
    assert bad.status_code == 400
    # guided_choice validates the result: a random model does not answer with one of the choices
    chat = {"model": "tiny", "messages": [{"role": "user", "content": "pick"}], "max_tokens": 4, "temperature": 0,
            "enable_thinking": False}
    g = client.post("/v1/chat/completions", json=dict(chat, guided_choice=["yes", "no"])).json()["choices"][0]
    assert g["finish_details"]["reason"] == "schema_violation"
    ok = client.post("/v1/chat/completions", json=dict(chat, max_tokens=3, guided_choice=["yes", "no"],
                                                       logit_bias={str(client.post("/v1/hipengine/tokenize", json={"text": "n"}).json()["tokens"][0]): 100}))
    assert ok.status_code == 200
    # refused before generation
    for extra, param in (({"grammar": "root ::= 'a'"}, "grammar"), ({"guided_grammar": "x"}, "grammar"),
                         ({"response_format": {"type": "yaml"}}, "response_format"),
                         ({"guided_regex": "("}, "guided_regex"), ({"top_logprobs": 3}, "top_logprobs"),
                         ({"logprobs": True, "top_logprobs": 21}, "top_logprobs")):
        r = client.post("/v1/chat/completions", json=dict(chat, **extra))
        assert r.status_code == 400 and r.json()["error"]["param"] == param, (extra, r.text)
    lp = client.post("/v1/chat/completions", json=dict(chat, logprobs=True, top_logprobs=2)).json()["choices"][0]
    assert len(lp["logprobs"]["content"]) == 4 and len(lp["logprobs"]["content"][0]["top_logprobs"]) == 2
    t = client.post("/v1/hipengine/tokenize", json={"messages": [{"role": "user", "content": "hi"}]}).json()
    assert t["count"] > 2 and client.post("/v1/hipengine/count_tokens", json={"text": "hello"}).json()["count"] == 5


def test_full_queue_answers_429_with_retry_after():
    import threading
    import time
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=1024)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="tiny", max_queued_requests=1))) as c:
            c.post("/v1/completions", json={"model": "tiny", "prompt": "warm", "max_tokens": 2})      # engine resident
            done = {}

            def long_one():
                done["r"] = c.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 500,
                                                            "ignore_eos": True, "temperature": 0})
            t = threading.Thread(target=long_one)
            t.start()
            time.sleep(0.15)                      # the long request is inside the gate before the probes start
            busy = None
            deadline = time.time() + 10
            while time.time() < deadline and t.is_alive():
                r = c.post("/v1/completions", json={"model": "tiny", "prompt": "x", "max_tokens": 1})
                if r.status_code == 429:
                    busy = r
                    break
                time.sleep(0.005)
            t.join(timeout=60)
            assert done["r"].status_code == 200 and done["r"].json()["usage"]["completion_tokens"] == 500
            assert busy is not None, "the second request was never refused while the first one ran"
            assert busy.json()["error"]["code"] == "engine_busy" and int(busy.headers["Retry-After"]) >= 1
            assert busy.json()["error"]["hipengine"]["retryable"] is True
            after = c.post("/v1/completions", json={"model": "tiny", "prompt": "x", "max_tokens": 1})
            assert after.status_code == 200                                     # the queue has room again
            ready = c.get("/ready").json()
            assert ready["batcher"]["rejected_busy"] >= 1 and ready["batcher"]["in_flight"] == 0
    finally:
        llm.close()


def test_serving_load_harness_runs_against_its_own_server_on_the_host_backend(capsys):
    """The Poisson load generator end to end: it brings up the server in a thread, drives it over real sockets and
    prints one JSON line; with speculative decoding on the host backend the server block reports the cycles."""
    from hipengine_b200.benchmark.serving_load import main
    rc = main(["--model", "tiny-hybrid-mtp", "--backend", "cpu_reference", "--requests", "5", "--concurrency", "2",
               "--rate", "40", "--min-prompt", "12", "--max-prompt", "40", "--shared-prefix", "4", "--output-tokens", "6",
               "--max-active", "2", "--port", "18997", "--mtp", "on", "--mtp-depth", "2", "--endpoint", "chat",
               "--gpu-sampler"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["completed"] == 5 and out["failed"] == 0 and out["generated_tok_per_s"] > 0
    assert out["ttft_p50_ms"] > 0 and out["config"]["endpoint"] == "chat" and out["config"]["mtp"] == "on"
    assert "gpu" in out and ("error" in out["gpu"] or out["gpu"]["samples"] >= 0)


def test_malformed_requests_are_client_errors_and_never_reach_the_engine(client):
    """Token ids outside the vocabulary (prompt, bias, suppression), an empty prompt, zero or negative max_tokens and
    sampler values out of range all answer 400 in the envelope, and the engine stays healthy afterwards (an id that
    reached the embedding table would index device memory out of range)."""
    base = {"model": "tiny", "prompt": "a", "max_tokens": 2}
    for patch, needle in (({"prompt": [5, 999999]}, "outside the vocabulary"), ({"prompt": [[5, -1]]}, "outside the vocabulary"),
                          ({"prompt": ""}, "empty"), ({"max_tokens": 0}, "max_tokens"), ({"max_tokens": -5}, "max_tokens"),
                          ({"temperature": -1}, "temperature"), ({"top_p": 0}, "top_p"),
                          ({"logit_bias": {"999999": 5}}, "outside the vocabulary"),
                          ({"logit_bias": {"5": 500}}, "logit_bias")):
        r = client.post("/v1/completions", json=dict(base, **patch))
        assert r.status_code == 400 and needle in r.json()["error"]["message"], (patch, r.text)
        assert r.json()["error"]["hipengine"]["retryable"] is False
    with client.stream("POST", "/v1/completions", json=dict(base, prompt=[5, 999999], stream=True)) as r:
        assert r.status_code == 400
    r = client.post("/v1/completions", content=b"{not json", headers={"Content-Type": "application/json"})
    assert r.status_code == 400 and r.json()["error"]["code"] == "invalid_request"
    assert client.post("/v1/completions", json=base).status_code == 200
    ready = client.get("/ready").json()
    assert ready["ready"] and ready["engine_service"]["healthy"]


def test_refused_streams_answer_with_a_status_and_do_not_hold_the_admission_gate():
    """A live stream is checked before its response starts: a bad prompt or one that cannot fit the context is a 400,
    not an error event inside a 200 stream, and each refusal gives its place in the admission gate back (a gate of two
    places still serves after many refusals)."""
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=128)
    try:
        with TestClient(create_app(llm, ServerConfig(served_model_name="tiny", max_queued_requests=2))) as c:
            for _ in range(4):
                for body in ({"prompt": [5, 999999]}, {"prompt": [7] * 200}, {"prompt": ""}):
                    with c.stream("POST", "/v1/completions", json=dict({"model": "tiny", "max_tokens": 2, "stream": True},
                                                                       **body)) as r:
                        r.read()
                        assert r.status_code == 400 and r.headers["content-type"].startswith("application/json")
                chat = {"model": "tiny", "messages": [{"role": "user", "content": "x " * 300}], "max_tokens": 4, "stream": True}
                with c.stream("POST", "/v1/chat/completions", json=chat) as r:
                    r.read()
                    assert r.status_code == 400 and r.json()["error"]["code"] == "context_overflow"
            with c.stream("POST", "/v1/completions", json={"model": "tiny", "prompt": "ab", "max_tokens": 3, "stream": True}) as r:
                ev = _sse(r)
            assert r.status_code == 200 and ev[-1] == "[DONE]"
            assert c.post("/v1/completions", json={"model": "tiny", "prompt": "ab", "max_tokens": 2}).status_code == 200
    finally:
        llm.close()


def test_unknown_paths_unserved_modalities_and_bad_timeouts_answer_in_the_envelope(client):
    r = client.get("/v1/nope")
    assert r.status_code == 404 and r.json()["error"]["code"] == "not_found" and "/v1/nope" in r.json()["error"]["message"]
    r = client.get("/v1/completions")
    assert r.status_code == 405 and r.json()["error"]["code"] == "method_not_allowed"
    r = client.post("/v1/audio/songs", json={"model": "tiny", "lyrics": "la", "style": "pop"})
    assert r.status_code == 501 and r.json()["error"]["code"] == "unsupported_feature"
    r = client.post("/v1/completions", json={"model": "tiny", "prompt": "a", "max_tokens": 2, "timeout_ms": -5})
    assert r.status_code == 400 and r.json()["error"]["param"] == "timeout_ms"
    assert client.post("/v1/completions", json={"model": "tiny", "prompt": "a", "max_tokens": 2, "timeout_ms": 0}
                       ).status_code == 200                                          # zero means no deadline
    from hipengine_b200 import UnsupportedModalityError
    llm = client.app.state.llm
    for fn in (llm.generate_multimodal_detailed, llm.transcribe, llm.synthesize, llm.generate_song):
        with pytest.raises(UnsupportedModalityError, match="not served"):
            fn("x")


def test_session_documents_and_rollback_counts_are_validated(client):
    """A snapshot whose transcript could not have come from a chat request is refused when it is restored (not turned
    into a session that fails on every later use), and a rollback count must be a non-negative integer."""
    chat = {"model": "tiny", "messages": [{"role": "user", "content": "a"}], "max_tokens": 3, "enable_thinking": False}
    sid = client.post("/v1/chat/completions", json=dict(chat, session={"create": True})).json()["session"]["id"]
    snap = client.get(f"/v1/hipengine/sessions/{sid}/snapshot").json()
    assert snap["session"]["turns"] == 1 and len(snap["session"]["messages"]) == 2
    for patch in ({"messages": "x"}, {"messages": [{"role": "robot", "content": "x"}]}, {"messages": [{"role": "user", "content": 5}]},
                  {"messages": ["x"]}, {"turns": -1}, {"turns": "many"},
                  {"messages": [{"role": "assistant", "content": None, "tool_calls": "f"}]}):
        r = client.post("/v1/hipengine/sessions/restore", json=dict(snap, session=dict(snap["session"], **patch)))
        assert r.status_code == 400 and r.json()["error"]["code"] == "invalid_continuation", (patch, r.text)
    assert client.post("/v1/hipengine/sessions/restore", json=dict(snap, session=None)).status_code == 400
    rid = client.post("/v1/hipengine/sessions/restore", json=snap).json()
    assert rid["turns"] == 1
    r = client.post("/v1/chat/completions", json=dict(chat, session=rid["id"]))          # the restored session continues
    assert r.status_code == 200 and r.json()["usage"]["prompt_tokens"] > 26
    for bad in (-1, "two", 1.5, True):
        r = client.post(f"/v1/hipengine/sessions/{sid}/rollback", json={"turns": bad})
        assert r.status_code == 400 and r.json()["error"]["param"] == "turns", bad
    assert client.post(f"/v1/hipengine/sessions/{sid}/rollback", json={"turns": 0}).json()["turns"] == 1
    assert client.post(f"/v1/hipengine/sessions/{sid}/rollback").json() == {"id": sid, "turns": 0, "messages": 0}
