"""Auxiliary subsystems on the host: resource ledger, simulated KV backend, tracing helpers, load simulator."""
import pytest

from hipengine_b200.config import EngineConfig, KVConfig, SchedulerConfig
from hipengine_b200.generation.simulator import SimulatedRunner, poisson_arrivals, run_load_scenario
from hipengine_b200.generation.types import GenerationRequest
from hipengine_b200.kvcache.ledger import ResourceClaim, ResourceLedger, ResourceUnavailable
from hipengine_b200.kvcache.simulated import create_fake_kv_backend
from hipengine_b200.utils.tracing import FlightRecorder, LaunchCensus, StageTimer, nvtx_range


def test_ledger_all_or_nothing():
    led = ResourceLedger()
    led.register("kv_pages", 100)
    led.register("state_slots", 2)
    a = led.acquire("req1", [ResourceClaim("kv_pages", 60), ResourceClaim("state_slots", 1)])
    with pytest.raises(ResourceUnavailable) as e:
        led.acquire("req2", [ResourceClaim("state_slots", 1), ResourceClaim("kv_pages", 50)])
    assert e.value.resource == "kv_pages" and e.value.available == 40
    assert led.available("state_slots") == 1               # the refused set took nothing
    led.release(a)
    led.release(a)                                         # idempotent
    assert led.available("kv_pages") == 100
    snap = led.snapshot()
    assert snap["kv_pages"]["peak"] == 60 and snap["kv_pages"]["refused"] == 1
    with pytest.raises(ResourceUnavailable):
        led.acquire("req3", [ResourceClaim("unknown", 1)])


def test_simulated_kv_prefix_sharing():
    kv = create_fake_kv_backend("paged", capacity_tokens=1024)
    prompt = list(range(100))
    l1 = kv.admit(1, prompt, 20)
    assert l1 is not None and l1.cached_tokens == 0
    kv.publish_prefix(prompt, l1)
    l2 = kv.admit(2, prompt[:96] + [7, 7, 7], 20)
    assert l2.cached_tokens == 96 and l2.pages[:6] == l1.pages[:6]
    kv.release(1)
    kv.release(2)
    assert kv.admit(3, list(range(5000)), 10) is None       # larger than the pool
    with pytest.raises(ValueError):
        create_fake_kv_backend("nope")


def test_tracing_helpers_on_cpu():
    t = StageTimer(use_cuda=False)
    for _ in range(3):
        with t.stage("a"):
            sum(range(1000))
    s = t.summary()
    assert s["a"]["count"] == 3 and s["a"]["total_ms"] >= 0
    with nvtx_range("x"):
        pass
    c = LaunchCensus()
    with c.region("r"):
        pass
    assert c.report()["r"]["calls"] == 1
    fr = FlightRecorder(capacity=4)
    for i in range(10):
        fr.record("tick", i=i)
    d = fr.dump()
    assert len(d) == 4 and d[-1]["i"] == 9 and d[0]["seq"] == 7 and "tick" in fr.dump_json(last=1)


def _requests(n, seed=0, shared=0):
    import random
    rng = random.Random(seed)
    common = [rng.randrange(1000) for _ in range(shared)]
    out = []
    for i in range(n):
        body = [rng.randrange(1000) for _ in range(rng.randrange(64, 512))]
        out.append(GenerationRequest(prompt_token_ids=(common if i % 2 == 0 else []) + body, max_tokens=32,
                                     ignore_eos=True))
    return out


def test_load_scenario_is_deterministic_under_each_policy():
    def run(policy):
        cfg = EngineConfig(max_sequence_length=4096,
                           scheduler=SchedulerConfig(policy=policy, max_active_requests=16, max_pending_requests=256),
                           kv=KVConfig(prefix_cache="radix"))
        reqs = _requests(40, shared=128)
        return run_load_scenario(cfg, reqs, poisson_arrivals(40, rate_per_s=50.0, seed=1), max_concurrent=16)

    a, b = run("protect_decode"), run("protect_decode")
    assert a.summary() == b.summary()                      # virtual time: bit-for-bit repeatable
    assert a.completed == 40 and a.failed == 0 and a.total_tokens == 40 * 32
    assert a.cached_prompt_tokens > 0                      # half the prompts share a 128-token prefix
    c = run("protect_ttft")
    assert c.completed == 40
    assert c.total_tokens == a.total_tokens                # the policy changes latencies, never the outputs


def test_injected_decode_failure_is_contained():
    cfg = EngineConfig(max_sequence_length=2048, scheduler=SchedulerConfig(max_active_requests=4))
    reqs = _requests(4, seed=3)
    runner = SimulatedRunner(cfg, fail_decode_admission=[2])
    res = run_load_scenario(cfg, reqs, [0.0] * 4, max_concurrent=4, runner=runner)
    assert res.failed == 1 and res.completed == 3           # only the named request fails; the rest finish


def test_tool_call_grammar_generator():
    from hipengine_b200.generation.grammar import grammar_available, tool_call_grammar
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "unit": {"enum": ["c", "f"]},
                                         "days": {"type": "integer"}, "opts": {"type": "object"}},
        "required": ["city", "days"]}}},
        {"type": "function", "function": {"name": "noop", "parameters": {"type": "object", "properties": {}}}}]
    g = tool_call_grammar(tools)
    assert 'start: [text] call (ws call)*' in g
    assert '"<function=get_weather>"' in g and '"<function=noop>"' in g
    assert '"<parameter=city>"' in g and '[p_0_1]' in g            # optional parameter is bracketed
    assert 'p_0_0 [p_0_1] p_0_2 [p_0_3]' in g                       # schema order, required ones mandatory
    assert "json_value" in g and '"c" | "f"' in g
    single = tool_call_grammar(tools, allow_text_before=False, parallel=False, only="noop")
    assert "get_weather" not in single and single.startswith("start: call\n")
    import pytest
    with pytest.raises(ValueError):
        tool_call_grammar([{"function": {"name": "bad name"}}])
    with pytest.raises(ValueError):
        tool_call_grammar(tools, only="missing")
    assert isinstance(grammar_available(), bool)
