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


def test_cold_tier_roundtrip_lru_and_corruption(tmp_path):
    import numpy as np
    import torch
    from hipengine_b200.kvcache.tiering import (ColdTier, ColdTierCorruption, decode_object, encode_object,
                                                prefix_key, restore_is_worthwhile)
    kv = torch.randn(2, 4, 16, 32).bfloat16()
    state = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    blob, raw = encode_object({"kv": kv, "state": state}, {"tokens": 16})
    arrays, meta = decode_object(blob)
    assert meta == {"tokens": 16} and raw == kv.numel() * 2 + state.nbytes
    assert arrays["kv"].dtype == torch.bfloat16 and torch.equal(arrays["kv"], kv)
    assert np.array_equal(arrays["state"], state)
    bad = bytearray(blob)
    bad[-3] ^= 0x40
    import pytest
    with pytest.raises(ColdTierCorruption):
        decode_object(bytes(bad))
    with pytest.raises(ColdTierCorruption):
        decode_object(blob[:-1])

    k1, k2 = prefix_key("qwen/q4", [1, 2, 3]), prefix_key("qwen/q4", [1, 2, 4])
    assert k1 != k2 and k1 == prefix_key("qwen/q4", (1, 2, 3)) and k1 != prefix_key("other", [1, 2, 3])

    for directory in (None, str(tmp_path / "cold")):
        zeros = {"kv": torch.zeros(64, 1024)}                       # compresses well
        one = len(encode_object(zeros)[0])
        tier = ColdTier(capacity_bytes=2 * one + 16, directory=directory)
        assert tier.put("a", zeros, {"n": 1}) is not None
        assert tier.put("b", zeros) is not None
        assert tier.get("a")[1] == {"n": 1}                         # touch: "b" is now the oldest
        tier.put("c", zeros)
        assert "b" not in tier and "a" in tier and "c" in tier and tier.stats["evicted"] == 1
        assert tier.compression_ratio() > 50
        assert tier.put("huge", {"x": torch.randn(4096, 64)}) is None     # larger than the whole tier
        assert tier.get("missing") is None and tier.stats["misses"] == 1
        if directory:                                               # flip a byte on disk: dropped, not returned
            p = tier._path("c")
            raw_file = bytearray(open(p, "rb").read())
            raw_file[-1] ^= 0xFF
            open(p, "wb").write(bytes(raw_file))
            assert tier.get("c") is None and tier.stats["corrupt"] == 1 and "c" not in tier
            again = ColdTier(capacity_bytes=1 << 20, directory=directory)   # a new process adopts what is left
            assert "a" in again and torch.equal(again.get("a")[0]["kv"], zeros["kv"])
    # 4096 tokens at 16k tok/s = 256 ms of prefill against ~1 GB of state: restore loses; against 100 MB it wins
    assert not restore_is_worthwhile(4096, 10 ** 9, 10 ** 9, 16000.0)
    assert restore_is_worthwhile(4096, 2 * 10 ** 7, 4 * 10 ** 7, 16000.0)


def _wired_pool(n_pages):
    """PagePool + RadixCache wired the way the GPU runner wires them."""
    from hipengine_b200.kvcache.pool import PagePool
    from hipengine_b200.kvcache.radix import RadixCache
    pool = PagePool(n_pages, page_tokens=16)
    t = [0.0]

    def clock():
        t[0] += 1.0
        return t[0]

    radix = RadixCache(16, clock=clock)
    radix.on_retain = pool.retain_cache
    radix.on_release = pool.release_cache
    radix.page_refcount = lambda p: pool.refcount[p]
    pool.evict_hook = radix.evict
    return pool, radix


def test_admit_with_shared_prefix_on_a_full_pool_never_reuses_the_prefix_pages():
    """Seven usable pages, prefix A (4 pages) and prefix B (3 pages) cached, then a request that matches A and
    needs three more pages: the three must come from B, never from A itself."""
    from hipengine_b200.kvcache.pool import PoolExhausted
    pool, radix = _wired_pool(8)
    a_tok = list(range(64))
    b_tok = list(range(1000, 1048))
    la = pool.admit(1, 64, now_tokens=64)
    radix.insert(a_tok, la.pages)
    pool.release(1)
    lb = pool.admit(2, 48, now_tokens=48)
    radix.insert(b_tok, lb.pages)
    pool.release(2)
    assert pool.n_free == 0 and pool.n_evictable() == 7
    m = radix.match(a_tok + list(range(5000, 5048)))
    assert m.tokens == 64 and len(m.pages) == 4
    lease = pool.admit(3, 64 + 48, shared_prefix=m.pages, now_tokens=64 + 48)
    assert len(set(lease.pages)) == len(lease.pages) == 7
    assert lease.pages[:4] == m.pages
    assert not set(lease.pages[4:]) & set(m.pages)
    pool.assert_conserved()
    radix.assert_consistent()
    assert radix.match(a_tok + [1]).tokens == 64          # the matched prefix is still published
    # a request that cannot fit leaves the prefix refcounts as they were
    pool.release(3)
    m = radix.match(a_tok + list(range(5000, 5048)))
    before = list(pool.refcount)
    try:
        pool.admit(4, 64 + 16 * 20, shared_prefix=m.pages, now_tokens=64)
        raise AssertionError("expected PoolExhausted")
    except PoolExhausted:
        pass
    assert pool.refcount == before
    pool.assert_conserved()


def test_radix_eviction_is_strict_lru_across_newly_exposed_leaves():
    """A long stale chain must be evicted (leaf by leaf, parents as they become leaves) before a fresher leaf."""
    pool, radix = _wired_pool(12)
    old = list(range(48))
    l1 = pool.admit(1, 48, now_tokens=48)
    old_pages = list(l1.pages)
    radix.insert(old, old_pages)
    pool.release(1)
    fresh = list(range(900, 916))
    l2 = pool.admit(2, 16, now_tokens=16)
    radix.insert(fresh, l2.pages)
    pool.release(2)
    radix.match(fresh + [1])                               # touch: fresh is now the most recent
    freed = radix.evict(3)
    assert sorted(freed) == sorted(old_pages)
    assert radix.match(fresh + [1]).tokens == 16
    assert radix.match(old + [1]).tokens == 0
    pool.assert_conserved()


def test_in_tree_tool_call_grammar_matcher():
    """The automaton compiled from a tool list accepts exactly well-formed calls, token masks follow it through a
    toy vocabulary, and end-of-sequence is allowed only on a complete match."""
    import torch
    from hipengine_b200.generation.grammar import ToolCallAutomaton, ToolCallMatcher
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"},
                                         "unit": {"enum": ["c", "f"]}}, "required": ["city"]}}},
             {"type": "function", "function": {"name": "stop", "parameters": {"type": "object", "properties": {}}}}]
    auto = ToolCallAutomaton(tools)

    def accepts(text):
        s = auto.start_set
        for ch in text:
            s = auto.step(s, ch)
            if s is None:
                return False
        return auto.accepting(s)

    good = "Let me check.<tool_call>\n<function=get_weather><parameter=city>Oslo</parameter><parameter=days>3" \
           "</parameter></function>\n</tool_call>"
    assert accepts(good)
    assert accepts(good + "\n<tool_call><function=stop></function></tool_call>")          # parallel calls
    assert accepts("<tool_call><function=get_weather><parameter=city>X</parameter><parameter=unit>f</parameter>"
                   "</function></tool_call>")
    assert not accepts(good.replace("get_weather", "get_wether"))                           # unknown function
    assert not accepts(good.replace("<parameter=city>Oslo</parameter>", ""))                # required one missing
    assert not accepts(good.replace(">3<", ">three<"))                                      # integer expected
    assert not accepts(good[:-3])                                                           # incomplete
    vocab = ["<eos>", "<tool_call>", "<function=", "get_weather", "stop", ">", "<parameter=", "city", "days",
             "Oslo", "</parameter>", "</function>", "</tool_call>", "3", "x", "\n", "get_", "weather", "<", "/"]
    m = ToolCallMatcher(ToolCallAutomaton(tools, allow_text_before=False), vocab, eos_token_id=0)
    toks = lambda names: [vocab.index(n) for n in names]
    mask = m.allowed_mask()
    assert mask[vocab.index("<tool_call>")] and mask[vocab.index("<")] and not mask[vocab.index("x")] and not mask[0]
    for t in toks(["<tool_call>", "<function=", "get_", "weather", ">", "<parameter=", "city", ">", "Oslo",
                   "</parameter>"]):
        assert m.allowed_mask()[t], vocab[t]
        assert m.accept(t)
    mask = m.allowed_mask()
    assert mask[vocab.index("<parameter=")] and mask[vocab.index("</function>")] and not mask[vocab.index("Oslo")]
    for t in toks(["</function>", "</tool_call>"]):
        assert m.accept(t)
    assert m.finished() and m.allowed_mask()[0]                 # end-of-sequence now allowed
    assert isinstance(m.allowed_mask(), torch.Tensor) and not m.accept(vocab.index("x")) and m.dead()


def test_artifact_admission_plan_contract_and_memory_preflight():
    """Admission lists what cannot be served (missing tensors, block types without a reader, rows that are not whole
    blocks, a pool that does not fit) before anything is built; a servable checkpoint gets a plan digest."""
    import pytest
    import torch
    from hipengine_b200.config import EngineConfig
    from hipengine_b200.loading.admission import ArtifactRejected, admit, build_role_manifest, plan_contract, role_of
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.loading.weights import ModelWeights
    from hipengine_b200.models.config import TINY_HYBRID
    from hipengine_b200.quant.ggml import GGMLType
    assert role_of("blk.7.ffn_down.weight") == "ffn_down" and role_of("token_embd.weight") == "token_embd"
    w = build_random_model(TINY_HYBRID, seed=0)
    cfg = EngineConfig.from_env()
    rep = admit(w, cfg, free_bytes=10 ** 12)
    assert rep["admitted"] and rep["plan_complete"] and len(rep["plan_digest"]) == 16
    assert "ffn_down" in rep["role_manifest"] and rep["memory"]["fits"]
    assert admit(w, cfg, free_bytes=10 ** 12)["plan_digest"] == rep["plan_digest"]        # deterministic
    man = build_role_manifest(w)
    assert sum(man["attn_norm"].values()) == TINY_HYBRID.n_layers
    # does not fit
    with pytest.raises(ArtifactRejected) as e:
        admit(w, cfg, free_bytes=1 << 20)
    assert "GiB free" in str(e.value) and e.value.report["memory"]["fits"] is False
    # a missing tensor and a block type nobody reads
    t = dict(w.tensors)
    t.pop("blk.0.attn_norm.weight")
    bad = ModelWeights(w.config, t, dict(w.metadata))
    pc = plan_contract(bad)
    assert not pc.is_complete and pc.unsupported[0].slot == "blk.0.attn_norm.weight"
    q = t["blk.1.ffn_down.weight"]
    t["blk.1.ffn_down.weight"] = type(q)(q.name, 99 if 99 in GGMLType._value2member_map_ else GGMLType.Q5_K, q.shape, q.raw)
    pc2 = plan_contract(ModelWeights(w.config, t, dict(w.metadata)))
    assert pc2.digest != rep["plan_digest"]
    with pytest.raises(ArtifactRejected):
        admit(bad, cfg, free_bytes=10 ** 12)


def test_unsupported_kv_storage_is_refused_not_ignored():
    import pytest
    from hipengine_b200 import LLM
    with pytest.raises(ValueError, match="kv_storage"):
        LLM("tiny-dense", backend="cpu_reference", kv_storage="fp8")
    assert LLM("tiny-dense", backend="cpu_reference", kv_storage="auto").config.kv.storage == "bf16"
    from hipengine_b200.server.readiness import kv_capability
    from hipengine_b200.config import KVConfig
    from hipengine_b200.models.config import TINY_DENSE
    cap = kv_capability(TINY_DENSE, KVConfig())["storage"]
    assert cap["bf16"]["supported"] and not cap["int8"]["supported"] and cap["int8"]["granularity"] == "per_token_head"


def test_int8_kv_format_and_the_host_backend_that_serves_it():
    """INT8 KV per token and head: the quantiser's error bound, exact reproduction of what the reader sees, and the
    cpu_reference backend generating with that storage (close to exact-KV logits; the same engine API)."""
    import torch
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    from hipengine_b200.ref import ops as R
    from hipengine_b200.ref.model import RefModel
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 3, 64, generator=g) * torch.tensor([0.01, 1.0, 30.0])[None, :, None]
    q, sc = R.kv_int8_quantize(x)
    assert q.dtype == torch.int8 and sc.dtype == torch.float16 and sc.shape == (7, 3)
    deq = R.kv_int8_dequantize(q, sc)
    assert ((deq - x).abs() <= sc.float()[..., None] * 0.5 + 1e-7).all()           # half a step per element
    assert int(q.abs().max()) == 127 and torch.equal(R.kv_store_roundtrip(x, "int8"), deq)
    zero = torch.zeros(2, 1, 8)
    assert torch.equal(R.kv_int8_dequantize(*R.kv_int8_quantize(zero)), zero)     # an all-zero row stays zero
    q32, sc32 = R.kv_int8_quantize(x, torch.float32)
    assert sc32.dtype == torch.float32 and (R.kv_int8_dequantize(q32, sc32) - x).abs().max() <= deq.sub(x).abs().max() + 1e-3
    w = build_random_model(TINY_HYBRID, seed=3, std=0.05)
    toks = torch.randint(0, TINY_HYBRID.vocab, (48,), generator=g)
    exact, _ = RefModel(w).forward(toks)
    int8, _ = RefModel(w, kv_storage="int8").forward(toks)
    p, qq = torch.log_softmax(exact.double(), -1), torch.log_softmax(int8.double(), -1)
    kl = (p.exp() * (p - qq)).sum(-1)
    assert 0 < float(kl.max()) < 0.01 and (exact.argmax(-1) == int8.argmax(-1)).float().mean() > 0.9
    llm = LLM(w, backend="cpu_reference", kv_storage="int8", max_active_requests=2, max_sequence_length=128)
    try:
        assert llm.config.kv.storage == "int8"
        out = llm.generate_detailed([toks[:20].tolist()], SamplingParams(max_tokens=5, ignore_eos=True))[0]
        assert out.error is None and len(out.token_ids) == 5
        assert llm._get_engine().loop.runner.model.kv_storage == "int8"
    finally:
        llm.close()
    import hipengine_b200.llm as L
    if not torch.cuda.is_available():
        return
    with pytest.raises(ValueError, match="bf16 only"):
        L.LLM("tiny-dense", backend="cuda_sm100a", kv_storage="int8")


def test_decode_attention_split_policy():
    """One 64-key tile per CTA for a single short row, spans up to 1024 keys for wide batches, always whole tiles."""
    from hipengine_b200.ops.kernels import attn_decode_split
    assert attn_decode_split(4096, 1, 4) == (64, 64)
    sl, ns = attn_decode_split(4096, 16, 4)
    assert sl % 64 == 0 and 256 <= sl <= 512 and ns == -(-4096 // sl)
    assert attn_decode_split(4096, 64, 4)[0] == 1024
    assert attn_decode_split(262144, 1, 4) == (1024, 256)
    assert attn_decode_split(1, 1, 1) == (64, 1)


def test_pool_truncation_returns_speculative_pages_to_the_lease_credit():
    """A speculative cycle reserves pages for every draft; what the accepted prefix does not need goes back to the
    request's credit, and the next cycle takes it from there (page conservation holds throughout)."""
    from hipengine_b200.kvcache.pool import PagePool
    pool = PagePool(n_pages=32, page_tokens=16)
    lease = pool.admit(7, total_tokens=200, shared_prefix=[], now_tokens=40)     # 3 pages now, credit for the rest
    credit0 = lease.credit
    pool.append_pages(lease, 40 + 3 * 16)                                          # drafts reach three pages further
    assert len(lease.pages) == 6 and lease.credit == credit0 - 3
    dropped = pool.truncate_pages(lease, 41 + 1)                                   # one token accepted
    assert len(dropped) == 3 and len(lease.pages) == 3 and lease.credit == credit0
    pool.assert_conserved()
    pool.append_pages(lease, 40 + 2 * 16)
    assert len(lease.pages) == 5 and lease.credit == credit0 - 2 and pool.stats["truncated"] == 3
    pool.assert_conserved()
    pool.release(7)
    pool.assert_conserved()


def test_every_environment_switch_is_documented():
    """docs/ENVS.md lists every HE_* variable the source reads (getenv / os.environ)."""
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    doc = (root / "docs" / "ENVS.md").read_text()
    pat = re.compile(r"""(?:getenv\(\s*"|environ(?:\.get|\.setdefault)?\(\s*"|environ\[\s*"|"\s*in\s+e\b.*?|e\[")(HE_[A-Z0-9_]+)""")
    used = set()
    files = list((root / "hipengine_b200").rglob("*.py")) + list((root / "hipengine_b200" / "csrc").glob("*.c*")) + \
        [root / "bench.py", root / "__graft_entry__.py"]
    for f in files:
        text = f.read_text(errors="ignore")
        used |= set(pat.findall(text))
        used |= set(re.findall(r'if "(HE_[A-Z0-9_]+)" in e', text))
    missing = sorted(v for v in used if f"`{v}`" not in doc)
    assert not missing, f"undocumented environment switches: {missing}"
    assert len(used) >= 25


def test_scratch_canaries_detect_a_write_past_the_extent():
    import torch
    from hipengine_b200.models.executor import _Scratch
    sc = _Scratch(torch.device("cpu"), canaries=True)
    a = sc.get("a", (4, 8), torch.float32)
    b = sc.get("b", (16,), torch.bfloat16)
    a.fill_(1.0)
    b.fill_(2.0)
    assert sc.check_canaries() == []
    sc._raw["b"][16] = 7.0                      # one element past the buffer
    assert sc.check_canaries() == ["b"]
    big = sc.get("a", (64, 8), torch.float32)   # growth keeps the old buffer retired and re-arms the canary
    big.zero_()
    assert "a" not in sc.check_canaries() and len(sc.retired) == 1
    assert _Scratch(torch.device("cpu"), canaries=False).check_canaries() == []


def test_hot_vocab_rows_setting_and_recent_miss_rule():
    """The draft head slice: setting resolution, and the per-request rule that reads committed tokens only."""
    from hipengine_b200.speculative.draft_vocab import (DEFAULT_ROWS, DraftVocabBook, DraftVocabRule,
                                                        resolve_hot_vocab_rows)
    assert resolve_hot_vocab_rows("off", 248320) == 0 and resolve_hot_vocab_rows(None, 248320) == 0
    assert resolve_hot_vocab_rows("auto", 248320) == DEFAULT_ROWS
    assert resolve_hot_vocab_rows("auto", 2048) == 1024             # a slice that covers everything is no slice
    assert resolve_hot_vocab_rows("1000", 2048) == 960              # whole work items
    assert resolve_hot_vocab_rows(32, 2048) == 0
    rule = DraftVocabRule(rows=100, window=8)
    prompt = [1, 2, 3, 150, 4, 5]                                   # one miss at index 3
    assert rule.catch_up(prompt, []) == 6
    assert rule.fits(5) and not rule.fits(150) and not rule.fits(-1)
    gen = [7, 120]                                                  # second miss at index 7: two inside the window
    assert rule.catch_up(prompt, gen) == 2 and not rule.fits(7)
    gen += [1] * 3
    rule.catch_up(prompt, gen)
    assert not rule.fits(1)                                         # miss at 3 is among the last 8 of 11 scanned
    gen += [1]
    rule.catch_up(prompt, gen)
    assert rule.fits(1)                                             # 3 + 8 < 12: only one miss left in the window
    assert rule.catch_up(prompt, gen) == 0                          # append-only: nothing new, nothing read
    assert rule.catch_up([1, 2], []) == 2 and rule.fits(2)          # a shorter history is another request
    book = DraftVocabBook(rows=100, window=8)
    fits = [book.fits("a", [1, 2, 3], [], 3), book.fits("b", [1, 200, 300], [], 3)]
    assert fits == [True, False] and book.decide(fits) is False and book.decide(fits[:1]) is True
    assert book.as_dict()["small_head_cycles"] == 1 and book.as_dict()["full_head_cycles"] == 1 and len(book) == 2
    book.drop("a")
    book.clear()
    assert len(book) == 0


def test_gemma4_assistant_head_pairing_artifact_round_trip_and_reference(tmp_path):
    """The assistant (MTP) head: pairing checks, GGUF round trip with validation, and properties of the fp32
    reference that the specification states (same position and keys for every step of a draft, the backbone's
    embedding table on the way in, a sliding block sees the last window - 1 keys)."""
    from dataclasses import replace
    import torch
    from hipengine_b200.loading.gemma4 import (assistant_tensor_names, build_random_assistant, load_assistant_gguf,
                                                validate_assistant)
    from hipengine_b200.loading.synth import build_random_model, write_gguf
    from hipengine_b200.models.config import (GEMMA4_26B_A4B, GEMMA4_26B_ASSISTANT, TINY_GEMMA4,
                                              TINY_GEMMA4_ASSISTANT, TINY_HYBRID)
    from hipengine_b200.ref.gemma4 import AssistantRef
    from hipengine_b200.ref.model import RefModel, RefState
    GEMMA4_26B_ASSISTANT.check_pairing(GEMMA4_26B_A4B)
    assert [GEMMA4_26B_ASSISTANT.backbone_layer(i, GEMMA4_26B_A4B) for i in range(4)] == [28, 28, 28, 29]
    with pytest.raises(ValueError, match="not gemma4"):
        TINY_GEMMA4_ASSISTANT.check_pairing(TINY_HYBRID)
    with pytest.raises(ValueError, match="backbone width"):
        replace(TINY_GEMMA4_ASSISTANT, backbone_hidden=512).check_pairing(TINY_GEMMA4)
    hw = build_random_assistant(TINY_GEMMA4_ASSISTANT, TINY_GEMMA4, seed=2, std=0.05)
    assert sorted(hw.tensors) == sorted(assistant_tensor_names(TINY_GEMMA4_ASSISTANT)) and len(hw.tensors) == 48
    path = write_gguf(hw, tmp_path / "assistant.gguf")
    back = load_assistant_gguf(path, TINY_GEMMA4)
    assert replace(back.config, rms_eps=1e-6) == TINY_GEMMA4_ASSISTANT            # eps travels as fp32
    assert all(torch.equal(back[n].raw.reshape(-1), hw[n].raw.reshape(-1)) for n in hw.tensors)
    broken = type(hw)(hw.config, {k: v for k, v in hw.tensors.items() if k != "blk.2.attn_q.weight"}, hw.metadata)
    with pytest.raises(ValueError, match="missing blk.2.attn_q.weight"):
        validate_assistant(broken, TINY_GEMMA4)
    # ---- reference behaviour
    w = build_random_model(TINY_GEMMA4, seed=1, std=0.05)
    ref = RefModel(w)
    st = RefState()
    toks = torch.randint(0, 2048, (40,), generator=torch.Generator().manual_seed(0))
    h = ref._gemma.forward_raw(toks, st)
    k_before = {i: t.clone() for i, t in st.k.items()}
    ar = AssistantRef(hw, ref._gemma)
    lg, hn = ar.step(7, h[-1], st)
    assert lg.shape == (2048,) and hn.shape == (256,) and torch.isfinite(lg).all()
    assert st.pos == 40 and all(torch.equal(st.k[i], k_before[i]) for i in st.k)       # the head writes no KV
    d1 = ar.draft(7, h[-1], st, 3)
    assert d1 == ar.draft(7, h[-1], st, 3) and len(d1) == 3                          # stateless: same draft again
    lg2, _ = ar.step(8, h[-1], st)
    assert not torch.allclose(lg, lg2)                                                # the token matters
    # keys older than the window do not reach a sliding block; the full block still sees them
    st2 = st.clone()
    st2.k[4][:8] += 5.0                    # layer n-2 (sliding, window 32): rows 0..7 are outside (40-32, 40]
    lg3, _ = ar.step(7, h[-1], st2)
    assert torch.allclose(lg, lg3)
    st2.k[4][9] += 5.0                     # key 9 = position - window + 1: the oldest one a sliding block sees
    lg4, _ = ar.step(7, h[-1], st2)
    assert not torch.allclose(lg, lg4)
    st3 = st.clone()
    st3.k[5][:8] += 5.0                    # layer n-1 (full attention)
    lg5, _ = ar.step(7, h[-1], st3)
    assert not torch.allclose(lg, lg5)


def test_speculative_options_reach_the_engine_config():
    """--mtp-hot-vocab / --draft-model / the gemma4_mtp provider name travel from the flags and the LLM keywords
    into the speculative configuration the runner reads."""
    from hipengine_b200.llm import LLM
    from hipengine_b200.server.__main__ import build_parser
    a = build_parser().parse_args(["--model", "tiny-dense", "--speculative-mtp-serving", "on", "--speculative-provider",
                                   "gemma4_mtp", "--draft-model", "/models/mtp-head.gguf", "--mtp-hot-vocab", "auto"])
    assert (a.speculative_provider, a.draft_model, a.mtp_hot_vocab) == ("gemma4_mtp", "/models/mtp-head.gguf", "auto")
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=128,
              speculative_mtp_serving="on", speculative_provider="gemma4_mtp", draft_model="/models/mtp-head.gguf",
              mtp_hot_vocab=4096)
    try:
        sc = llm.config.speculative
        assert (sc.mode, sc.draft_model, sc.hot_vocab) == ("gemma4_mtp", "/models/mtp-head.gguf", "4096")
    finally:
        llm.close()
    off = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=128)
    try:
        assert off.config.speculative.mode == "off" and off.config.speculative.draft_model is None
    finally:
        off.close()


def test_log_style_formatter_load_timing_rows_and_startup_summary():
    import logging
    from hipengine_b200.server import log_style as L
    assert L.want_color("always", False) and not L.want_color("auto", False) and not L.want_color("never", True)
    rec = logging.LogRecord("he.server", logging.WARNING, __file__, 1, "pool at %d%%", (93,), None)
    plain, col = L.StyledFormatter(False).format(rec), L.StyledFormatter(True).format(rec)
    assert plain.endswith("WARNING he.server: pool at 93%") and "\x1b[" not in plain
    assert "\x1b[33m" in col and "pool at 93%" in col and col.endswith("pool at 93%")
    assert L.human_bytes(15 * 2 ** 30) == "15.00 GiB" and L.human_bytes(512) == "512 B" and L.human_bytes(None) == "-"
    startup = {"stages": [{"name": "load_weights", "seconds": 3.0, "ok": True},
                          {"name": "build_engine", "seconds": 1.0, "ok": False}],
               "error": "build_engine: RuntimeError: x", "memory": {"device_free_bytes": 2 ** 36,
                                                                     "device_total_bytes": 3 * 2 ** 36},
               "warmup_complete": False}
    rows = L.load_timing_rows(startup)
    assert rows[0] == "LOAD_TIMING stage=load_weights seconds=3.000 share=75.0% ok"
    assert rows[1].endswith("FAILED") and rows[2].startswith("LOAD_TIMING total seconds=4.000") and "error=" in rows[2]
    cap = {"max_context": 8192, "max_slots": 8, "weight_bytes": 15 * 2 ** 30, "kv_bytes_per_token": 65536,
           "kv_pool": {"pages_total": 4096, "page_tokens": 16},
           "speculative": {"provider": "nextn_mtp", "max_depth": 3, "graph_capture": True, "draft_head_rows": 98304}}
    text = "\n".join(L.startup_summary("qwen", "cuda_sm100a", cap, startup, {"tensor_parallel": 8, "prefix_cache": "off",
                                                                               "draft_model": None}))
    assert "weights 15.00 GiB" in text and "KV pool 4096 pages x 16 tokens (4.00 GiB)" in text
    assert "speculative provider nextn_mtp depth 3 (one graph per cycle), draft head slice 98304 rows" in text
    assert "option tensor_parallel=8" in text and "prefix_cache" not in text and "draft_model" not in text
    assert "64.00 GiB free of 192.00 GiB" in text and "not warmed up" in text
    L.install("INFO", False)
    L.install("INFO", False)                                  # idempotent: one styled handler, not two
    assert sum(1 for h in logging.getLogger().handlers if getattr(h, "_he_styled", False)) == 1
    for h in [h for h in logging.getLogger().handlers if getattr(h, "_he_styled", False)]:
        logging.getLogger().removeHandler(h)


def test_nvml_sampler_against_a_fake_nvml_reads_only():
    """Memory / clock / power / throttle-reason sampling over an injected NVML: peaks and medians are reported, only
    getters are ever called, and a box without a driver yields an error string instead of an exception."""
    import time
    from types import SimpleNamespace
    from hipengine_b200.utils.nvml_sampler import NvmlSampler, decode_reasons

    class FakeNvml:
        def __init__(self):
            self.calls, self.n = [], 0

        def __getattr__(self, name):                       # any setter (or unknown call) would land here
            raise AssertionError(f"unexpected NVML call {name}")

        def nvmlInit(self): self.calls.append("init")
        def nvmlShutdown(self): self.calls.append("shutdown")
        def nvmlDeviceGetHandleByIndex(self, i): return ("h", i)
        def nvmlDeviceGetMaxClockInfo(self, h, kind): return 1965

        def nvmlDeviceGetMemoryInfo(self, h):
            self.n += 1
            return SimpleNamespace(used=(10 + self.n) << 30, total=180 << 30)

        def nvmlDeviceGetClockInfo(self, h, kind): return 1965 if self.n % 2 else 1500
        def nvmlDeviceGetPowerUsage(self, h): return 985000
        def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 0x4 if self.n > 1 else 0x1

    fake = FakeNvml()
    s = NvmlSampler(device_index=3, interval_s=0.01, nvml=fake).start()
    deadline = time.time() + 5
    while len(s.samples) < 4 and time.time() < deadline:
        time.sleep(0.01)
    s.stop()
    rep = s.summary()
    assert rep["samples"] >= 4 and rep["mem_peak_bytes"] == (10 + rep["samples"]) << 30
    assert rep["sm_max_mhz"] == 1965 and rep["sm_min_mhz"] == 1500 and rep["power_w"] == 985.0
    assert rep["reasons"] == ["sw_power_cap"] and rep["rejecting_reasons"] == []
    assert fake.calls == ["init", "shutdown"]
    assert decode_reasons(0x8 | 0x40 | 0x1) == ["hw_slowdown", "hw_thermal_slowdown"]

    class NoDriver:
        def nvmlInit(self): raise RuntimeError("driver not loaded")
    with NvmlSampler(nvml=NoDriver()) as dead:
        pass
    assert dead.summary()["samples"] == 0 and "driver not loaded" in dead.summary()["error"]


def test_command_line_dispatch(capsys):
    from hipengine_b200 import __version__, cli
    assert cli.main(["version"]) == 0 and __version__ in capsys.readouterr().out
    assert cli.main([]) == 0 and "serve" in capsys.readouterr().out
    assert cli.main(["nonsense"]) == 2
    for argv in (["bench", "serving", "--help"], ["serve", "--help"], ["chat", "--help"], ["router", "--help"],
                 ["bench", "micro", "--help"], ["bench", "--help"]):
        with pytest.raises(SystemExit) as ei:
            cli.main(argv)
        assert ei.value.code == 0, argv
        assert "usage" in capsys.readouterr().out.lower()


def test_scheduler_policies_trade_first_token_latency_against_decode_smoothness():
    """Under a burst of long prompts arriving while others decode, `protect_ttft` must reach first tokens sooner and
    `protect_decode` must keep the inter-token latency tail lower; every policy produces the same tokens."""
    import random

    def run(policy, **kw):
        cfg = EngineConfig(max_sequence_length=8192,
                           scheduler=SchedulerConfig(policy=policy, max_active_requests=16, max_pending_requests=256,
                                                     max_prefill_chunk_tokens=1024, round_prefill_token_budget=1024,
                                                     **kw),
                           kv=KVConfig(prefix_cache="off"))
        rng = random.Random(5)
        reqs = [GenerationRequest(prompt_token_ids=[rng.randrange(1000) for _ in range(rng.randrange(1500, 4000))],
                                  max_tokens=96, ignore_eos=True) for _ in range(24)]
        res = run_load_scenario(cfg, reqs, poisson_arrivals(24, rate_per_s=12.0, seed=2), max_concurrent=16)
        assert res.completed == 24 and res.total_tokens == 24 * 96
        return res.summary()

    dec, ttft = run("protect_decode"), run("protect_ttft")
    fair, budget = run("fair", fair_prefill_burst_chunks=2), run("token_budget", round_decode_row_budget=8)
    assert ttft["ttft_p50_ms"] < dec["ttft_p50_ms"], (ttft, dec)
    assert dec["itl_p99_ms"] <= ttft["itl_p99_ms"], (dec, ttft)
    for s in (fair, budget):
        assert s["tokens"] == dec["tokens"] and s["ttft_p99_ms"] > 0 and s["itl_p50_ms"] > 0
    assert min(dec["ttft_p50_ms"], ttft["ttft_p50_ms"]) <= fair["ttft_p50_ms"] <= max(dec["ttft_p99_ms"], ttft["ttft_p99_ms"])


def test_model_family_declarations_cover_the_loader_and_describe_a_geometry():
    from hipengine_b200.loading.model_loader import SUPPORTED_ARCHS
    from hipengine_b200.models.config import GEMMA4_26B_A4B, NAMED_CONFIGS, QWEN35_27B
    from hipengine_b200.models.registry import plugin_for, supported_architectures
    assert sorted(SUPPORTED_ARCHS) == supported_architectures()            # every loadable architecture is declared
    d = plugin_for("qwen35").describe(QWEN35_27B)
    assert d["layers"] == {"full": 16, "linear": 48} and d["ffn"] == "dense" and "mtp" not in d["speculative_providers"]
    assert "mtp" in plugin_for("qwen35").describe(NAMED_CONFIGS["qwen35-27b-mtp"])["speculative_providers"]
    g = plugin_for("gemma4").describe(GEMMA4_26B_A4B)
    assert g["layers"] == {"global": 5, "sliding": 25} and g["ffn"] == "moe" and g["chat_template"] == "gemma"
    assert "gemma4_mtp" in g["speculative_providers"] and g["tensor_parallel"] is False
    with pytest.raises(KeyError, match="supported"):
        plugin_for("mamba")
    import importlib
    for arch in supported_architectures():
        mod, cls = plugin_for(arch).executor.rsplit(".", 1)
        assert hasattr(importlib.import_module(mod), cls)


def test_server_entry_point_prints_its_resolved_configuration(capsys):
    import json
    from hipengine_b200.server.__main__ import main
    rc = main(["--model", "tiny-dense", "--info", "--kv-storage", "int8", "--prefill-decode-policy", "fair",
               "--max-active-requests", "3", "--batch-window-ms", "1.5", "--speculative-mtp-serving", "auto",
               "--mtp-hot-vocab", "auto", "--log-color", "never"])
    assert rc == 0
    doc = json.loads(capsys.readouterr().out)
    assert doc["engine"]["kv"]["storage"] == "int8" and doc["engine"]["scheduler"]["policy"] == "fair"
    assert doc["engine"]["scheduler"]["max_active_requests"] == 3 and doc["server"]["batch_window_ms"] == 1.5


def test_radix_cache_compatibility_key_ttl_tenant_quota_and_snapshot_matches():
    from hipengine_b200.kvcache.radix import PrefixCompatibilityKey, RadixCache
    now = [100.0]
    key = PrefixCompatibilityKey(model="m", quant="q4_k_m")
    rc = RadixCache(page_tokens=4, compat=key, ttl_seconds=10.0, tenant_quota_pages=3, clock=lambda: now[0])
    retained, freed = [], []
    rc.on_retain = retained.extend
    rc.on_snapshot_free = freed.append
    toks = list(range(20))
    assert rc.insert(toks, [11, 12, 13, 14, 15], snapshots={8: 70}, tenant="a") == 3       # quota: three pages only
    assert retained == [11, 12, 13] and rc.tenant_pages["a"] == 3
    m = rc.match(toks + [99])
    assert m.tokens == 12 and m.pages == [11, 12, 13]
    assert rc.match(toks[:12]).tokens == 8                     # never the whole prompt: one token must remain
    snap = rc.match(toks + [99], require_snapshot=True)
    assert snap.tokens == 8 and snap.snapshot == 70            # the deepest boundary that carries recurrent state
    assert rc.match(toks + [99], compat=PrefixCompatibilityKey(model="m", quant="q8_0")).tokens == 0
    assert rc.match(toks + [99], compat=key).tokens == 12
    assert rc.insert(toks, [21, 22, 23], snapshots={8: 71}, tenant="b") == 0 and freed == [71]   # duplicates are given back
    assert rc.insert([50, 51, 52, 53, 54], [31], tenant="b") == 1 and rc.tenant_pages["b"] == 1  # b has its own quota
    now[0] += 11.0
    assert rc.match(toks + [99]).tokens == 0                   # entries older than the TTL are not served
    st = rc.snapshot_stats()
    assert st["hits"] == 4 and st["lookups"] == 6
    rc.assert_consistent()
