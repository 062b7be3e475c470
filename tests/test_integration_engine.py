"""LLM API -> EngineService -> EngineLoop -> CpuReferenceRunner on tiny random-init models (no GPU)."""
import threading
import time

import pytest
import torch

from hipengine_b200 import LLM, SamplingParams
from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_DENSE, TINY_HYBRID
from hipengine_b200.ref.model import RefModel


@pytest.fixture(scope="module")
def dense():
    w = build_random_model(TINY_DENSE, seed=0)
    llm = LLM(w, backend="cpu_reference", max_active_requests=4, max_sequence_length=256)
    yield w, llm
    llm.close()


def test_config1_greedy_matches_fp32_reference(dense):
    w, llm = dense
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 4096, (32,), generator=g).tolist()
    out = llm.generate_detailed(prompt, SamplingParams(max_tokens=16, ignore_eos=True))[0]
    ref_tokens, ref_logits = RefModel(w).generate(prompt, 16)
    assert out.token_ids == ref_tokens
    assert out.finish.reason == "length" and out.telemetry.prompt_tokens == 32
    assert torch.isfinite(ref_logits).all()


def test_batch_of_requests_and_continuous_batching(dense):
    w, llm = dense
    prompts = [[1, 2, 3, 4], [10, 11], [100, 200, 300, 400, 500, 600], [7], [9, 9, 9]]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    outs = llm.generate_detailed(prompts, sp)
    ref = RefModel(w)
    for p, o in zip(prompts, outs):
        assert o.token_ids == ref.generate(p, 5)[0]


def test_streaming_yields_every_token_once(dense):
    _, llm = dense
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    full = llm.generate_detailed([5, 6, 7], sp)[0].token_ids
    chunks = list(llm.stream_detailed([5, 6, 7], sp))
    assert [t for c in chunks for t in c.token_ids] == full
    assert chunks[-1].finished and chunks[-1].finish.reason == "length"


def test_stop_sequences_trim_and_hold_back(dense):
    _, llm = dense
    base = llm.generate_detailed([5, 6, 7], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids
    stop = tuple(base[3:5])
    sp = SamplingParams(max_tokens=8, ignore_eos=True, stop_token_sequences=(stop,))
    out = llm.generate_detailed([5, 6, 7], sp)[0]
    first = next(i for i in range(len(base) - 1) if tuple(base[i:i + 2]) == stop)
    assert out.token_ids == base[:first] and out.finish.reason == "stop" and out.finish.stop_sequence == stop
    streamed = [t for c in llm.stream_detailed([5, 6, 7], sp) for t in c.token_ids]
    assert streamed == base[:first]
    out = llm.generate_detailed([5, 6, 7], SamplingParams(max_tokens=8, ignore_eos=True, stop_token_ids=(base[2],)))[0]
    assert out.token_ids == base[:base.index(base[2])]


def test_seeded_sampling_is_reproducible_and_seed_sensitive(dense):
    _, llm = dense
    sp = SamplingParams(max_tokens=8, temperature=1.0, top_k=50, seed=123, ignore_eos=True)
    a = llm.generate_detailed([1, 2, 3], sp)[0].token_ids
    b = llm.generate_detailed([1, 2, 3], sp)[0].token_ids
    assert a != [] and len(a) == 8
    assert a == b                                       # the same seed repeats the draw, whatever the request id
    c = llm.generate_detailed([1, 2, 3], SamplingParams(max_tokens=8, temperature=1.0, top_k=50, seed=124,
                                                        ignore_eos=True))[0].token_ids
    assert c != a                                       # another seed draws differently
    rows = llm.generate_detailed([[1, 2, 3]] * 3, sp)
    assert len({tuple(o.token_ids) for o in rows}) >= 2 and rows[0].token_ids == a    # rows of a batch are told apart
    unseeded = SamplingParams(max_tokens=8, temperature=1.0, top_k=50, ignore_eos=True)
    assert llm.generate_detailed([1, 2, 3], unseeded)[0].token_ids != llm.generate_detailed([1, 2, 3], unseeded)[0].token_ids


def test_logprobs_and_processors(dense):
    _, llm = dense
    sp = SamplingParams(max_tokens=3, logprobs=True, top_logprobs=3, ignore_eos=True)
    out = llm.generate_detailed([3, 4, 5], sp)[0]
    assert len(out.logprobs) == 3 and all(len(lp.top) == 3 for lp in out.logprobs)
    assert all(lp.logprob <= 0 for lp in out.logprobs)
    assert out.logprobs[0].top[0][0] == out.token_ids[0]
    banned = out.token_ids[0]
    out2 = llm.generate_detailed([3, 4, 5], SamplingParams(max_tokens=3, suppress_token_ids=(banned,),
                                                          ignore_eos=True))[0]
    assert banned not in out2.token_ids
    out3 = llm.generate_detailed([3, 4, 5], SamplingParams(max_tokens=2, logit_bias={17: 100.0}, ignore_eos=True))[0]
    assert out3.token_ids == [17, 17]
    out4 = llm.generate_detailed([3, 4, 5], SamplingParams(max_tokens=4, forced_tokens_pending=(9, 8),
                                                          ignore_eos=True))[0]
    assert out4.token_ids[:2] == [9, 8]


def test_context_overflow_is_rejected(dense):
    _, llm = dense
    out = llm.generate_detailed(list(range(10, 250)), SamplingParams(max_tokens=64))[0]
    assert out.finish.reason == "error" and "context_overflow" in out.error


def test_cancellation_token_and_deadline(dense):
    _, llm = dense

    class Tok:
        cancelled = False
    tok = Tok()
    sp = SamplingParams(max_tokens=200, ignore_eos=True, cancellation_token=tok)
    res = {}
    th = threading.Thread(target=lambda: res.setdefault("o", llm.generate_detailed([1, 2], sp)[0]))
    th.start()
    time.sleep(0.15)
    tok.cancelled = True
    th.join(timeout=30)
    assert res["o"].finish.reason == "cancelled" and len(res["o"].token_ids) < 200
    out = llm.generate_detailed([1, 2], SamplingParams(max_tokens=200, ignore_eos=True,
                                                      deadline_at=time.time() + 0.1))[0]
    assert out.finish.reason == "deadline_exceeded"


def test_hybrid_model_through_the_engine():
    w = build_random_model(TINY_HYBRID, seed=1)
    with LLM(w, backend="cpu_reference", max_active_requests=2, max_sequence_length=128) as llm:
        outs = llm.generate_detailed([[1, 2, 3, 4, 5], [9, 8, 7]], SamplingParams(max_tokens=4, ignore_eos=True))
        ref = RefModel(w)
        assert outs[0].token_ids == ref.generate([1, 2, 3, 4, 5], 4)[0]
        assert outs[1].token_ids == ref.generate([9, 8, 7], 4)[0]
        text = llm.generate("hi", SamplingParams(max_tokens=3))
        assert isinstance(text[0], str)
        h = llm.engine_service_health()
        assert h["healthy"] and h["driver_alive"]
        snap = llm.live_loop_snapshot()
        assert snap["counters"]["finished"] >= 3


def test_required_tool_call_is_grammar_constrained_token_by_token():
    """With a tool choice that demands a call, the in-tree grammar matcher masks the logits of every step: a random
    model (which would emit noise) produces text that is at every point a prefix of a well-formed tool call."""
    import json
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.generation.constraints import ToolCallConstraintSpec
    from hipengine_b200.generation.grammar import ToolCallAutomaton
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_DENSE
    tools = [{"type": "function", "function": {"name": "lookup", "parameters": {
        "type": "object", "properties": {"n": {"type": "integer"}, "flag": {"type": "boolean"}},
        "required": ["n", "flag"]}}}]
    llm = LLM(build_random_model(TINY_DENSE, seed=4, std=0.05), backend="cpu_reference", max_active_requests=2,
              max_sequence_length=256)
    try:
        spec = ToolCallConstraintSpec(("lookup",), "required", None, tools_json=json.dumps(tools))
        sp = SamplingParams(max_tokens=96, temperature=0.8, seed=7, tool_call_constraint=spec)
        out = llm.generate_detailed(llm.tokenize("call the tool"), sp)[0]
        text = llm._get_tokenizer().decode(out.token_ids)
        auto = ToolCallAutomaton(tools)
        s = auto.start_set
        for ch in text:
            s = auto.step(s, ch)
            assert s is not None, text          # never leaves the grammar
        free = SamplingParams(max_tokens=24, temperature=0.8, seed=7)
        noise = llm._get_tokenizer().decode(llm.generate_detailed(llm.tokenize("call the tool"), free)[0].token_ids)
        assert noise != text[:len(noise)]
        if out.finish.reason in ("stop_eos", "stop"):
            assert auto.accepting(s)
    finally:
        llm.close()


def test_llm_batches_fit_context_and_speculative_plan_helpers():
    """Host-side helpers of the public API: grouped submission of several batches, the context-fit estimate, the
    serving-plan question, and the refusal to run 'speculative' generation on an engine without a provider."""
    from hipengine_b200.llm import LLM, SamplingParams
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=4, max_sequence_length=128)
    try:
        sp = SamplingParams(max_tokens=3, ignore_eos=True)
        flat = llm.generate_detailed([[1, 2, 3], [4, 5], [6, 7, 8, 9]], sp)
        grouped = llm.submit_independent_batches_detailed([[[1, 2, 3], [4, 5]], [], [[6, 7, 8, 9]]], sp)
        assert [len(g) for g in grouped] == [2, 0, 1]
        assert [o.token_ids for g in grouped for o in g] == [o.token_ids for o in flat]
        per_batch = llm.submit_independent_batches_detailed([[[1, 2, 3]], [[4, 5]]],
                                                            [sp, SamplingParams(max_tokens=5, ignore_eos=True)])
        assert [len(g[0].token_ids) for g in per_batch] == [3, 5]
        with pytest.raises(ValueError, match="one SamplingParams per batch"):
            llm.submit_independent_batches_detailed([[[1]], [[2]]], [sp])
        fit = llm.fit_context(list(range(100)), max_tokens=40)
        assert fit == {"prompt_tokens": 100, "max_context": 128, "max_new_tokens": 28, "fits": True,
                       "fits_with_max_tokens": False}
        assert llm.fit_context("hello")["prompt_tokens"] == llm.count_tokens("hello")
        assert not llm.fit_context(list(range(128)))["fits"]
        plan = llm.resolve_speculative_mtp_serving_plan(sp)
        assert not plan.use_mtp and plan.reason == "disabled"
        with pytest.raises(ValueError, match="without a speculative provider"):
            llm.generate_speculative_detailed([[1, 2, 3]], sp)
        chunks = list(llm.stream_speculative_mtp_detailed([1, 2, 3], sp))       # falls back to step-by-step decoding
        assert [t for c in chunks for t in c.token_ids] == flat[0].token_ids
    finally:
        llm.close()
    spec = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=128,
               speculative_mtp_serving="on", speculative_provider="prompt_lookup")
    try:
        p = spec.resolve_speculative_mtp_serving_plan(SamplingParams(max_tokens=3))
        assert p.reason in ("ok", "no_nextn_block")                                # the CPU runner has no verifier
        assert spec.resolve_speculative_mtp_serving_plan(SamplingParams(logit_bias={5: 2.0})).reason in (
            "sampler_not_reproducible", "no_nextn_block")
    finally:
        spec.close()


def _sim_engine(spec_depth=0, accept=0.0, **kw):
    from dataclasses import replace
    from hipengine_b200.config import EngineConfig, SchedulerConfig, SpeculativeConfig
    from hipengine_b200.generation.engine_service import engine_from_runner
    from hipengine_b200.generation.simulator import SimulatedRunner
    cfg = EngineConfig(max_sequence_length=512, scheduler=SchedulerConfig(max_active_requests=4),
                       speculative=SpeculativeConfig(mode="mtp" if spec_depth else "off", draft_depth=max(spec_depth, 1)))
    runner = SimulatedRunner(cfg, spec_depth=spec_depth, spec_accept_rate=accept, **kw)
    return engine_from_runner(runner, cfg, None), runner


@pytest.mark.parametrize("accept", [0.0, 0.6, 1.0])
def test_speculative_cycles_on_the_simulated_runner_equal_plain_decoding(accept):
    """The loop's speculative path on the host: multi-token commits, clipping at max_tokens, a stop sequence and an
    EOS that fall inside a cycle, telemetry and counters -- and token-for-token equality with plain decoding."""
    from hipengine_b200.generation.types import GenerationRequest
    plain, _ = _sim_engine()
    try:
        base = plain.generate([GenerationRequest(prompt_token_ids=list(range(5, 25)), max_tokens=23, ignore_eos=True)])[0]
    finally:
        plain.close()
    cont = base.token_ids
    assert len(cont) == 23
    reqs = lambda: [
        GenerationRequest(prompt_token_ids=list(range(5, 25)), max_tokens=23, ignore_eos=True),
        GenerationRequest(prompt_token_ids=list(range(5, 25)), max_tokens=7, ignore_eos=True),
        GenerationRequest(prompt_token_ids=list(range(5, 25)), max_tokens=23, ignore_eos=True,
                          stop_token_sequences=((cont[9], cont[10]),)),
        GenerationRequest(prompt_token_ids=list(range(5, 25)), max_tokens=23, eos_token_id=cont[12]),
    ]
    plain, _ = _sim_engine()
    try:
        want = plain.generate(reqs())
    finally:
        plain.close()
    spec, runner = _sim_engine(spec_depth=3, accept=accept)
    try:
        got = spec.generate(reqs())
        for w, g in zip(want, got):
            assert g.error is None and g.token_ids == w.token_ids and g.finish.reason == w.finish.reason
        assert [len(g.token_ids) for g in got][:2] == [23, 7] and got[2].finish.reason == "stop"
        assert len(got[2].token_ids) < 23 and len(got[3].token_ids) <= 13
        full = got[0].telemetry
        assert full.speculative_cycles >= 1 and full.speculative_drafted >= 3
        if accept == 1.0:
            assert full.speculative_accepted == full.speculative_drafted or full.speculative_cycles <= 7
            assert full.speculative_cycles <= 8                    # ~4 tokens per cycle
        if accept == 0.0:
            assert full.speculative_accepted == 0
        assert all(w.telemetry.speculative_cycles == 0 for w in want)
        snap = spec.loop.snapshot()
        assert snap["counters"]["spec_cycles"] >= 4 and runner.spec_stats["cycles"] >= 1
    finally:
        spec.close()


def test_speculative_failure_is_contained_and_processed_requests_decode_step_by_step():
    from hipengine_b200.generation.types import GenerationRequest
    spec, runner = _sim_engine(spec_depth=3, accept=0.8, fail_decode_admission=[1])
    try:
        outs = spec.generate([GenerationRequest(prompt_token_ids=list(range(10 + i)), max_tokens=9, ignore_eos=True)
                              for i in range(3)])
        errs = [o for o in outs if o.error]
        assert len(errs) == 1 and "execution_failed[verify/partial]" in errs[0].error
        assert all(len(o.token_ids) == 9 for o in outs if not o.error)
        cycles_before = runner.spec_stats["cycles"]
        biased = spec.generate([GenerationRequest(prompt_token_ids=[1, 2, 3], max_tokens=6, ignore_eos=True,
                                                  logit_bias=((7, 1.5),))])[0]
        assert biased.error is None and len(biased.token_ids) == 6 and biased.telemetry.speculative_cycles == 0
        assert runner.spec_stats["cycles"] == cycles_before         # a processed request never entered a cycle
    finally:
        spec.close()


def test_load_scenario_in_virtual_time_shows_when_drafting_pays():
    """Virtual-time load over the simulated runner with the measured cycle costs: a high acceptance rate raises the
    throughput, a low one is caught by the adaptive planner (drafting stops after its observation window) so that
    it costs little."""
    from dataclasses import replace
    from hipengine_b200.config import EngineConfig, SchedulerConfig, SpeculativeConfig
    from hipengine_b200.generation.simulator import SimulatedRunner, poisson_arrivals, run_load_scenario
    from hipengine_b200.generation.types import GenerationRequest

    def run(depth, accept, adaptive=True):
        cfg = EngineConfig(max_sequence_length=2048, scheduler=SchedulerConfig(max_active_requests=4),
                           speculative=SpeculativeConfig(mode="mtp" if depth else "off", draft_depth=max(depth, 1),
                                                         adaptive_depth=adaptive))
        reqs = [GenerationRequest(prompt_token_ids=list(range(3, 3 + 64 + i)), max_tokens=400, ignore_eos=True)
                for i in range(4)]
        runner = SimulatedRunner(cfg, spec_depth=depth, spec_accept_rate=accept)
        res = run_load_scenario(cfg, reqs, poisson_arrivals(4, 50.0, seed=1), max_concurrent=4, runner=runner)
        assert res.completed == 4 and res.total_tokens == 1600
        return res.summary()["tok_per_s"], runner.spec_stats

    plain, _ = run(0, 0.0)
    good, st_good = run(3, 0.9)
    poor, st_poor = run(3, 0.2)
    stubborn, _ = run(3, 0.2, adaptive=False)
    assert good > 1.25 * plain, (good, plain)
    assert st_good["accepted"] / st_good["drafted"] > 0.8
    assert poor > 0.85 * plain and poor > 1.3 * stubborn, (poor, plain, stubborn)
    assert st_poor["fallback_steps"] > st_poor["cycles"]           # the planner stopped drafting


def test_nextn_speculative_decoding_on_the_cpu_reference_backend_equals_plain_greedy():
    """The host oracle of the NextN cycle through the public API: same tokens as plain greedy decoding for hybrid
    requests of different lengths, cycles and drafts in the telemetry, requests that are not eligible (sampled,
    biased) decode step by step on the same engine with the draft block kept in step."""
    from hipengine_b200.llm import LLM, SamplingParams
    kw = dict(backend="cpu_reference", max_active_requests=3, max_sequence_length=128, prefix_cache="off")
    plain = LLM("tiny-hybrid-mtp", **kw)
    spec = LLM("tiny-hybrid-mtp", speculative_mtp_serving="on", speculative_candidate_budget=3, **kw)
    try:
        prompts = [list(range(7, 7 + n)) for n in (5, 19)]
        sp = SamplingParams(max_tokens=11, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert y.error is None and x.token_ids == y.token_ids and len(y.token_ids) == 11
        assert all(o.telemetry.speculative_cycles >= 3 and o.telemetry.speculative_drafted >= 3 for o in b)
        assert all(o.telemetry.speculative_cycles == 0 for o in a)
        assert spec.resolve_speculative_mtp_serving_plan(sp).use_mtp
        runner = spec._get_engine().loop.runner
        assert runner.spec_stats["cycles"] >= 6 and not runner.states and not runner.draft_states
        biased = SamplingParams(max_tokens=6, ignore_eos=True, logit_bias={9: 3.0})
        assert spec.generate_detailed(prompts[:1], biased)[0].token_ids == plain.generate_detailed(prompts[:1], biased)[0].token_ids
        cycles = runner.spec_stats["cycles"]
        sampled = spec.generate_detailed(prompts[:1], SamplingParams(max_tokens=6, temperature=0.8, seed=5, ignore_eos=True))[0]
        assert len(sampled.token_ids) == 6 and runner.spec_stats["cycles"] == cycles     # sampled: no host cycle
    finally:
        plain.close()
        spec.close()


def test_gemma4_assistant_head_speculative_decoding_on_the_cpu_reference_backend():
    """The host oracle of the Gemma 4 assistant-head cycle through the public API: plain greedy tokens, cycles in the
    telemetry, the head given as loaded weights."""
    from hipengine_b200.llm import LLM, SamplingParams
    from hipengine_b200.loading.gemma4 import build_random_assistant
    from hipengine_b200.models.config import TINY_GEMMA4, TINY_GEMMA4_ASSISTANT
    hw = build_random_assistant(TINY_GEMMA4_ASSISTANT, TINY_GEMMA4, seed=6, std=0.05)
    kw = dict(backend="cpu_reference", max_active_requests=2, max_sequence_length=128, prefix_cache="off")
    plain = LLM("tiny-gemma4", **kw)
    spec = LLM("tiny-gemma4", speculative_mtp_serving="on", speculative_provider="gemma4_mtp", draft_model=hw,
               speculative_candidate_budget=2, **kw)
    try:
        prompts = [list(range(11, 11 + n)) for n in (6, 40)]                 # the second one exceeds the window
        sp = SamplingParams(max_tokens=7, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert y.error is None and x.token_ids == y.token_ids
        assert all(o.telemetry.speculative_cycles >= 2 and o.telemetry.speculative_drafted >= 2 for o in b)
        runner = spec._get_engine().loop.runner
        assert runner.assistant is not None and runner.spec_stats["cycles"] >= 4 and not runner.draft_states
    finally:
        plain.close()
        spec.close()


@pytest.mark.parametrize("provider", ["prompt_lookup", "ngram"])
def test_history_drafters_on_the_cpu_reference_backend(provider):
    """prompt_lookup / ngram on the host backend: a repetitive prompt gives proposals, the accepted ones shorten the
    run, and the tokens stay those of plain greedy decoding."""
    from hipengine_b200.llm import LLM, SamplingParams
    kw = dict(backend="cpu_reference", max_active_requests=2, max_sequence_length=256, prefix_cache="off")
    plain = LLM("tiny-dense", **kw)
    spec = LLM("tiny-dense", speculative_mtp_serving="on", speculative_provider=provider,
               speculative_candidate_budget=3, **kw)
    try:
        prompts = [[5, 6, 7, 8, 9] * 6, list(range(30, 47))]
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert y.error is None and x.token_ids == y.token_ids
        runner = spec._get_engine().loop.runner
        assert runner.lookup is not None and runner.spec_stats["cycles"] >= 1          # the repetitive prompt drafted
        assert b[0].telemetry.speculative_drafted >= 1
    finally:
        plain.close()
        spec.close()


def test_python_api_refuses_ids_outside_the_vocabulary(dense):
    _, llm = dense
    vocab = llm.vocab_size
    for prompt, sp, needle in (([1, vocab], SamplingParams(max_tokens=2), "prompt token id"),
                               ([-1, 2], SamplingParams(max_tokens=2), "prompt token id"),
                               ([], SamplingParams(max_tokens=2), "empty"),
                               ([1, 2], SamplingParams(max_tokens=2, forced_tokens_pending=(vocab + 5,)), "forced_tokens_pending"),
                               ([1, 2], SamplingParams(max_tokens=2, suppress_token_ids=(vocab,)), "suppress_token_ids"),
                               ([1, 2], SamplingParams(max_tokens=2, logit_bias={vocab: 1.0}), "logit_bias")):
        with pytest.raises(ValueError, match=needle):
            llm.generate_detailed([prompt], sp)
    assert len(llm.generate_detailed([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))[0].token_ids) == 2
    assert llm.engine_service_health()["healthy"]
