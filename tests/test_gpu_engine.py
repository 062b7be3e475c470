"""LLM API on the sm_100a backend: continuous batching, prefix-cache hits with recurrent-state snapshots,
sampling modes, and agreement with the CPU reference engine."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    from dataclasses import replace
    from hipengine_b200 import LLM
    from hipengine_b200.config import EngineConfig, KVConfig
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    w = build_random_model(TINY_HYBRID, seed=2, std=0.05)
    cfg = EngineConfig(kv=KVConfig(snapshot_interval_tokens=64, max_snapshots=4))
    llm = LLM(w.to("cuda"), backend="cuda_sm100a", max_active_requests=4, max_sequence_length=512,
              engine_config=cfg)
    cpu = LLM(w, backend="cpu_reference", max_active_requests=4, max_sequence_length=512)
    yield llm, cpu
    llm.close()
    cpu.close()


def test_greedy_agrees_with_cpu_reference_engine(setup):
    from hipengine_b200 import SamplingParams
    llm, cpu = setup
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 17)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = llm.generate_detailed(prompts, sp)
    b = cpu.generate_detailed(prompts, sp)
    agree = sum(x == y for oa, ob in zip(a, b) for x, y in zip(oa.token_ids, ob.token_ids))
    assert agree >= 14, (agree, [o.token_ids for o in a], [o.token_ids for o in b])   # 18 tokens; near-ties may flip
    assert all(o.finish.reason == "length" for o in a)


def test_prefix_cache_hit_restores_recurrent_state(setup):
    from hipengine_b200 import SamplingParams
    llm, _ = setup
    g = torch.Generator().manual_seed(6)
    shared = torch.randint(0, 2048, (130,), generator=g).tolist()
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    first = llm.generate_detailed(shared + [11, 12, 13], sp)[0]
    again = llm.generate_detailed(shared + [11, 12, 13], sp)[0]
    other = llm.generate_detailed(shared + [99, 98], sp)[0]
    assert first.telemetry.cached_prompt_tokens == 0
    assert again.telemetry.cached_prompt_tokens == 128      # two 64-token snapshot boundaries
    assert other.telemetry.cached_prompt_tokens == 128
    assert again.token_ids == first.token_ids               # resumed from the snapshot: identical continuation
    cap = llm.resident_capacity_estimate()
    assert cap["prefix_cache"]["hits"] >= 2
    assert cap["kv_pool"]["pages_cached"] >= 8


def test_sampled_and_processed_rows_share_a_batch(setup):
    from hipengine_b200 import SamplingParams
    llm, _ = setup
    sps = [SamplingParams(max_tokens=5, ignore_eos=True),
           SamplingParams(max_tokens=5, temperature=0.8, top_k=20, seed=7, ignore_eos=True),
           SamplingParams(max_tokens=5, logit_bias={33: 100.0}, ignore_eos=True),
           SamplingParams(max_tokens=5, logprobs=True, top_logprobs=2, ignore_eos=True)]
    outs = llm.generate_detailed([[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11]], sps)
    assert outs[2].token_ids == [33] * 5
    assert len(outs[3].logprobs) == 5 and outs[3].logprobs[0].top[0][0] == outs[3].token_ids[0]
    assert all(len(o.token_ids) == 5 for o in outs)
    streamed = [t for c in llm.stream_detailed([1, 2, 3], sps[0]) for t in c.token_ids]
    assert streamed == outs[0].token_ids


def test_pool_is_conserved_after_traffic(setup):
    llm, _ = setup
    eng = llm._get_engine()
    runner = eng.loop.runner
    runner.pool.assert_conserved()
    runner.radix.assert_consistent()
    assert len(runner.free_slots) == runner.max_slots


def test_mtp_serving_matches_plain_greedy_and_reports_cycles():
    """Speculative MTP through the public API: same greedy tokens as the autoregressive engine, with cycles,
    drafted and accepted counts in the telemetry."""
    from dataclasses import replace
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    w = build_random_model(replace(TINY_HYBRID, nextn_layers=1), seed=4, std=0.05).to("cuda")
    plain = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off")
    spec = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off",
               speculative_mtp_serving="on", speculative_candidate_budget=3)
    try:
        g = torch.Generator().manual_seed(9)
        prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (12, 31)]
        sp = SamplingParams(max_tokens=14, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert x.token_ids == y.token_ids
            assert len(y.token_ids) == 14 and y.finish.reason == "length"
        assert all(o.telemetry.speculative_cycles >= 1 and o.telemetry.speculative_drafted >= 3 for o in b)
        assert all(o.telemetry.speculative_cycles == 0 for o in a)
        # sampled requests go through the exact accept kernel and still respect the length budget
        s = spec.generate_detailed(prompts[:1], SamplingParams(max_tokens=9, temperature=0.8, seed=3, ignore_eos=True))[0]
        assert len(s.token_ids) == 9 and all(0 <= t < 2048 for t in s.token_ids)
    finally:
        plain.close()
        spec.close()


def test_mtp_hot_vocab_serving_keeps_greedy_tokens_and_counts_head_choices():
    """The hot-vocabulary draft head through the public API: the per-request rule picks the head cycle by cycle,
    the tokens stay those of plain greedy decoding, and finished requests leave no rule behind."""
    from dataclasses import replace
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    w = build_random_model(replace(TINY_HYBRID, nextn_layers=1), seed=4, std=0.05).to("cuda")
    plain = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off")
    spec = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off",
               speculative_mtp_serving="on", speculative_candidate_budget=3, mtp_hot_vocab=1536)
    try:
        g = torch.Generator().manual_seed(11)
        prompts = [torch.randint(0, 1536, (n,), generator=g).tolist() for n in (12, 31)]     # inside the slice
        sp = SamplingParams(max_tokens=14, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert x.token_ids == y.token_ids
        runner = spec._get_engine().loop.runner
        book = runner.draft_vocab
        assert book is not None and book.rows == 1536 and len(book) == 0
        st = book.as_dict()
        assert st["small_head_cycles"] + st["full_head_cycles"] >= 1
        assert runner.capacity()["speculative"]["draft_head_rows"] == 1536
        assert runner.snapshot()["draft_vocab"]["rows"] == 1536
    finally:
        plain.close()
        spec.close()


def test_cold_tier_brings_an_evicted_prefix_back():
    """A small pool forces the radix cache to evict the first prompt's blocks; with the cold tier on they are
    offloaded (KV rows + recurrent-state snapshots) and restored at the next admission, and the continuation is the
    one the first run produced."""
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.config import EngineConfig, KVConfig
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    w = build_random_model(TINY_HYBRID, seed=2, std=0.05).to("cuda")
    cfg = EngineConfig(kv=KVConfig(snapshot_interval_tokens=64, max_snapshots=8, pool_pages=41,
                                   cold_restore_prefill_tok_s=1.0))
    llm = LLM(w, backend="cuda_sm100a", max_active_requests=1, max_sequence_length=256, engine_config=cfg,
              kv_cold_tier_bytes=256 << 20)
    try:
        g = torch.Generator().manual_seed(16)
        first_prompt = torch.randint(0, 2048, (140,), generator=g).tolist()
        sp = SamplingParams(max_tokens=4, ignore_eos=True)
        first = llm.generate_detailed(first_prompt, sp)[0]
        runner = llm._get_engine().loop.runner
        assert runner.cold is not None
        for _ in range(6):                                   # other traffic: pushes the first prompt out of the pool
            llm.generate_detailed(torch.randint(0, 2048, (200,), generator=g).tolist(), sp)
        assert runner.stats.get("cold_offloaded_blocks", 0) >= 8
        assert runner.radix.match(first_prompt, require_snapshot=True).tokens == 0     # really gone from the pool
        again = llm.generate_detailed(first_prompt, sp)[0]
        assert runner.stats.get("cold_restored_tokens", 0) >= 64
        assert again.telemetry.cached_prompt_tokens in (64, 128)
        assert again.token_ids == first.token_ids
        runner.pool.assert_conserved()
    finally:
        llm.close()


def test_status_word_of_a_failed_device_wait_makes_the_engine_unhealthy():
    """A kernel whose bounded wait gave up records a status code and skips its update.  The serving path reads that
    word with every per-step read-back: the request fails, the service turns unhealthy and refuses new work (the
    code is injected on the host here: nothing on the device waits or faults)."""
    from hipengine_b200 import LLM, SamplingParams
    from hipengine_b200.generation.engine_service import EngineUnavailable
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_HYBRID
    from hipengine_b200.ops import kernels as K
    w = build_random_model(TINY_HYBRID, seed=3, std=0.05)
    llm = LLM(w.to("cuda"), backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256)
    try:
        ok = llm.generate_detailed([1, 2, 3, 4], SamplingParams(max_tokens=3, ignore_eos=True))[0]
        assert len(ok.token_ids) == 3
        K.status_tensor("cuda")[0] = 1            # what comm_push_reduce / the GEMM pipelines write on a timeout
        torch.cuda.synchronize()
        bad = llm.generate_detailed([5, 6, 7, 8], SamplingParams(max_tokens=4, ignore_eos=True))[0]
        assert bad.finish.reason == "error" and "status" in (bad.error or "").lower(), (bad.finish, bad.error)
        assert int(K.status_tensor("cuda")[0].item()) == 0          # consumed
        with pytest.raises(EngineUnavailable):
            llm.generate_detailed([9, 10], SamplingParams(max_tokens=2))
    finally:
        K.status_tensor("cuda").zero_()
        llm.close()
