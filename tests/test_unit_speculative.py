"""Speculative decoding host logic: transaction stages, exact sampling law, depth planner, serving admission."""
import pytest
import torch

from hipengine_b200.speculative import (SpecTransaction, Stage, TransactionError, acceptance_probability,
                                        plan_draft_depth, residual_distribution, resolve_mtp_serving_plan,
                                        sampled_accept_from_distributions)
from hipengine_b200.speculative.policy import expected_tokens
from hipengine_b200.speculative.sampling import greedy_accept


def test_transaction_order_and_rollback():
    undone = []
    t = SpecTransaction([1, 2], on_rollback=lambda x: undone.append(x.stage))
    with pytest.raises(TransactionError):
        t.advance(Stage.DRAFTED)                       # cannot skip stages
    for st in (Stage.RESERVED, Stage.TARGET_OPEN, Stage.PROVIDER_OPEN, Stage.DRAFTED):
        t.advance(st)
    t.rollback()
    assert t.stage == Stage.ROLLED_BACK and undone == [Stage.DRAFTED] and t.done
    with pytest.raises(TransactionError):
        t.advance(Stage.VERIFIED)
    t2 = SpecTransaction([3], on_rollback=lambda x: undone.append("t2"))
    t2.advance(Stage.RESERVED)
    t2.cancel()                                         # nothing mutated yet: the hook must not run
    assert undone == [Stage.DRAFTED]
    t3 = SpecTransaction([4])
    for st in (Stage.RESERVED, Stage.TARGET_OPEN, Stage.PROVIDER_OPEN, Stage.DRAFTED, Stage.VERIFIED, Stage.ACCEPTED,
               Stage.READBACK, Stage.COMMITTING):
        t3.advance(st)
    with pytest.raises(TransactionError):
        t3.rollback()                                   # a commit in flight is not reversible
    t3.advance(Stage.COMMITTED)
    assert t3.trace[0] == "new" and t3.trace[-1] == "committed" and len(t3.trace) == 10


def test_greedy_accept_prefix():
    assert greedy_accept([5, 6, 7], [5, 6, 9, 1]) == (2, [5, 6, 9])
    assert greedy_accept([5, 6, 7], [4, 6, 7, 1]) == (0, [4])
    assert greedy_accept([5, 6, 7], [5, 6, 7, 8]) == (3, [5, 6, 7, 8])


def test_residual_and_acceptance():
    p = torch.tensor([0.5, 0.3, 0.2])
    q = torch.tensor([0.2, 0.6, 0.2])
    assert acceptance_probability(p, q, 0) == 1.0
    assert abs(acceptance_probability(p, q, 1) - 0.5) < 1e-6
    r = residual_distribution(p, q)
    torch.testing.assert_close(r, torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64))


def test_sampled_law_preserves_target_distribution():
    g = torch.Generator().manual_seed(0)
    V = 6
    p = torch.softmax(torch.randn(2, V, generator=g), -1)          # K = 1: rows p_0 (verify) and p_1 (bonus)
    q = torch.softmax(torch.randn(1, V, generator=g), -1)
    counts = torch.zeros(V)
    n = 20000
    u = torch.rand(n, 4, generator=g)
    draws = torch.multinomial(q[0], n, replacement=True, generator=g)
    for i in range(n):
        _, out = sampled_accept_from_distributions([int(draws[i])], p, q, u[i].tolist())
        counts[out[0]] += 1
    torch.testing.assert_close(counts / n, p[0], atol=0.015, rtol=0)


def test_planner_and_serving_rules():
    assert plan_draft_depth(3, remaining_tokens=100, context_room=100) == 3
    assert plan_draft_depth(3, remaining_tokens=2, context_room=100) == 1
    assert plan_draft_depth(3, remaining_tokens=100, context_room=1) == 0
    assert plan_draft_depth(3, 100, 100, drafted=300, accepted=0) == 0        # nothing ever accepted: stop drafting
    assert plan_draft_depth(3, 100, 100, drafted=300, accepted=270) == 3
    assert abs(expected_tokens(0.5, 2) - 1.75) < 1e-9
    from hipengine_b200.speculative.policy import break_even_accept_rate, cycle_cost
    assert abs(cycle_cost(3) - 2.32) < 1e-9                                   # measured: 2.33 autoregressive steps
    assert abs(break_even_accept_rate(1) - 0.44) < 1e-6                       # 1 + a = 1.44
    assert 0.6 < break_even_accept_rate(3) < 0.7 and break_even_accept_rate(3, 0.5, 0.6) == 1.0
    assert plan_draft_depth(3, 100, 100, drafted=300, accepted=120) == 0       # 40 % acceptance does not pay here
    assert plan_draft_depth(3, 100, 100, drafted=300, accepted=120, adaptive=False) == 3
    assert plan_draft_depth(3, 100, 100, drafted=300, accepted=180) >= 1       # 60 % does
    ok = resolve_mtp_serving_plan("on", True, 0.0, False, False, False)
    assert ok.use_mtp and ok.sampling_mode == "greedy"
    assert resolve_mtp_serving_plan("on", True, 0.7, False, False, False).sampling_mode == "sampled"
    assert not resolve_mtp_serving_plan("off", True, 0.0, False, False, False).use_mtp
    assert resolve_mtp_serving_plan("on", False, 0.0, False, False, False).reason == "no_nextn_block"
    assert resolve_mtp_serving_plan("on", True, 0.0, True, False, False).reason == "sampler_not_reproducible"
    assert resolve_mtp_serving_plan("auto", True, 0.0, False, False, False, breaker_open=True).reason == "circuit_open"


def test_prompt_lookup_and_ngram_drafters_and_registry():
    from hipengine_b200.speculative.providers import (NGramCacheDrafter, PromptLookupDrafter,
                                                      SpeculativeProviderConfig, build_speculative_provider,
                                                      register_builtin_speculative_providers,
                                                      speculative_provider_names)
    d = PromptLookupDrafter(min_ngram=2, max_ngram=3)
    hist = [5, 6, 7, 8, 9, 1, 2, 6, 7, 8]
    assert d.propose(hist, 3) == [9, 1, 2]              # "6 7 8" seen before, followed by 9 1 2
    assert d.propose([1, 2, 3, 4], 3) == []             # nothing repeats
    assert d.propose([4, 4, 4, 4], 2) == [4]            # most recent earlier match, continuation clipped by the end
    hist2 = [1, 2, 3, 9, 1, 2, 3, 7, 1, 2, 3]
    assert d.propose(hist2, 1) == [7]                   # the latest occurrence wins over the first
    g = NGramCacheDrafter(min_ngram=2, max_ngram=2, table_entries=4)
    g.observe([10, 11, 12, 13, 14])
    assert g.propose([99, 10, 11], 2) == [12, 13]       # learnt from another request
    g.observe(list(range(100, 140)))
    assert len(g.table) <= 4                            # bounded
    assert register_builtin_speculative_providers() == ["gemma4_mtp", "mtp", "ngram", "prompt_lookup"]
    assert "prompt_lookup" in speculative_provider_names()

    class _NoNextN:
        has_nextn = False
    assert build_speculative_provider(_NoNextN(), SpeculativeProviderConfig(name="mtp")) is None
    import pytest
    with pytest.raises(ValueError):
        build_speculative_provider(_NoNextN(), SpeculativeProviderConfig(name="eagle"))
