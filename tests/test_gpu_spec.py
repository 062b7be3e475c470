"""NextN draft block, speculative accept kernels and the whole MTP cycle on the GPU."""
from dataclasses import replace

import pytest
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_HYBRID
from hipengine_b200.ref import ops as R
from hipengine_b200.ref.model import RefModel, RefState

pytestmark = pytest.mark.gpu

CFG = replace(TINY_HYBRID, nextn_layers=1)


def _prompt(n, seed=3):
    return torch.randint(0, CFG.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("n", [6, 40], ids=["gemv", "gemm"])
def test_nextn_block_matches_reference(n):
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    from hipengine_b200.ops import kernels as K
    w = build_random_model(CFG, seed=0, std=0.05)
    ref = RefModel(w)
    ex = HybridExecutor(w.to("cuda"), max_slots=1, max_context=128)
    toks = _prompt(n)
    st = RefState()
    hid_ref = ref.forward_hidden(torch.tensor(toks), st)                 # post-norm hiddens [n, H]
    dstate = RefState()
    want = []
    zero = torch.zeros(CFG.hidden)
    for j in range(n):                                                   # row j: token j with the hidden of j-1
        lg, _ = ref.nextn_step(toks[j], hid_ref[j - 1] if j else zero, j, dstate)
        want.append(lg)
    want = torch.stack(want)
    # position 0 has no predecessor: both sides feed a zero hidden there (what the runner does after a prefill)
    b = make_batch([(0, 0, toks)], "cuda")
    hprev = torch.cat([zero[None], hid_ref[:-1]]).cuda().contiguous()
    h = ex.nextn_forward(b, hprev)
    got = torch.cat([ex.nextn_logits(h[r0:r0 + 8]).clone() for r0 in range(0, n, 8)]).cpu()
    rel = ((got - want).abs().max() / want.std()).item()
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean().item()
    assert torch.isfinite(got).all() and rel < 0.4 and agree >= 0.8, (rel, agree)


def test_greedy_accept_kernel():
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.speculative.sampling import greedy_accept
    g = torch.Generator().manual_seed(0)
    Rr, Kd = 64, 3
    tgt = torch.randint(0, 4, (Rr, Kd + 1), generator=g)
    dr = torch.randint(0, 4, (Rr, Kd), generator=g)
    dr[:8] = tgt[:8, :Kd]                                                # some fully accepted chains
    n_acc = torch.zeros(Rr, dtype=torch.int32, device="cuda")
    out = torch.zeros(Rr, Kd + 1, dtype=torch.int64, device="cuda")
    K.spec_accept_greedy(dr.cuda(), tgt.cuda(), n_acc, out)
    for r in range(Rr):
        n, emitted = greedy_accept(dr[r].tolist(), tgt[r].tolist())
        assert int(n_acc[r]) == n
        assert out[r].tolist() == emitted + [-1] * (Kd - n)


def test_sampled_accept_kernel_preserves_target_distribution():
    from hipengine_b200.ops import kernels as K
    g = torch.Generator().manual_seed(1)
    V, Kd, Rr = 32, 2, 8192
    p_row = torch.randn(Kd + 1, V, generator=g) * 1.5
    drafts_one = torch.tensor([int(p_row[0].argmax()), int(p_row[1].argmax())])    # greedy drafts: q is a point mass
    p = p_row[None].expand(Rr, -1, -1).contiguous().cuda()
    dr = drafts_one[None].expand(Rr, -1).contiguous().cuda()
    temp = torch.ones(Rr, device="cuda")
    seed = torch.arange(Rr, dtype=torch.int64, device="cuda") * 7919 + 13
    ctr = torch.zeros(Rr, dtype=torch.int64, device="cuda")
    n_acc = torch.zeros(Rr, dtype=torch.int32, device="cuda")
    out = torch.zeros(Rr, Kd + 1, dtype=torch.int64, device="cuda")
    K.spec_accept_sampled(p, None, dr, temp, seed, ctr, n_acc, out)
    first = out[:, 0].cpu()
    hist = torch.bincount(first, minlength=V).float() / Rr
    torch.testing.assert_close(hist, torch.softmax(p_row[0], -1), atol=0.02, rtol=0)
    # second emitted token, among chains whose first draft was accepted, follows p_1
    acc = (n_acc.cpu() >= 1)
    second = out[acc.cuda(), 1].cpu()
    hist2 = torch.bincount(second, minlength=V).float() / max(1, int(acc.sum()))
    torch.testing.assert_close(hist2, torch.softmax(p_row[1], -1), atol=0.04, rtol=0)
    assert bool(((out >= -1) & (out < V)).all())


def _greedy_reference_tokens(w, prompt, n_new):
    from hipengine_b200.models.executor import HybridExecutor
    ex = HybridExecutor(w, max_slots=1, max_context=256)
    lg = ex.prefill(0, prompt)
    toks = [int(lg.argmax(-1))]
    for i in range(n_new - 1):
        lg = ex.forward_logits(0, [toks[-1]], len(prompt) + i)
        toks.append(int(lg.argmax(-1)))
    return toks


@pytest.mark.parametrize("mode", ["drafted", "all_accepted", "partly_accepted"])
def test_mtp_cycle_reproduces_greedy_decode(mode):
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    from hipengine_b200.speculative.mtp import MTPCycle
    w = build_random_model(CFG, seed=0, std=0.05).to("cuda")
    prompt = _prompt(24, seed=5)
    n_new = 17
    want = _greedy_reference_tokens(w, prompt, n_new)
    ex = HybridExecutor(w, max_slots=2, max_context=256)
    mtp = MTPCycle(ex, max_depth=3, max_requests=2)
    slot = 1
    b = make_batch([(slot, 0, prompt)], "cuda")
    h = ex.forward(b)
    mtp.after_prefill(b, h)
    got = [int(ex.logits(h[b.T - 1:b.T]).argmax(-1))]
    assert got[0] == want[0]
    accepted_total = 0
    while len(got) < n_new:
        pos = len(prompt) + len(got) - 1                 # position of the last committed token
        override = None
        if mode != "drafted":
            nxt = want[len(got):len(got) + 3]
            nxt = nxt + [0] * (3 - len(nxt))
            if mode == "partly_accepted":
                nxt[1] = (nxt[1] + 1) % CFG.vocab        # second draft wrong: exactly one draft is accepted
            override = torch.tensor([nxt])
        res, txn = mtp.cycle([slot], [got[-1]], [pos], 3, draft_override=override)
        assert txn.trace[-1] == "committed"
        got += res[0].tokens
        accepted_total += res[0].accepted
        if mode == "all_accepted" and len(got) + 3 < n_new:
            assert res[0].accepted == 3
        if mode == "partly_accepted" and len(got) + 3 < n_new:
            assert res[0].accepted == 1
    assert got[:n_new] == want, (got, want)
    if mode == "all_accepted":
        assert accepted_total >= 9


@pytest.mark.parametrize("n_req", [1, 2])
def test_graphed_mtp_cycle_is_one_launch_and_reproduces_greedy_decode(n_req):
    """propose -> verify -> accept -> commit -> cursor update as ONE captured graph launched through the native
    cycle launcher: tokens equal plain greedy decoding, one capture and one row install serve every cycle."""
    from hipengine_b200.core import runtime as RT
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    from hipengine_b200.speculative.mtp import GraphedMTPCycle
    w = build_random_model(CFG, seed=0, std=0.05).to("cuda")
    prompts = [_prompt(24, seed=5), _prompt(31, seed=9)][:n_req]
    n_new = 14
    want = [_greedy_reference_tokens(w, p, n_new) for p in prompts]
    ex = HybridExecutor(w, max_slots=3, max_context=256)
    mtp = GraphedMTPCycle(ex, max_depth=3, max_requests=2)
    slots = [2, 0][:n_req]
    got = []
    for slot, p in zip(slots, prompts):
        b = make_batch([(slot, 0, p)], "cuda")
        h = ex.forward(b)
        mtp.after_prefill(b, h)
        got.append([int(ex.logits(h[b.T - 1:b.T]).argmax(-1))])
    launches0 = RT._lib().he_native_graph_launches()
    cycles = 0
    while min(len(g) for g in got) < n_new:
        pos = [len(p) + len(g) - 1 for p, g in zip(prompts, got)]
        res, txn = mtp.cycle(slots, [g[-1] for g in got], pos, 3)
        assert txn.trace[-1] == "committed"
        for g, r in zip(got, res):
            assert 1 <= len(r.tokens) == r.accepted + 1 <= 4
            g += r.tokens
        cycles += 1
    for g, wv in zip(got, want):
        n = min(len(g), n_new)
        assert g[:n] == wv[:n], (g, wv)
    st = mtp.graph_stats
    assert st["captures"] == 1 and st["replays"] == cycles and st["installs"] == 1 and st["eager"] == 0
    assert RT._lib().he_native_graph_launches() - launches0 == cycles      # one native launch per cycle
    assert list(st["kernels_per_graph"].values())[0] > 20


@pytest.mark.parametrize("graphed", [False, True], ids=["eager", "graph"])
def test_hot_vocab_draft_head_scores_a_row_prefix_and_keeps_greedy_output(graphed):
    """Drafting with the leading slice of the head: the slice's logits are the full head's first rows, every draft
    lies inside the slice, the emitted tokens are still those of plain greedy decoding (verification uses the full
    head), and the graphed cycle keeps one graph per head choice."""
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    from hipengine_b200.speculative.draft_vocab import resolve_hot_vocab_rows
    from hipengine_b200.speculative.mtp import GraphedMTPCycle, MTPCycle
    rows = resolve_hot_vocab_rows(CFG.vocab // 4, CFG.vocab)
    assert 0 < rows < CFG.vocab and rows % 64 == 0
    w = build_random_model(CFG, seed=0, std=0.05).to("cuda")
    prompt = _prompt(24, seed=5)
    n_new = 14
    want = _greedy_reference_tokens(w, prompt, n_new)
    ex = HybridExecutor(w, max_slots=1, max_context=256)
    mtp = (GraphedMTPCycle if graphed else MTPCycle)(ex, max_depth=3, max_requests=1, draft_head_rows=rows)
    assert mtp.capability().as_dict()["draft_head_rows"] == rows
    b = make_batch([(0, 0, prompt)], "cuda")
    h = ex.forward(b)
    mtp.after_prefill(b, h)
    full = ex.nextn_logits(h[:4]).clone()
    part = ex.nextn_logits(h[:4], head_rows=rows).clone()
    assert part.shape == (4, rows) and torch.allclose(part, full[:, :rows], rtol=1e-5, atol=1e-6)
    got = [int(ex.logits(h[b.T - 1:b.T]).argmax(-1))]
    cycle_no = 0
    while len(got) < n_new:
        small = cycle_no % 3 != 2                           # every third cycle drafts with the full head
        res, txn = mtp.cycle([0], [got[-1]], [len(prompt) + len(got) - 1], 3, small_head=small)
        assert txn.trace[-1] == "committed"
        if graphed and small:
            assert int(mtp.drafts[0].max()) < rows
        got += res[0].tokens
        cycle_no += 1
    assert got[:n_new] == want, (got, want)
    if graphed:
        assert mtp.graph_stats["captures"] == 2 and mtp.graph_stats["eager"] == 0


def test_lookup_cycle_with_known_chains_needs_no_nextn_block():
    """Chain verify with host-supplied drafts on a checkpoint WITHOUT a NextN block: the true greedy continuation is
    accepted in full (plus the bonus token), a corrupted chain is cut at the first wrong token, and the committed
    sequence equals plain greedy decode either way."""
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    from hipengine_b200.speculative.mtp import ChainVerifyCycle
    w = build_random_model(TINY_HYBRID, seed=0, std=0.05).to("cuda")
    prompt = _prompt(24, seed=9)
    n_new = 14
    want = _greedy_reference_tokens(w, prompt, n_new)
    ex = HybridExecutor(w, max_slots=1, max_context=256)
    cyc = ChainVerifyCycle(ex, max_depth=3, max_requests=1)
    b = make_batch([(0, 0, prompt)], "cuda")
    h = ex.forward(b)
    got = [int(ex.logits(h[b.T - 1:b.T]).argmax(-1))]
    step = 0
    while len(got) < n_new:
        nxt = want[len(got):len(got) + 3]
        nxt = nxt + [0] * (3 - len(nxt))
        corrupt = step % 2 == 1
        if corrupt:
            nxt[0] = (nxt[0] + 1) % TINY_HYBRID.vocab
        res, txn = cyc.cycle_with_drafts([0], [got[-1]], [len(prompt) + len(got) - 1], [nxt])
        assert txn.trace[-1] == "committed"
        if len(got) + 4 < n_new:
            assert res[0].accepted == (0 if corrupt else 3)
        got += res[0].tokens
        step += 1
    assert got[:n_new] == want


@pytest.mark.parametrize("provider", ["prompt_lookup", "ngram"])
def test_lookup_provider_serving_matches_plain_greedy(provider):
    """The engine with a host drafter must emit exactly the tokens of the plain engine.  The n-gram provider is
    seeded with the true continuation (as if another request had produced it), so its chains are accepted."""
    from hipengine_b200 import LLM, SamplingParams
    w = build_random_model(TINY_HYBRID, seed=0, std=0.05).to("cuda")
    prompt = _prompt(12, seed=11) * 4
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    plain = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off")
    want = plain.generate_token_ids([prompt], sp)[0]
    plain.close()
    spec = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off",
               speculative_mtp_serving="on", speculative_provider=provider)
    cyc = spec._get_engine().loop.runner.mtp
    if provider == "ngram":
        cyc.drafter.span = 32
        cyc.drafter.observe(prompt + want)
    got = spec.generate_token_ids([prompt], sp)[0]
    stats = dict(cyc.stats)
    spec.close()
    assert got == want
    assert stats["cycles"] + stats["skipped_cycles"] >= 1          # the drafter was consulted
    if provider == "ngram":
        assert stats["accepted"] >= 6, stats
