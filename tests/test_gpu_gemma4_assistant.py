"""Gemma 4 assistant (MTP) head on the GPU against its fp32 reference, and the draft / verify cycle built on it."""
import pytest
import torch

from hipengine_b200.loading.gemma4 import build_random_assistant
from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_GEMMA4, TINY_GEMMA4_ASSISTANT
from hipengine_b200.ref.gemma4 import AssistantRef
from hipengine_b200.ref.model import RefModel, RefState

pytestmark = pytest.mark.gpu


def _kl(p_logits, q_logits):
    p = torch.log_softmax(p_logits.double(), -1)
    q = torch.log_softmax(q_logits.double(), -1)
    return float((p.exp() * (p - q)).sum(-1))


def _prompt(n, seed):
    return torch.randint(0, TINY_GEMMA4.vocab, (n,), generator=torch.Generator().manual_seed(seed))


def _cached_rows(ex, layer, slot, n):
    """K and V rows 0 .. n-1 of one request read back from the executor's paged cache: [n, Hkv, D] fp32 each."""
    from hipengine_b200.models.executor import PAGE
    bt = ex.block_table[slot].cpu()
    kv = ex.kv[layer]
    ks = [kv[int(bt[p // PAGE]), 0, :, p % PAGE, :] for p in range(n)]
    vs = [kv[int(bt[p // PAGE]), 1, :, p % PAGE, :] for p in range(n)]
    return torch.stack(ks).float().cpu(), torch.stack(vs).float().cpu()


def test_assistant_head_steps_match_reference_and_write_no_kv():
    """Two requests of different lengths (one shorter than the sliding window, one longer) through three chained
    head steps: logits and the recurrent hidden follow the fp32 reference, tokens are teacher-forced to the
    reference's proposals, and the backbone's KV is bit-identical before and after (the head owns no KV).  The
    reference head is fed the K/V rows and the seed hidden the GPU backbone produced, so only the head is compared."""
    from hipengine_b200.models import make_executor
    from hipengine_b200.models.executor import make_batch
    from hipengine_b200.models.gemma4_assistant import Gemma4AssistantHead
    cfg = TINY_GEMMA4
    w = build_random_model(cfg, seed=1, std=0.05)
    hw = build_random_assistant(TINY_GEMMA4_ASSISTANT, cfg, seed=2, std=0.05)
    ref = RefModel(w)
    ar = AssistantRef(hw, ref._gemma)
    ex = make_executor(w.to("cuda"), max_slots=2, max_context=128)
    head = Gemma4AssistantHead(ex, hw)
    reqs = [(1, _prompt(40, 0)), (0, _prompt(20, 5))]
    states, seeds = [], []
    for slot, toks in reqs:
        h_gpu = ex.forward(make_batch([(slot, 0, toks.tolist())], "cuda"))
        seeds.append(h_gpu[-1].cpu().clone())
        st = RefState(pos=len(toks))
        for layer in (cfg.n_layers - 2, cfg.n_layers - 1):
            st.k[layer], st.v[layer] = _cached_rows(ex, layer, slot, len(toks))
        states.append(st)
        assert torch.isfinite(seeds[-1]).all() and st.k[cfg.n_layers - 1].shape == (len(toks), 1, 128)
    kv_before = {i: ex.kv[i].clone() for i in (cfg.n_layers - 2, cfg.n_layers - 1)}
    slot = torch.tensor([s for s, _ in reqs], dtype=torch.int32, device="cuda")
    n_past = torch.tensor([len(t) for _, t in reqs], dtype=torch.int32, device="cuda")
    tok = [7, 1500]
    h_ref = list(seeds)
    h_gpu = torch.stack(seeds).cuda()
    report = []                                   # (step, request, KL, relative error of the hidden, argmax agrees)
    for step in range(3):
        want = [ar.step(tok[r], h_ref[r], states[r]) for r in range(2)]
        logits, h_next = head.forward_batch(torch.tensor(tok, device="cuda"), h_gpu, slot, n_past, 40)
        logits, h_next = logits.cpu(), h_next.cpu()
        assert torch.isfinite(logits).all() and logits.shape == (2, cfg.vocab)
        for r in range(2):
            lg_ref, hn_ref = want[r]
            top2 = lg_ref.topk(2).values
            decided = float(top2[0] - top2[1]) > 0.1
            rel = float((h_next[r] - hn_ref).abs().max() / hn_ref.abs().max())
            report.append((step, r, round(_kl(lg_ref, logits[r]), 5), round(rel, 4),
                           (not decided) or int(logits[r].argmax()) == int(lg_ref.argmax())))
        tok = [int(want[r][0].argmax()) for r in range(2)]
        h_ref = [want[r][1] for r in range(2)]
        h_gpu = head.h_next[:2]                                  # the head's own recurrent rows, fed straight back
    assert all(kl < 0.05 and rel < 0.15 and same for (_s, _r, kl, rel, same) in report), report
    for i, t in kv_before.items():
        assert torch.equal(ex.kv[i], t)


@pytest.mark.parametrize("mode", ["drafted", "all_accepted", "partly_accepted"])
def test_assistant_cycle_reproduces_greedy_decode(mode):
    from hipengine_b200.models import make_executor
    from hipengine_b200.models.executor import make_batch
    from hipengine_b200.models.gemma4_assistant import Gemma4AssistantHead
    from hipengine_b200.speculative.gemma4_mtp import AssistantMTPCycle
    cfg = TINY_GEMMA4
    w = build_random_model(cfg, seed=3, std=0.05).to("cuda")
    hw = build_random_assistant(TINY_GEMMA4_ASSISTANT, cfg, seed=4, std=0.05)
    prompt = _prompt(45, 7).tolist()
    n_new = 13
    ex0 = make_executor(w, max_slots=1, max_context=128)
    lg = ex0.prefill(0, prompt)
    want = [int(lg.argmax(-1))]
    for i in range(n_new - 1):
        want.append(int(ex0.forward_logits(0, [want[-1]], len(prompt) + i).argmax(-1)))
    ex = make_executor(w, max_slots=2, max_context=128)
    cyc = AssistantMTPCycle(ex, Gemma4AssistantHead(ex, hw), max_depth=3, max_requests=2)
    assert cyc.capability().as_dict()["provider"] == "gemma4_mtp"
    slot = 1
    b = make_batch([(slot, 0, prompt)], "cuda")
    h = ex.forward(b)
    cyc.after_prefill(b, h)
    got = [int(ex.logits(h[b.T - 1:b.T]).argmax(-1))]
    assert got[0] == want[0]
    while len(got) < n_new:
        pos = len(prompt) + len(got) - 1                     # position of the last committed token
        override = None
        if mode != "drafted":
            nxt = want[len(got):len(got) + 3]
            nxt = nxt + [0] * (3 - len(nxt))
            if mode == "partly_accepted":
                nxt[1] = (nxt[1] + 1) % cfg.vocab            # second draft wrong: exactly one draft is accepted
            override = torch.tensor([nxt])
        res, txn = cyc.cycle([slot], [got[-1]], [pos], 3, draft_override=override)
        assert txn.trace[-1] == "committed" and 1 <= len(res[0].tokens) <= 4
        if mode == "all_accepted" and len(got) + 4 < n_new:
            assert res[0].accepted == 3
        if mode == "partly_accepted" and len(got) + 4 < n_new:
            assert res[0].accepted == 1
        got += res[0].tokens
    assert got[:n_new] == want, (got, want)


def test_gemma4_mtp_provider_through_the_public_api():
    """`speculative_provider="gemma4_mtp"` with the head passed as `draft_model`: same greedy tokens as the plain
    engine, cycles and drafts counted in the telemetry."""
    from hipengine_b200 import LLM, SamplingParams
    w = build_random_model(TINY_GEMMA4, seed=2, std=0.05).to("cuda")
    hw = build_random_assistant(TINY_GEMMA4_ASSISTANT, TINY_GEMMA4, seed=6, std=0.05)
    plain = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off")
    spec = LLM(w, backend="cuda_sm100a", max_active_requests=2, max_sequence_length=256, prefix_cache="off",
               speculative_mtp_serving="on", speculative_provider="gemma4_mtp", draft_model=hw,
               speculative_candidate_budget=3)
    try:
        prompts = [_prompt(n, 11 + n).tolist() for n in (12, 40)]
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        a = plain.generate_detailed(prompts, sp)
        b = spec.generate_detailed(prompts, sp)
        for x, y in zip(a, b):
            assert x.token_ids == y.token_ids and len(y.token_ids) == 10
        assert all(o.telemetry.speculative_cycles >= 1 and o.telemetry.speculative_drafted >= 3 for o in b)
        cap = spec._get_engine().loop.runner.capacity()["speculative"]
        assert cap["provider"] == "gemma4_mtp" and cap["attachment"] == "assistant_head"
    finally:
        plain.close()
        spec.close()
