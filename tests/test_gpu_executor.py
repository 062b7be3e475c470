"""End-to-end: GPU executor logits vs the fp32 reference model at identical (teacher-forced) contexts."""
import pytest
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_DENSE, TINY_HYBRID
from hipengine_b200.ref.model import RefModel

pytestmark = pytest.mark.gpu


def _kl(p_logits, q_logits):
    p = torch.log_softmax(p_logits.double(), -1)
    q = torch.log_softmax(q_logits.double(), -1)
    return (p.exp() * (p - q)).sum(-1)


def _compare(cfg, n_prompt, n_decode, seed=0, std=0.05):
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    w = build_random_model(cfg, seed=seed, std=std)
    ref = RefModel(w)
    ex = HybridExecutor(w.to("cuda"), max_slots=2, max_context=256)
    g = torch.Generator().manual_seed(seed + 1)
    toks = torch.randint(0, cfg.vocab, (n_prompt + n_decode,), generator=g)
    ref_logits, _ = ref.forward(toks)
    # prefill rows [0, n_prompt) in one packed batch (GEMM path when > 8 rows), then decode one row at a time
    got = [ex.forward_logits(1, toks[:n_prompt].tolist(), 0).cpu()]
    for t in range(n_prompt, n_prompt + n_decode):
        got.append(ex.forward_logits(1, [int(toks[t])], t).cpu())
    got = torch.cat(got, 0)
    kl = _kl(ref_logits, got)
    # top-1 agreement counted where the reference's own margin is not a near-tie
    top2 = ref_logits.topk(2, -1).values
    decided = (top2[:, 0] - top2[:, 1]) > 0.02
    agree = ref_logits.argmax(-1) == got.argmax(-1)
    top1 = (agree | ~decided).float().mean().item()
    return kl, top1, ref_logits, got


@pytest.mark.parametrize("cfg", [TINY_DENSE, TINY_HYBRID], ids=["dense", "hybrid"])
def test_decode_path_matches_reference(cfg):
    kl, top1, ref_logits, got = _compare(cfg, 4, 6)
    assert torch.isfinite(got).all()
    rel = ((got - ref_logits).abs().max() / ref_logits.std()).item()
    assert kl.max() < 0.05 and top1 >= 0.8 and rel < 0.4, (kl.max().item(), top1, rel)


def test_prefill_with_six_value_heads_uses_padded_gate_projection():
    """Six value heads (the per-rank count of the 27B at eight-way tensor parallelism) make the alpha/beta projection
    12 rows wide: it is padded to 16 rows and stays on the tensor-core GEMM."""
    from dataclasses import replace
    cfg = replace(TINY_HYBRID, ssm_v_heads=6, ssm_groups=2)
    kl, top1, ref_logits, got = _compare(cfg, 40, 3)
    assert torch.isfinite(got).all()
    assert kl.max() < 0.05 and top1 >= 0.8, (kl.max().item(), top1)


@pytest.mark.parametrize("cfg", [TINY_DENSE, TINY_HYBRID], ids=["dense", "hybrid"])
def test_prefill_path_matches_reference(cfg):
    kl, top1, ref_logits, got = _compare(cfg, 40, 3)
    assert torch.isfinite(got).all()
    rel = ((got - ref_logits).abs().max() / ref_logits.std()).item()
    assert kl.max() < 0.05 and top1 >= 0.8 and rel < 0.4, (kl.max().item(), top1, rel)


def test_two_slots_are_isolated():
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    cfg = TINY_HYBRID
    w = build_random_model(cfg, seed=3, std=0.05)
    ex = HybridExecutor(w.to("cuda"), max_slots=2, max_context=128)
    ex.small_rows = 8            # both runs on the same numeric path: the property under test is slot isolation
    a = [5, 6, 7, 8, 9]
    b = [100, 200, 300]
    la = ex.forward_logits(0, a, 0).clone()
    ex.reset_slot(0)
    # same request on slot 0 while slot 1 runs a different one in the same packed batch
    batch = make_batch([(0, 0, a), (1, 0, b)], "cuda")
    h = ex.forward(batch)
    lab = ex.logits(h[:5]).clone()
    assert torch.allclose(la, lab, atol=2e-2, rtol=2e-2)


def test_decode_graph_replays_through_native_launcher():
    """Graph decode must equal eager decode, and the replay goes through the native control-block launcher."""
    from hipengine_b200.models.decode_graph import DecodeGraphRunner
    from hipengine_b200.models.executor import HybridExecutor
    cfg = TINY_HYBRID
    w = build_random_model(cfg, seed=5, std=0.05).to("cuda")
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(2)).tolist()

    def run(use_graphs):
        ex = HybridExecutor(w, max_slots=1, max_context=128)
        r = DecodeGraphRunner(ex, max_rows=1, use_graphs=use_graphs)
        first = int(ex.prefill(0, prompt).argmax(-1))
        r.set_rows([0], [first], [len(prompt)])
        out = [first]
        for _ in range(6):
            r.step(1, 128)
            out.append(int(r.tokens[0]))
        return out, r

    eager, _ = run(False)
    graph, r = run(True)
    assert eager == graph
    assert r.stats["captures"] == 1 and r.stats["hits"] == 5
    if r.native_launch and any(r._execs.values()):
        assert r.stats["native_launches"] == 6


def test_old_graph_survives_scratch_growth_and_later_captures():
    """A graph captured while scratch buffers were small must stay valid after a long prefill has grown them and
    after further captures (which empty the allocator cache): retired scratch buffers are kept mapped."""
    from hipengine_b200.models.decode_graph import DecodeGraphRunner
    from hipengine_b200.models.executor import HybridExecutor
    cfg = TINY_HYBRID
    w = build_random_model(cfg, seed=6, std=0.05).to("cuda")
    g = torch.Generator().manual_seed(4)
    short = torch.randint(0, cfg.vocab, (10,), generator=g).tolist()
    long = torch.randint(0, cfg.vocab, (400,), generator=g).tolist()

    def run(use_graphs):
        ex = HybridExecutor(w, max_slots=3, max_context=512)
        r = DecodeGraphRunner(ex, max_rows=2, use_graphs=use_graphs)
        out = []
        t0 = int(ex.prefill(0, short).argmax(-1))
        r.set_rows([0], [t0], [len(short)])
        for _ in range(3):
            r.step(1, 512)                                  # graph for 1 row, captured with small scratch
            out.append(int(r.tokens[0]))
        t1 = int(ex.prefill(1, long).argmax(-1))            # grows every scratch buffer
        r.set_rows([0, 1], [out[-1], t1], [len(short) + 3, len(long)])
        for _ in range(2):
            r.step(2, 512)                                  # second capture
            out += [int(r.tokens[0]), int(r.tokens[1])]
        last0 = int(r.tokens[0])
        r.set_rows([0], [last0], [len(short) + 5])
        for _ in range(3):
            r.step(1, 512)                                  # replays the first graph
            out.append(int(r.tokens[0]))
        torch.cuda.synchronize()
        return out, ex

    eager, _ = run(False)
    graph, ex = run(True)
    assert graph == eager
    assert ex.scratch.retired_bytes() > 0


def test_27b_width_layers_match_fp32_reference():
    """Four layers (three Gated-DeltaNet + one gated full-attention) at the 27B model's real widths -- hidden 5120,
    head_dim 256, 24/4 heads, 48 value heads of 128, FFN 17408, the Q4_K_M-style mix of block types -- against the
    fp32 reference on the same weights: a 300-row prefill (tensor-core GEMMs in pair mode, chunked scan, flash
    prefill), packed 5-row decode (int8 GEMV) and a 24-row packed step (split-K tensor-core path)."""
    from dataclasses import replace
    from hipengine_b200.models.config import NAMED_CONFIGS
    from hipengine_b200.models.executor import HybridExecutor, make_batch
    cfg = replace(NAMED_CONFIGS["qwen35-27b"], n_layers=4, vocab=8192)
    w = build_random_model(cfg, seed=11, device="cuda", recipe="q4_k_m")
    ref = RefModel(w, device="cuda")
    ex = HybridExecutor(w, device="cuda", max_slots=2, max_context=512)
    n_prompt, n_dec = 300, 5
    toks = torch.randint(0, cfg.vocab, (n_prompt + n_dec + 24,), generator=torch.Generator().manual_seed(12))
    ref_logits, _ = ref.forward(toks.to("cuda"))
    ref_logits = ref_logits.float().cpu()
    got = [ex.forward_logits(1, toks[:n_prompt].tolist(), 0).cpu()]
    for t in range(n_prompt, n_prompt + n_dec):
        got.append(ex.forward_logits(1, [int(toks[t])], t).cpu())
    t0 = n_prompt + n_dec
    got.append(ex.forward_logits(1, toks[t0:t0 + 24].tolist(), t0).cpu())
    got = torch.cat(got, 0)
    assert torch.isfinite(got).all()
    kl = _kl(ref_logits, got)
    top2 = ref_logits.topk(2, -1).values
    decided = (top2[:, 0] - top2[:, 1]) > 0.05 * ref_logits.std()
    agree = ref_logits.argmax(-1) == got.argmax(-1)
    top1 = (agree | ~decided).float().mean().item()
    rel = ((got - ref_logits).norm() / ref_logits.norm()).item()
    assert kl.max() < 0.05 and top1 >= 0.9 and rel < 0.08, (kl.max().item(), top1, rel)


def test_graph_replayed_prefill_equals_eager_prefill():
    """A single-chunk prefill replayed from a CUDA graph (keyed by slot, start position and row count) produces the
    logits and the state of the eager prefill, for token ids that change from call to call."""
    from hipengine_b200.models.executor import HybridExecutor
    cfg = TINY_HYBRID
    w = build_random_model(cfg, seed=7, std=0.05).to("cuda")
    ex = HybridExecutor(w, max_slots=2, max_context=512)
    ex_ref = HybridExecutor(w, max_slots=2, max_context=512)
    g = torch.Generator().manual_seed(8)
    for call in range(4):                       # call 0 eager, call 1 captures, calls 2.. replay
        toks = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
        ex.reset_slot(1)
        ex_ref.reset_slot(1)
        got = ex.prefill(1, toks, graph=True).clone()
        want = ex_ref.prefill(1, toks, graph=False)
        assert torch.equal(got, want), call
        nxt = int(want.argmax(-1))
        assert torch.equal(ex.forward_logits(1, [nxt], 300), ex_ref.forward_logits(1, [nxt], 300))
    assert "graph" in ex._prefill_graphs[(1, 0, 300)]
