"""Reference forward: incremental decode equals one-shot prefill; chunked GDN equals the serial rule."""
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_DENSE, TINY_HYBRID, TINY_HYBRID_MOE
from hipengine_b200.ref import ops as R
from hipengine_b200.ref.model import RefModel


def _check_incremental(cfg, n=12, tol=2e-4):
    w = build_random_model(cfg, seed=0)
    m = RefModel(w)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (n,), generator=g)
    full, _ = m.forward(toks)
    st = m.new_state()
    a, st = m.forward(toks[:5], st)
    rows = [a]
    for t in range(5, n):
        lg, st = m.forward(toks[t:t + 1], st)
        rows.append(lg)
    inc = torch.cat(rows, 0)
    assert torch.allclose(full, inc, atol=tol, rtol=1e-3), (full - inc).abs().max()
    assert torch.isfinite(full).all()


def test_dense_incremental():
    _check_incremental(TINY_DENSE)


def test_hybrid_incremental():
    _check_incremental(TINY_HYBRID)


def test_hybrid_moe_incremental():
    _check_incremental(TINY_HYBRID_MOE, n=8)


def test_gdn_chunked_matches_serial():
    g = torch.Generator().manual_seed(0)
    T, H, D = 150, 3, 32
    q = R.l2norm(torch.randn(T, H, D, generator=g)) * D ** -0.5
    k = R.l2norm(torch.randn(T, H, D, generator=g))
    v = torch.randn(T, H, D, generator=g)
    decay = torch.exp(-torch.rand(T, H, generator=g))
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    s0 = torch.randn(H, D, D, generator=g) * 0.1
    o1, s1 = R.gdn_recurrent(q, k, v, decay, beta, s0)
    o2, s2 = R.gdn_chunked(q, k, v, decay, beta, s0, chunk=64)
    assert torch.allclose(o1, o2, atol=1e-4), (o1 - o2).abs().max()
    assert torch.allclose(s1, s2, atol=1e-4)


def test_moe_route_ties_prefer_lower_id():
    lg = torch.zeros(1, 8)
    idx, w = R.moe_route(lg, 3)
    assert idx.tolist() == [[0, 1, 2]]
    assert torch.allclose(w.sum(-1), torch.ones(1))


def test_tiny_dense_greedy_generation_config1():
    """Tiny dense benchmark config: 32-token prompt, 16 greedy tokens, logits finite and reproducible."""
    w = build_random_model(TINY_DENSE, seed=0)
    m = RefModel(w)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 4096, (32,), generator=g).tolist()
    out1, lg1 = m.generate(prompt, 16)
    out2, lg2 = m.generate(prompt, 16)
    assert out1 == out2 and len(out1) == 16 and lg1.shape == (16, 4096)
    assert torch.equal(lg1, lg2)


def test_gemma4_reference_incremental_equals_batch():
    """Gemma 4 oracle: feeding a prompt in two pieces (KV carried over, sliding window exceeded) gives the same
    logits as one pass, and the logits respect the soft-cap."""
    import torch
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_GEMMA4
    from hipengine_b200.ref.model import RefModel
    w = build_random_model(TINY_GEMMA4, seed=0, std=0.05)
    m = RefModel(w)
    toks = torch.randint(0, TINY_GEMMA4.vocab, (48,), generator=torch.Generator().manual_seed(0))
    full, _ = m.forward(toks)
    a, st = m.forward(toks[:37])
    b, _ = m.forward(toks[37:], st)
    torch.testing.assert_close(torch.cat([a, b]), full, atol=2e-4, rtol=2e-4)
    assert float(full.abs().max()) <= TINY_GEMMA4.final_softcap
    # global layers have no attn_v tensor (V = K) and a wider head
    assert "blk.5.attn_v.weight" not in w.tensors and "blk.0.attn_v.weight" in w.tensors
    assert w["blk.5.attn_k.weight"].shape[0] == TINY_GEMMA4.global_kv_heads * TINY_GEMMA4.global_head_dim
