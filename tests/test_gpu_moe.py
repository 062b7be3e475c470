"""Mixture-of-experts kernels and the MoE executor paths against the fp32 reference."""
import pytest
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import TINY_HYBRID_MOE
from hipengine_b200.ref import ops as R
from hipengine_b200.ref.model import RefModel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,k,T", [(16, 4, 5), (128, 8, 33), (256, 8, 70), (512, 10, 3)])
def test_route_matches_reference(E, k, T):
    from hipengine_b200.ops import kernels as K
    g = torch.Generator(device="cuda").manual_seed(E + T)
    logits = torch.randn(T, E + 8, device="cuda", generator=g) * 3
    logits[0, 3] = logits[0, 1]          # an exact tie: the lower id must win
    ids = torch.empty(T, k, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, k, device="cuda")
    K.moe_route(logits, k, ids, wts, n_experts=E)
    ridx, rw = R.moe_route(logits[:, :E].cpu(), k)
    assert torch.equal(ids.cpu().long(), ridx)
    torch.testing.assert_close(wts.cpu(), rw, atol=1e-5, rtol=1e-4)


def test_group_and_gather_round_trip():
    from hipengine_b200.ops import kernels as K
    T, k, E, Hd = 300, 4, 16, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.randint(0, E, (T, k), device="cuda", generator=g).to(torch.int32)
    ids[:, 0] = 7                          # one crowded expert spanning several tiles
    bound = K.moe_sorted_rows_bound(T * k, E)
    pos = torch.empty(T * k, dtype=torch.int32, device="cuda")
    tiles = torch.empty(bound // 128, dtype=torch.int32, device="cuda")
    meta = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.moe_group(ids, E, pos, tiles, meta)
    pos_c, tiles_c, flat = pos.cpu().long(), tiles.cpu(), ids.cpu().flatten().long()
    assert pos_c.unique().numel() == T * k and int(pos_c.max()) < int(meta[0]) <= bound
    assert torch.equal(tiles_c[pos_c // 128].long(), flat)       # every pair sits in a tile of its own expert
    x = torch.randn(T, Hd, device="cuda", generator=g).to(torch.bfloat16)
    xs = torch.zeros(bound, Hd, device="cuda", dtype=torch.bfloat16)
    K.moe_gather(x, pos, k, xs)
    assert torch.equal(xs[pos.long()].cpu(), x.repeat_interleave(k, 0).cpu())


def test_grouped_gemm_matches_per_expert_matmul():
    from hipengine_b200.ops import gemm as GM
    from hipengine_b200.ops import kernels as K
    E, Nn, Kd = 6, 320, 256
    g = torch.Generator(device="cuda").manual_seed(1)
    w = (torch.randn(E * Nn, Kd, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    groups = torch.tensor([2, -1, 5, 0, 0, -1, 3], dtype=torch.int32, device="cuda")
    M = groups.numel() * 128
    a = torch.randn(M, Kd, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.zeros(M, Nn, device="cuda", dtype=torch.bfloat16)
    GM.gemm_bf16_grouped(a, w, out, E, groups)
    GM.check_status(a.device)
    for tm, e in enumerate(groups.tolist()):
        rows = slice(tm * 128, (tm + 1) * 128)
        if e < 0:
            assert float(out[rows].float().abs().max()) == 0.0
            continue
        ref = a[rows].float() @ w[e * Nn:(e + 1) * Nn].float().t()
        torch.testing.assert_close(out[rows].float(), ref, atol=3e-2, rtol=3e-2)


def _kl(p_logits, q_logits):
    p = torch.log_softmax(p_logits.double(), -1)
    q = torch.log_softmax(q_logits.double(), -1)
    return (p.exp() * (p - q)).sum(-1)


@pytest.mark.parametrize("n_prompt,n_decode", [(4, 5), (40, 2), (150, 2)], ids=["decode", "selected", "grouped"])
def test_moe_executor_matches_reference(n_prompt, n_decode):
    from hipengine_b200.models.executor import HybridExecutor
    cfg = TINY_HYBRID_MOE
    w = build_random_model(cfg, seed=0, std=0.05)
    ref = RefModel(w)
    ex = HybridExecutor(w.to("cuda"), max_slots=2, max_context=256)
    toks = torch.randint(0, cfg.vocab, (n_prompt + n_decode,), generator=torch.Generator().manual_seed(1))
    ref_logits, _ = ref.forward(toks)
    got = [ex.forward_logits(1, toks[:n_prompt].tolist(), 0).cpu()]
    for t in range(n_prompt, n_prompt + n_decode):
        got.append(ex.forward_logits(1, [int(toks[t])], t).cpu())
    got = torch.cat(got, 0)
    assert torch.isfinite(got).all()
    kl = _kl(ref_logits, got)
    rel = ((got - ref_logits).abs().max() / ref_logits.std()).item()
    top2 = ref_logits.topk(2, -1).values
    decided = (top2[:, 0] - top2[:, 1]) > 0.02
    top1 = ((ref_logits.argmax(-1) == got.argmax(-1)) | ~decided).float().mean().item()
    # a near-tie in the router can pick a different expert than the fp32 reference, so the max-abs bound is
    # looser than for dense models; KL and top-1 agreement carry the check
    assert kl.mean() < 0.01 and kl.max() < 0.15 and top1 >= 0.8 and rel < 1.5, (kl.mean().item(), kl.max().item(), top1, rel)


@pytest.mark.parametrize("T", [3, 40, 200], ids=["decode", "selected", "grouped"])
def test_moe_block_matches_reference_on_identical_input(T):
    """The FFN block alone, fed the same residual rows as the reference: only an exact router near-tie can
    differ, so nearly every row must agree closely."""
    from hipengine_b200.loading.weights import ffn_norm_slot
    from hipengine_b200.models import moe as M
    from hipengine_b200.models.executor import HybridExecutor
    cfg = TINY_HYBRID_MOE
    w = build_random_model(cfg, seed=2, std=0.05)
    ref = RefModel(w)
    ex = HybridExecutor(w.to("cuda"), max_slots=1, max_context=64)
    h0 = torch.randn(T, cfg.hidden, generator=torch.Generator().manual_seed(T))
    i = 1
    norm_w = ex.F(i, ffn_norm_slot(cfg))
    want = ref.ffn(i, R.rmsnorm(h0, ref.W(i, ffn_norm_slot(cfg)), cfg.rms_eps))
    h = h0.cuda().clone()
    M.moe_ffn(ex, i, h, T, norm_w, T <= 8)
    got = (h.cpu() - h0)
    assert torch.isfinite(got).all()
    err = (got - want).abs().amax(-1) / want.abs().amax(-1).clamp(min=1e-6)
    assert (err < 0.06).float().mean() >= 0.97, err
