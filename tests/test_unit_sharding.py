"""Tensor-parallel sharding math on CPU: per-rank partial outputs of every row-parallel block must add up to
the unsharded block, using the fp32 reference model on each shard."""
import torch

from hipengine_b200.loading.synth import build_random_model
from hipengine_b200.models.config import QWEN35_27B, QWEN35_35B_A3B, TINY_HYBRID_TP
from hipengine_b200.parallel.sharding import TPPlan, shard_weights
from hipengine_b200.ref import ops as R
from hipengine_b200.ref.model import RefModel, RefState


def test_plans_cover_everything_exactly_once():
    for cfg in (QWEN35_27B, TINY_HYBRID_TP):
        for tp in (1, 2, 4, 8):
            if cfg is TINY_HYBRID_TP and tp > 2:
                continue
            plans = [TPPlan.make(cfg, tp, r) for r in range(tp)]
            assert sorted(h for p in plans for h in p.v_heads) == list(range(cfg.ssm_v_heads))
            assert sum(p.ffn_cols[1] - p.ffn_cols[0] for p in plans) == cfg.ffn
            assert sum(p.vocab_rows[1] - p.vocab_rows[0] for p in plans) == cfg.vocab
            assert sum(p.q_heads[1] - p.q_heads[0] for p in plans) == cfg.n_heads
            for p in plans:
                # every local V head must read the right local K head: local_h % local_G
                G = cfg.ssm_groups
                for l, h in enumerate(p.v_heads):
                    assert p.k_groups[0] + l % p.local.ssm_groups == h % G
                gqa = cfg.n_heads // cfg.n_kv_heads
                for q in range(*p.q_heads):
                    assert p.kv_heads[0] <= q // gqa < p.kv_heads[1]
                assert p.ffn_cols[0] % 256 == 0 and p.ffn_cols[1] % 256 == 0
    p = TPPlan.make(QWEN35_27B, 8, 5)
    assert p.local.n_kv_heads == 1 and p.kv_heads == (2, 3) and p.local.n_heads == 3
    experts = [TPPlan.make(QWEN35_35B_A3B, 8, r).experts for r in range(8)]
    assert experts[0] == (0, 32) and experts[-1] == (224, 256)


def test_partial_blocks_sum_to_full_block():
    cfg = TINY_HYBRID_TP
    tp = 2
    w = build_random_model(cfg, seed=0, std=0.05)
    full = RefModel(w)
    shards = [RefModel(shard_weights(w, tp, r)[0]) for r in range(tp)]
    T = 6
    x = torch.randn(T, cfg.hidden, generator=torch.Generator().manual_seed(0))
    pos = torch.arange(T)
    for i in range(cfg.n_layers):
        if cfg.is_full_attention_layer(i):
            want = full.full_attention(i, x, RefState(), pos)
            got = sum(s.full_attention(i, x, RefState(), pos) for s in shards)
        else:
            want = full.linear_attention(i, x, RefState())
            got = sum(s.linear_attention(i, x, RefState()) for s in shards)
        torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(sum(s.ffn(i, x) for s in shards), full.ffn(i, x), atol=2e-4, rtol=2e-4)
    # vocab-parallel head: concatenated shard logits are the full logits
    hn = R.rmsnorm(x, full.w["output_norm.weight"], cfg.rms_eps)
    want = full.logits_from_hidden(hn)
    got = torch.cat([s.logits_from_hidden(hn) for s in shards], -1)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_shards_keep_exact_gguf_blocks():
    cfg = TINY_HYBRID_TP
    w = build_random_model(cfg, seed=1, std=0.05)
    s0, p0 = shard_weights(w, 2, 0)
    s1, p1 = shard_weights(w, 2, 1)
    t = w["blk.0.ffn_down.weight"]
    a, b = s0["blk.0.ffn_down.weight"], s1["blk.0.ffn_down.weight"]
    assert torch.equal(torch.cat([a.raw, b.raw], 1), t.raw.reshape(t.n_rows, -1))
    assert torch.equal(torch.cat([a.dequant(), b.dequant()], 1), t.dequant())
