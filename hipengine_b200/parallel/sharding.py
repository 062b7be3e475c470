"""Tensor-parallel sharding of a hybrid Qwen3.5 checkpoint kept in its GGUF quantisation.

Shards fall on quantisation-block boundaries: a row-parallel (K-split) shard is a whole number of 256-element
super-blocks, so every rank keeps bit-exact GGUF blocks and the split changes no numerics besides the order of
the final sum.

* full attention: Q heads are split evenly; KV heads are split when ``n_kv_heads % tp == 0`` and otherwise
  replicated (rank ``r`` uses KV head ``r // (tp / n_kv_heads)``).  ``attn_q`` rows are per-head ``[Q | gate]``.
* gated delta-net: split by K-head group.  V head ``h`` reads K head ``h % G``, so rank ``r`` owning K heads
  ``[g0, g1)`` takes the V heads ``{h : g0 <= h % G < g1}`` in ascending order, which keeps ``local_h % local_G``
  pointing at the right local K head.  ``G / tp`` must be even so that pairs of 128-wide V heads form whole
  256-element blocks of ``ssm_out``'s K axis.
* dense FFN: the 256-column blocks of the FFN width are dealt out as evenly as possible (17408 = 68 blocks:
  TP8 gives 9/9/9/9/8/8/8/8).
* MoE: experts are dealt out in contiguous ranges (expert parallelism over the replicated activations); the
  shared expert runs on the rank that owns the fewest routed experts (the last one).
* lm_head / embeddings: the head is vocab-parallel by rows; the embedding table is replicated.

The per-rank result is an ordinary ``ModelWeights`` with a *local* ``ModelConfig`` (fewer heads, narrower FFN),
so the single-GPU executor runs it unchanged apart from the reductions after row-parallel projections.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, List, Tuple

import torch

from ..loading.weights import ModelWeights, QTensor
from ..models.config import ModelConfig
from ..quant.ggml import layout_of


def _even_split(n: int, parts: int, r: int) -> Tuple[int, int]:
    base, rem = divmod(n, parts)
    lo = r * base + min(r, rem)
    return lo, lo + base + (1 if r < rem else 0)


@dataclass
class TPPlan:
    tp: int
    rank: int
    q_heads: Tuple[int, int]          # [lo, hi) global Q heads
    kv_heads: Tuple[int, int]
    k_groups: Tuple[int, int]         # GDN K heads
    v_heads: List[int]                # GDN V heads (global ids, ascending)
    ffn_cols: Tuple[int, int]
    vocab_rows: Tuple[int, int]
    experts: Tuple[int, int]
    owns_shared_expert: bool
    local: ModelConfig

    @staticmethod
    def make(cfg: ModelConfig, tp: int, rank: int) -> "TPPlan":
        assert 0 <= rank < tp
        H, Hkv = cfg.n_heads, cfg.n_kv_heads
        assert H % tp == 0, f"n_heads {H} not divisible by tp {tp}"
        hq = H // tp
        q = (rank * hq, (rank + 1) * hq)
        if Hkv % tp == 0:
            kv = (rank * (Hkv // tp), (rank + 1) * (Hkv // tp))
        else:
            assert tp % Hkv == 0, f"tp {tp} must divide or be a multiple of n_kv_heads {Hkv}"
            g = rank // (tp // Hkv)
            kv = (g, g + 1)
        k_groups, v_heads = (0, 0), []
        if cfg.is_hybrid:
            G, Hv = cfg.ssm_groups, cfg.ssm_v_heads
            assert G % tp == 0 and Hv % G == 0, "GDN K-head groups must split evenly"
            gl = G // tp
            assert tp == 1 or (gl * cfg.ssm_state) % 256 == 0, "GDN shard must cover whole 256-column blocks"
            k_groups = (rank * gl, (rank + 1) * gl)
            v_heads = [h for h in range(Hv) if k_groups[0] <= h % G < k_groups[1]]
        ffn_cols = (0, 0)
        if cfg.ffn > 0:
            assert cfg.ffn % 256 == 0
            b0, b1 = _even_split(cfg.ffn // 256, tp, rank)
            ffn_cols = (b0 * 256, b1 * 256)
        experts = _even_split(cfg.n_experts, tp, rank) if cfg.is_moe else (0, 0)
        vocab = _even_split(cfg.vocab, tp, rank)
        local = replace(cfg, n_heads=hq, n_kv_heads=kv[1] - kv[0],
                        ssm_groups=(k_groups[1] - k_groups[0]) if cfg.is_hybrid else cfg.ssm_groups,
                        ssm_v_heads=len(v_heads) if cfg.is_hybrid else cfg.ssm_v_heads,
                        ffn=ffn_cols[1] - ffn_cols[0])
        return TPPlan(tp, rank, q, kv, k_groups, v_heads, ffn_cols, vocab, experts, rank == tp - 1, local)


def _take_rows(t: QTensor, idx: torch.Tensor) -> QTensor:
    if len(t.shape) == 1:   # plain vector (F32 per-head parameters): pick elements
        esz = t.raw.numel() // t.shape[0]
        raw = t.raw.reshape(t.shape[0], esz)[idx.to(t.raw.device)].reshape(1, -1).contiguous()
        return QTensor(t.name, t.ggml_type, (int(idx.numel()),), raw)
    raw = t.raw.reshape(t.n_rows, -1)[idx.to(t.raw.device)].contiguous()
    return QTensor(t.name, t.ggml_type, (int(idx.numel()),) + tuple(t.shape[1:]), raw)


def _take_col_ranges(t: QTensor, ranges: List[Tuple[int, int]]) -> QTensor:
    lay = layout_of(t.ggml_type)
    parts, width = [], 0
    raw2 = t.raw.reshape(t.n_rows, -1)
    for c0, c1 in ranges:
        assert c0 % lay.block_elems == 0 and c1 % lay.block_elems == 0, "shard must fall on quant-block boundaries"
        parts.append(raw2[:, c0 // lay.block_elems * lay.block_bytes:c1 // lay.block_elems * lay.block_bytes])
        width += c1 - c0
    return QTensor(t.name, t.ggml_type, tuple(t.shape[:-1]) + (width,), torch.cat(parts, 1).contiguous())


def _ranges(ids: List[int], width: int) -> List[Tuple[int, int]]:
    """Merge consecutive unit ids into [lo*width, hi*width) column ranges."""
    out: List[Tuple[int, int]] = []
    for i in ids:
        if out and out[-1][1] == i * width:
            out[-1] = (out[-1][0], (i + 1) * width)
        else:
            out.append((i * width, (i + 1) * width))
    return out


def shard_weights(w: ModelWeights, tp: int, rank: int) -> Tuple[ModelWeights, TPPlan]:
    """Slice a full checkpoint into rank ``rank``'s tensor-parallel shard."""
    cfg = w.config
    plan = TPPlan.make(cfg, tp, rank)
    if tp == 1:
        return w, plan
    D, S = cfg.head_dim, cfg.ssm_state
    out: Dict[str, QTensor] = {}
    ar = lambda lo, hi: torch.arange(lo, hi)
    qmul = 2 if cfg.gated_attention else 1
    G = cfg.ssm_groups
    for name, t in w.tensors.items():
        slot = name.split(".", 2)[2] if name.startswith("blk.") else name
        if slot == "attn_q.weight":
            out[name] = _take_rows(t, ar(plan.q_heads[0] * D * qmul, plan.q_heads[1] * D * qmul))
        elif slot in ("attn_k.weight", "attn_v.weight"):
            out[name] = _take_rows(t, ar(plan.kv_heads[0] * D, plan.kv_heads[1] * D))
        elif slot == "attn_output.weight":
            out[name] = _take_col_ranges(t, [(plan.q_heads[0] * D, plan.q_heads[1] * D)])
        elif slot in ("attn_qkv.weight", "ssm_conv1d.weight"):
            kq = ar(plan.k_groups[0] * S, plan.k_groups[1] * S)
            v = torch.cat([ar(h * S, (h + 1) * S) for h in plan.v_heads]) + 2 * G * S
            out[name] = _take_rows(t, torch.cat([kq, kq + G * S, v]))
        elif slot == "attn_gate.weight":
            out[name] = _take_rows(t, torch.cat([ar(h * S, (h + 1) * S) for h in plan.v_heads]))
        elif slot in ("ssm_alpha.weight", "ssm_beta.weight", "ssm_a", "ssm_dt.bias"):
            out[name] = _take_rows(t, torch.tensor(plan.v_heads))
        elif slot == "ssm_out.weight":
            out[name] = _take_col_ranges(t, _ranges(plan.v_heads, S))
        elif slot in ("ffn_gate.weight", "ffn_up.weight"):
            out[name] = _take_rows(t, ar(*plan.ffn_cols))
        elif slot == "ffn_down.weight":
            out[name] = _take_col_ranges(t, [plan.ffn_cols])
        elif slot in ("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"):
            n = t.shape[1]
            sub = _take_rows(QTensor(t.name, t.ggml_type, (t.shape[0] * n, t.shape[2]), t.raw),
                             ar(plan.experts[0] * n, plan.experts[1] * n))
            out[name] = QTensor(t.name, t.ggml_type, (plan.experts[1] - plan.experts[0], n, t.shape[2]), sub.raw)
        elif name == "output.weight" or (name == "token_embd.weight" and "output.weight" not in w.tensors):
            if name == "token_embd.weight":
                out[name] = t                      # tied: full table for the lookup ...
                out["output.weight"] = _take_rows(t, ar(*plan.vocab_rows))   # ... and a row shard as the head
            else:
                out[name] = _take_rows(t, ar(*plan.vocab_rows))
        else:
            out[name] = t                          # norms, router, shared expert, embeddings: replicated
    meta = dict(w.metadata)
    meta["tp"] = {"size": tp, "rank": rank}
    return ModelWeights(plan.local, out, meta), plan
