"""Gemma 4 (26B-A4B family) tensor map, GGUF metadata overrides and random-init builder.

Per layer (GGUF names): ``attn_norm, attn_q, attn_k, [attn_v], attn_output, attn_q_norm, attn_k_norm,
post_attention_norm, ffn_norm, ffn_gate, ffn_up, ffn_down, post_ffw_norm_1, ffn_gate_inp(.weight/.scale),
pre_ffw_norm_2, ffn_gate_up_exps (gate rows then up rows per expert), ffn_down_exps(.weight/.scale),
post_ffw_norm_2, post_ffw_norm, layer_output_scale``.  Global layers have no ``attn_v`` (V = K), 2 KV heads and
head dim 512; sliding layers 8 KV heads, head dim 256, window 1024.  Source of the contract: the reference's
model card ``docs/model-cards/MODEL-GEMMA4.md:128-205`` and its loader ``hipengine/loading/gemma4_gguf.py:99-174``.
Expert ``down`` rows have K = 704, which is not a multiple of the 256-element K-quant super-block, so real files
store them as Q5_1 / Q8_0; the random-init recipe uses Q8_0 there (``hipengine/loading/gemma4_gguf_device.py:277``).
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..models.config import ModelConfig
from ..quant.ggml import GGMLType
from .weights import ModelWeights


def gemma4_config_overrides(info) -> Dict[str, Any]:
    md = info.metadata
    g = lambda k, d=None: md.get(f"gemma4.{k}", d)
    kvs = g("attention.head_count_kv")
    hidden = int(g("embedding_length"))
    out: Dict[str, Any] = dict(
        qk_norm=True, attn_scale=1.0, gated_attention=False, act="gelu_tanh", tie_embeddings=True,
        final_softcap=float(g("final_logit_softcapping", 30.0)), embed_scale=float(hidden) ** 0.5,
        sliding_window=int(g("attention.sliding_window", 1024)), full_attention_interval=0,
        rope_theta=float(g("rope.freq_base", 1e6)), swa_rope_theta=float(g("rope.freq_base_swa", 1e4)),
    )
    if isinstance(kvs, (list, tuple)) and len(kvs) > 1:
        swa = max(kvs)
        glob = min(kvs)
        first_global = next((i for i, v in enumerate(kvs) if v == glob), len(kvs) - 1)
        out.update(n_kv_heads=int(swa), global_kv_heads=int(glob), swa_pattern=first_global + 1)
    out["head_dim"] = int(g("attention.key_length_swa", g("attention.key_length", 256)))
    out["global_head_dim"] = int(g("attention.key_length", out["head_dim"]))
    out["rope_dim"] = out["head_dim"]
    return out


def build_random_gemma4(cfg: ModelConfig, seed: int = 0, device="cpu", recipe: str = "q4_k_xl",
                        std: float = 0.02) -> ModelWeights:
    from .synth import _Builder, config_to_metadata
    if recipe == "q4_k_m":
        recipe = "q4_k_xl"
    b = _Builder(cfg, seed, device, recipe, std)
    base, hi = b.base_type(), b.hi_type()
    H, E, F, Fd = cfg.hidden, cfg.n_experts, cfg.expert_ffn, cfg.ffn
    b.matrix("token_embd.weight", (cfg.vocab, H), hi)
    b.f32("output_norm.weight", b.ones(H) + b.randn(H, std=0.02))
    near1 = lambda n: b.ones(n) + b.randn(n, std=0.05)
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        D, Hkv = cfg.layer_head_dim(i), cfg.layer_kv_heads(i)
        glob = cfg.is_global_layer(i)
        b.f32(p + "attn_norm.weight", near1(H))
        b.matrix(p + "attn_q.weight", (cfg.n_heads * D, H), base)
        b.matrix(p + "attn_k.weight", (Hkv * D, H), base)
        if not glob:
            b.matrix(p + "attn_v.weight", (Hkv * D, H), hi)
        b.matrix(p + "attn_output.weight", (H, cfg.n_heads * D), base)
        # attention scale is 1.0, so unit norm weights would give scores of order sqrt(D) and a one-hot softmax;
        # trained checkpoints learn small norm weights -- use D**-0.25 each so q.k is of order 1
        b.f32(p + "attn_q_norm.weight", near1(D) * (D ** -0.25))
        b.f32(p + "attn_k_norm.weight", near1(D) * (D ** -0.25))
        b.f32(p + "post_attention_norm.weight", near1(H))
        b.f32(p + "ffn_norm.weight", near1(H))
        b.matrix(p + "ffn_gate.weight", (Fd, H), base)
        b.matrix(p + "ffn_up.weight", (Fd, H), base)
        b.matrix(p + "ffn_down.weight", (H, Fd), hi)
        b.f32(p + "post_ffw_norm_1.weight", near1(H))
        # the router input is RMS-normed and divided by sqrt(hidden), so unit-scale rows give logits of order 1
        b.f32(p + "ffn_gate_inp.weight", b.randn(E, H, std=1.0))
        b.f32(p + "ffn_gate_inp.scale", near1(H))
        b.f32(p + "pre_ffw_norm_2.weight", near1(H))
        b.matrix(p + "ffn_gate_up_exps.weight", (E, 2 * F, H), base)
        b.matrix(p + "ffn_down_exps.weight", (E, H, F), GGMLType.Q8_0)
        b.f32(p + "ffn_down_exps.scale", near1(E))
        b.f32(p + "post_ffw_norm_2.weight", near1(H))
        b.f32(p + "post_ffw_norm.weight", near1(H))
        b.f32(p + "layer_output_scale.weight", b.ones(1) * (1.0 - 0.01 * (i % 3)))
    md = config_to_metadata(cfg) if True else {}
    return ModelWeights(cfg, b.out, md)
