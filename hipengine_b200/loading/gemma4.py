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


# ----------------------------------------------------------------------------- assistant (MTP) head artifact
ASSISTANT_ARCH = "gemma4-assistant"
ASSISTANT_BLOCK_SLOTS = ("attn_norm", "layer_output_scale", "attn_q", "attn_q_norm", "attn_output",
                         "post_attention_norm", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down", "post_ffw_norm")
ASSISTANT_GLOBAL_TENSORS = ("token_embd.weight", "output_norm.weight", "nextn.pre_projection.weight",
                            "nextn.post_projection.weight")


def assistant_tensor_names(acfg) -> list:
    """Every tensor the head's forward reads (``rope_freqs`` is carried by real files but not read: a block's RoPE is
    that of the backbone layer whose KV it attends against)."""
    names = list(ASSISTANT_GLOBAL_TENSORS)
    for i in range(acfg.n_blocks):
        names += [f"blk.{i}.{s}.weight" for s in ASSISTANT_BLOCK_SLOTS]
    return names


def assistant_expected_shapes(acfg, backbone: ModelConfig) -> Dict[str, tuple]:
    """Torch shapes (rows, cols) of every tensor, derived from the two configs; used to validate an artifact."""
    Ha, Hb, F = acfg.hidden, acfg.backbone_hidden, acfg.ffn
    out: Dict[str, tuple] = {"token_embd.weight": (acfg.vocab, Ha), "output_norm.weight": (Ha,),
                             "nextn.pre_projection.weight": (Ha, 2 * Hb), "nextn.post_projection.weight": (Hb, Ha)}
    for i in range(acfg.n_blocks):
        D = backbone.layer_head_dim(acfg.backbone_layer(i, backbone))
        p = f"blk.{i}."
        out.update({p + "attn_norm.weight": (Ha,), p + "layer_output_scale.weight": (1,),
                    p + "attn_q.weight": (acfg.n_heads * D, Ha), p + "attn_q_norm.weight": (D,),
                    p + "attn_output.weight": (Ha, acfg.n_heads * D), p + "post_attention_norm.weight": (Ha,),
                    p + "ffn_norm.weight": (Ha,), p + "ffn_gate.weight": (F, Ha), p + "ffn_up.weight": (F, Ha),
                    p + "ffn_down.weight": (Ha, F), p + "post_ffw_norm.weight": (Ha,)})
    return out


def assistant_config_from_gguf(info):
    """``AssistantConfig`` from the metadata of a ``gemma4-assistant`` file
    (reference: ``hipengine/loading/gemma4_assistant_gguf.py``, keys listed in
    ``docs/reference/GEMMA4-ASSISTANT-MTP.md:36-56``)."""
    from ..models.config import AssistantConfig
    if info.architecture != ASSISTANT_ARCH:
        raise ValueError(f"not an assistant head: general.architecture is {info.architecture!r}")
    g = lambda k, d=None: info.metadata.get(f"{ASSISTANT_ARCH}.{k}", d)
    n_blocks = int(g("block_count"))
    pat = g("attention.sliding_window_pattern")
    if isinstance(pat, (list, tuple)) and len(pat) == n_blocks:
        swa = tuple(bool(x) for x in pat)
    else:
        swa = tuple([True] * (n_blocks - 1) + [False])
    vocab = g("vocab_size")
    if vocab is None:
        vocab = info.tensor("token_embd.weight").torch_shape[0]
    return AssistantConfig(n_blocks=n_blocks, hidden=int(g("embedding_length")),
                           backbone_hidden=int(g("embedding_length_out")), ffn=int(g("feed_forward_length")),
                           n_heads=int(g("attention.head_count")), vocab=int(vocab), swa_blocks=swa,
                           rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)))


def validate_assistant(weights: ModelWeights, backbone: ModelConfig) -> None:
    """Pairing + tensor-map + shape checks of a head against the backbone it will draft for; raises with every
    problem listed."""
    acfg = weights.config
    acfg.check_pairing(backbone)
    errs = []
    for name, shape in assistant_expected_shapes(acfg, backbone).items():
        t = weights.get(name)
        if t is None:
            errs.append(f"missing {name}")
        elif tuple(t.shape) != tuple(shape):
            errs.append(f"{name}: shape {tuple(t.shape)} != {tuple(shape)}")
    if errs:
        raise ValueError("assistant head artifact rejected: " + "; ".join(errs[:8]))


def load_assistant_gguf(path, backbone: ModelConfig, device="cpu") -> ModelWeights:
    """Read a ``gemma4-assistant`` GGUF file (local path only) and validate it against ``backbone``."""
    import numpy as np
    from .gguf import GGUFReader, discover_gguf_files
    from .weights import QTensor
    files = discover_gguf_files(path)
    if not files:
        raise FileNotFoundError(f"no GGUF file at {path}")
    rd = GGUFReader(files[0])
    try:
        acfg = assistant_config_from_gguf(rd.info)
        tensors = {}
        for name, ti in rd.info.tensors.items():
            host = torch.from_numpy(np.array(rd.tensor_data(name), copy=True))
            tensors[name] = QTensor(name, ti.ggml_type, ti.torch_shape, host.to(device))
        w = ModelWeights(acfg, tensors, dict(rd.info.metadata))
    finally:
        rd.close()
    validate_assistant(w, backbone)
    return w


def assistant_metadata(acfg) -> Dict[str, Any]:
    a = ASSISTANT_ARCH
    return {"general.architecture": a, f"{a}.block_count": acfg.n_blocks, f"{a}.embedding_length": acfg.hidden,
            f"{a}.embedding_length_out": acfg.backbone_hidden, f"{a}.feed_forward_length": acfg.ffn,
            f"{a}.attention.head_count": acfg.n_heads, f"{a}.vocab_size": acfg.vocab,
            f"{a}.attention.sliding_window_pattern": [int(x) for x in acfg.swa_blocks],
            f"{a}.attention.layer_norm_rms_epsilon": float(acfg.rms_eps), f"{a}.nextn_predict_layers": acfg.n_blocks}


def build_random_assistant(acfg, backbone: ModelConfig, seed: int = 0, device="cpu", std: float = 0.02) -> ModelWeights:
    """Random-init assistant head for ``backbone`` (Q8_0 matrices and F32 norms, as the published artifact)."""
    from .synth import _Builder
    acfg.check_pairing(backbone)
    b = _Builder(backbone, seed, device, "q8_0", std)
    Ha, Hb, F = acfg.hidden, acfg.backbone_hidden, acfg.ffn
    near1 = lambda n: b.ones(n) + b.randn(n, std=0.05)
    b.matrix("token_embd.weight", (acfg.vocab, Ha), GGMLType.Q8_0)
    b.f32("output_norm.weight", near1(Ha))
    b.matrix("nextn.pre_projection.weight", (Ha, 2 * Hb), GGMLType.Q8_0)
    b.matrix("nextn.post_projection.weight", (Hb, Ha), GGMLType.Q8_0, std=1.0 / (Ha ** 0.5))
    for i in range(acfg.n_blocks):
        D = backbone.layer_head_dim(acfg.backbone_layer(i, backbone))
        p = f"blk.{i}."
        b.f32(p + "attn_norm.weight", near1(Ha))
        b.f32(p + "layer_output_scale.weight", b.ones(1) * (1.0 - 0.02 * i))
        b.matrix(p + "attn_q.weight", (acfg.n_heads * D, Ha), GGMLType.Q8_0)
        # scale 1.0 attention against backbone keys whose norm weights are ~D**-0.25: keep q.k of order 1
        b.f32(p + "attn_q_norm.weight", near1(D) * (D ** -0.25))
        b.matrix(p + "attn_output.weight", (Ha, acfg.n_heads * D), GGMLType.Q8_0)
        b.f32(p + "post_attention_norm.weight", near1(Ha))
        b.f32(p + "ffn_norm.weight", near1(Ha))
        b.matrix(p + "ffn_gate.weight", (F, Ha), GGMLType.Q8_0)
        b.matrix(p + "ffn_up.weight", (F, Ha), GGMLType.Q8_0)
        b.matrix(p + "ffn_down.weight", (Ha, F), GGMLType.Q8_0)
        b.f32(p + "post_ffw_norm.weight", near1(Ha))
    return ModelWeights(acfg, b.out, assistant_metadata(acfg))
