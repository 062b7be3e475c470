"""Random-init checkpoints in real GGUF encodings.

There is no network here for real checkpoints, so benchmarks and tests run on
weights drawn from N(0, 0.02) and quantized with the Q4_K_M-style recipe
(Q4_K for most matrices, Q6_K for the output head and for ``attn_v`` /
``ffn_down`` in the "more bits" layers, F32 for norms, routers and the small
SSM parameters).  Tensors are produced directly on the target device in row
chunks, so a 27B-parameter model is built on the GPU in seconds without ever
existing in fp32.  ``write_gguf`` serialises the same bytes to a GGUF file.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Optional

import torch

from ..models.config import ModelConfig
from ..quant.ggml import GGMLType, quantize, row_bytes
from .gguf import GGUFWriter
from .weights import ModelWeights, QTensor, ffn_norm_slot


def use_more_bits(i_layer: int, n_layers: int) -> bool:
    """llama.cpp's layer rule for the Q4_K_M / Q5_K_M mixes."""
    return (i_layer < n_layers // 8 or i_layer >= 7 * n_layers // 8
            or (i_layer - n_layers // 8) % 3 == 2)


def _pick(kind: GGMLType, k: int) -> GGMLType:
    if kind in (GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q5_K) and k % 256 != 0:
        return GGMLType.Q8_0 if k % 32 == 0 else GGMLType.F16
    return kind


class _Builder:
    def __init__(self, cfg: ModelConfig, seed: int, device, recipe: str, std: float):
        self.cfg = cfg
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.recipe = recipe
        self.std = std
        self.out: Dict[str, QTensor] = {}

    def base_type(self) -> GGMLType:
        return {"q4_k_m": GGMLType.Q4_K, "q4_k": GGMLType.Q4_K, "q8_0": GGMLType.Q8_0,
                "q6_k": GGMLType.Q6_K, "f16": GGMLType.F16, "bf16": GGMLType.BF16,
                "q4_k_xl": GGMLType.Q4_K}[self.recipe]

    def hi_type(self) -> GGMLType:
        return {"q4_k_m": GGMLType.Q6_K, "q4_k_xl": GGMLType.Q8_0}.get(self.recipe, self.base_type())

    def matrix(self, name: str, shape, kind: GGMLType, std: Optional[float] = None) -> None:
        std = self.std if std is None else std
        k = shape[-1]
        kind = _pick(kind, k)
        rows = 1
        for s in shape[:-1]:
            rows *= s
        rb = row_bytes(kind, k)
        raw = torch.empty(rows, rb, dtype=torch.uint8, device=self.device)
        chunk = max(1, min(rows, (64 << 20) // max(k, 1)))
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            w = torch.randn(r1 - r0, k, generator=self.gen, device=self.device, dtype=torch.float32) * std
            raw[r0:r1] = quantize(w, kind)
        self.out[name] = QTensor(name, kind, tuple(shape), raw)

    def f32(self, name: str, value: torch.Tensor) -> None:
        v = value.to(device=self.device, dtype=torch.float32).contiguous()
        shape = tuple(v.shape)
        raw = v.reshape(-1 if v.dim() == 1 else v.shape[0], -1) if v.dim() > 1 else v.reshape(1, -1)
        self.out[name] = QTensor(name, GGMLType.F32, shape, raw.view(torch.uint8))

    def randn(self, *shape, std=1.0) -> torch.Tensor:
        return torch.randn(*shape, generator=self.gen, device=self.device, dtype=torch.float32) * std

    def ones(self, *shape) -> torch.Tensor:
        return torch.ones(*shape, device=self.device, dtype=torch.float32)

    def rand(self, *shape) -> torch.Tensor:
        return torch.rand(*shape, generator=self.gen, device=self.device, dtype=torch.float32)


def build_random_model(cfg: ModelConfig, seed: int = 0, device="cpu", recipe: str = "q4_k_m",
                       std: float = 0.02) -> ModelWeights:
    """Random-init weights for ``cfg`` (Qwen3.5-family hybrids and plain dense decoders)."""
    if cfg.arch == "gemma4":
        from .gemma4 import build_random_gemma4
        return build_random_gemma4(cfg, seed=seed, device=device, recipe=recipe, std=std)
    b = _Builder(cfg, seed, device, recipe, std)
    base, hi = b.base_type(), b.hi_type()
    H = cfg.hidden
    b.matrix("token_embd.weight", (cfg.vocab, H), base)
    b.f32("output_norm.weight", b.ones(H))
    if not cfg.tie_embeddings:
        b.matrix("output.weight", (cfg.vocab, H), hi)
    n_blocks = cfg.n_layers + cfg.nextn_layers
    for i in range(n_blocks):
        is_nextn = i >= cfg.n_layers
        full = True if is_nextn else cfg.is_full_attention_layer(i)
        more = use_more_bits(min(i, cfg.n_layers - 1), cfg.n_layers)
        p = f"blk.{i}."
        b.f32(p + "attn_norm.weight", b.ones(H) + b.randn(H, std=0.02))
        b.f32(p + ffn_norm_slot(cfg), b.ones(H) + b.randn(H, std=0.02))
        if full:
            b.matrix(p + "attn_q.weight", (cfg.q_proj_width, H), base)
            b.matrix(p + "attn_k.weight", (cfg.kv_width, H), base)
            b.matrix(p + "attn_v.weight", (cfg.kv_width, H), hi if more else base)
            b.matrix(p + "attn_output.weight", (H, cfg.q_width), base)
            if cfg.qk_norm:
                b.f32(p + "attn_q_norm.weight", b.ones(cfg.head_dim) + b.randn(cfg.head_dim, std=0.02))
                b.f32(p + "attn_k_norm.weight", b.ones(cfg.head_dim) + b.randn(cfg.head_dim, std=0.02))
        else:
            Hv, inner, C = cfg.ssm_v_heads, cfg.ssm_inner, cfg.linear_qkv_width
            b.matrix(p + "attn_qkv.weight", (C, H), base)
            b.matrix(p + "attn_gate.weight", (inner, H), base)
            b.f32(p + "ssm_a", -(0.5 + 7.5 * b.rand(Hv)))
            b.f32(p + "ssm_alpha.weight", b.randn(Hv, H, std=std))
            b.f32(p + "ssm_beta.weight", b.randn(Hv, H, std=std))
            b.f32(p + "ssm_conv1d.weight", b.randn(C, cfg.conv_kernel, std=0.5))
            b.f32(p + "ssm_dt.bias", b.randn(Hv, std=0.5))
            b.f32(p + "ssm_norm.weight", b.ones(cfg.ssm_state) + b.randn(cfg.ssm_state, std=0.02))
            b.matrix(p + "ssm_out.weight", (H, inner), base)
        if cfg.is_moe:
            E, F = cfg.n_experts, cfg.expert_ffn
            b.f32(p + "ffn_gate_inp.weight", b.randn(E, H, std=std))
            b.matrix(p + "ffn_gate_exps.weight", (E, F, H), base)
            b.matrix(p + "ffn_up_exps.weight", (E, F, H), base)
            b.matrix(p + "ffn_down_exps.weight", (E, H, F), hi if more else base)
            if cfg.shared_ffn:
                S = cfg.shared_ffn
                b.f32(p + "ffn_gate_inp_shexp.weight", b.randn(1, H, std=std))
                b.matrix(p + "ffn_gate_shexp.weight", (S, H), GGMLType.Q8_0 if recipe != "f16" else base)
                b.matrix(p + "ffn_up_shexp.weight", (S, H), GGMLType.Q8_0 if recipe != "f16" else base)
                b.matrix(p + "ffn_down_shexp.weight", (H, S), GGMLType.Q8_0 if recipe != "f16" else base)
        else:
            b.matrix(p + "ffn_gate.weight", (cfg.ffn, H), base)
            b.matrix(p + "ffn_up.weight", (cfg.ffn, H), base)
            b.matrix(p + "ffn_down.weight", (H, cfg.ffn), hi if more else base)
        if is_nextn:
            b.matrix(p + "nextn.eh_proj.weight", (H, 2 * H), GGMLType.Q8_0 if recipe != "f16" else base)
            b.f32(p + "nextn.enorm.weight", b.ones(H))
            b.f32(p + "nextn.hnorm.weight", b.ones(H))
    meta = config_to_metadata(cfg)
    meta["general.name"] = f"random-init {cfg.arch} seed={seed} recipe={recipe}"
    return ModelWeights(cfg, b.out, meta)


def config_to_metadata(cfg: ModelConfig) -> Dict[str, object]:
    a = cfg.arch
    m: Dict[str, object] = {
        "general.architecture": a,
        f"{a}.block_count": cfg.n_layers + cfg.nextn_layers,
        f"{a}.embedding_length": cfg.hidden,
        f"{a}.feed_forward_length": cfg.ffn,
        f"{a}.context_length": cfg.max_context,
        f"{a}.vocab_size": cfg.vocab,
        f"{a}.attention.head_count": cfg.n_heads,
        f"{a}.attention.head_count_kv": cfg.n_kv_heads,
        f"{a}.attention.key_length": cfg.head_dim,
        f"{a}.attention.value_length": cfg.head_dim,
        f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
        f"{a}.rope.dimension_count": cfg.rope_dim,
        f"{a}.rope.freq_base": float(cfg.rope_theta),
    }
    if cfg.is_hybrid:
        m[f"{a}.full_attention_interval"] = cfg.full_attention_interval
        m[f"{a}.ssm.inner_size"] = cfg.ssm_inner
        m[f"{a}.ssm.group_count"] = cfg.ssm_groups
        m[f"{a}.ssm.state_size"] = cfg.ssm_state
        m[f"{a}.ssm.conv_kernel"] = cfg.conv_kernel
        m[f"{a}.ssm.time_step_rank"] = cfg.ssm_v_heads
    if cfg.is_moe:
        m[f"{a}.expert_count"] = cfg.n_experts
        m[f"{a}.expert_used_count"] = cfg.n_experts_used
        m[f"{a}.expert_feed_forward_length"] = cfg.expert_ffn
        m[f"{a}.expert_shared_feed_forward_length"] = cfg.shared_ffn
    if cfg.nextn_layers:
        m[f"{a}.nextn_predict_layers"] = cfg.nextn_layers
    if cfg.sliding_window:
        m[f"{a}.attention.sliding_window"] = cfg.sliding_window
        m[f"{a}.attention.sliding_window_pattern"] = cfg.swa_pattern
        m[f"{a}.attention.key_length_swa"] = cfg.head_dim
        m[f"{a}.attention.key_length"] = cfg.global_head_dim or cfg.head_dim
        m[f"{a}.attention.head_count_kv_global"] = cfg.global_kv_heads or cfg.n_kv_heads
        m[f"{a}.final_logit_softcapping"] = float(cfg.final_softcap)
    if cfg.gated_attention:
        m[f"{a}.attention.gated"] = True
    if cfg.qk_norm:
        m[f"{a}.attention.qk_norm"] = True
    return m


def write_gguf(weights: ModelWeights, path, tokenizer_vocab: Optional[list] = None) -> Path:
    """Serialise ``weights`` (already in GGML encodings) to a GGUF v3 file."""
    w = GGUFWriter(path, weights.config.arch)
    for k, v in weights.metadata.items():
        if k in ("general.architecture", "general.alignment"):
            continue
        if isinstance(v, float):
            w.add_f32(k, v)
        else:
            w.add_meta(k, v)
    if tokenizer_vocab is not None:
        w.add_meta("tokenizer.ggml.model", "gpt2")
        w.add_meta("tokenizer.ggml.tokens", list(tokenizer_vocab))
    for name, t in weights.tensors.items():
        w.add_tensor_raw(name, t.shape, t.ggml_type, t.raw.cpu().numpy())
    return w.write()
