"""Model geometry for the supported decoder families.

One dataclass covers plain dense decoders, the Qwen3.5-family hybrid
(Gated-DeltaNet linear attention + gated full attention, dense or MoE FFN) and
Gemma 4 (sliding-window/global attention + MoE).  The three pinned Qwen3.5
geometries mirror the identities the reference pins in
``hipengine/kernels/policy.py:103-153``; the Gemma 4 26B-A4B numbers come from
``docs/model-cards/MODEL-GEMMA4.md:128-155`` of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class ModelConfig:
    arch: str = "qwen35"                 # general.architecture of the GGUF file
    n_layers: int = 4
    hidden: int = 256
    vocab: int = 4096
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 768
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_dim: int = 64                   # rotated dims per head (partial rotary when < head_dim)
    # attention flavour
    gated_attention: bool = False        # attn_q projects [Q | gate] per head; out *= sigmoid(gate)
    qk_norm: bool = False
    attn_scale: Optional[float] = None   # None -> head_dim ** -0.5
    # hybrid schedule: layer i is full attention iff (i + 1) % full_attention_interval == 0
    full_attention_interval: int = 0     # 0 -> every layer is full attention
    # Gated DeltaNet (linear attention) geometry
    ssm_groups: int = 0                  # number of K heads
    ssm_v_heads: int = 0                 # number of V heads (= time_step_rank)
    ssm_state: int = 128                 # Dk = Dv
    conv_kernel: int = 4
    # MoE
    n_experts: int = 0
    n_experts_used: int = 0
    expert_ffn: int = 0
    shared_ffn: int = 0
    # Gemma-style extras
    sliding_window: int = 0
    swa_pattern: int = 0                 # every swa_pattern-th layer is global, the rest sliding
    global_head_dim: int = 0
    global_kv_heads: int = 0
    final_softcap: float = 0.0
    embed_scale: float = 1.0
    act: str = "silu"                    # "silu" | "gelu_tanh"
    tie_embeddings: bool = False
    # MTP / NextN draft blocks appended after the main stack
    nextn_layers: int = 0
    max_context: int = 8192

    swa_rope_theta: float = 10000.0      # Gemma: sliding layers rotate the whole head with this base
    global_rope_fraction: float = 0.25   # Gemma: global layers rotate this fraction of the head ("proportional")

    # ---- derived
    def is_global_layer(self, i: int) -> bool:
        """Gemma-style schedule: every ``swa_pattern``-th layer attends globally, the rest use a sliding window."""
        return self.swa_pattern > 0 and (i + 1) % self.swa_pattern == 0

    def layer_head_dim(self, i: int) -> int:
        return self.global_head_dim if (self.is_global_layer(i) and self.global_head_dim) else self.head_dim

    def layer_kv_heads(self, i: int) -> int:
        return self.global_kv_heads if (self.is_global_layer(i) and self.global_kv_heads) else self.n_kv_heads

    def layer_window(self, i: int) -> int:
        return 0 if (self.swa_pattern == 0 or self.is_global_layer(i)) else self.sliding_window

    @property
    def is_hybrid(self) -> bool:
        return self.full_attention_interval > 0

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def ssm_inner(self) -> int:
        return self.ssm_v_heads * self.ssm_state

    @property
    def linear_qkv_width(self) -> int:
        return 2 * self.ssm_groups * self.ssm_state + self.ssm_inner

    @property
    def q_width(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def q_proj_width(self) -> int:
        return self.q_width * (2 if self.gated_attention else 1)

    def is_full_attention_layer(self, i: int) -> bool:
        if not self.is_hybrid:
            return True
        return (i + 1) % self.full_attention_interval == 0

    def layer_kinds(self) -> Tuple[str, ...]:
        return tuple("full" if self.is_full_attention_layer(i) else "linear" for i in range(self.n_layers))

    @property
    def n_full_layers(self) -> int:
        return sum(1 for k in self.layer_kinds() if k == "full")

    @property
    def n_linear_layers(self) -> int:
        return self.n_layers - self.n_full_layers

    def scale(self) -> float:
        return self.attn_scale if self.attn_scale is not None else self.head_dim ** -0.5

    def kv_bytes_per_token(self, elem_bytes: int = 2) -> int:
        return self.n_full_layers * 2 * self.n_kv_heads * self.head_dim * elem_bytes

    def recurrent_state_bytes(self) -> int:
        gdn = self.n_linear_layers * self.ssm_v_heads * self.ssm_state * self.ssm_state * 4
        conv = self.n_linear_layers * self.linear_qkv_width * self.conv_kernel * 4
        return gdn + conv

    def with_layers(self, n_layers: int) -> "ModelConfig":
        return replace(self, n_layers=n_layers)


# Tiny dense decoder of the CPU reference backend benchmark (4 layers, hidden 256, Q4_K weights).
TINY_DENSE = ModelConfig(arch="qwen3", n_layers=4, hidden=256, vocab=4096, n_heads=4, n_kv_heads=2,
                         head_dim=64, ffn=768, rms_eps=1e-6, rope_theta=1e6, rope_dim=64)

# Dense hybrid 27B: 64 layers [3 GDN + 1 gated full attention] x 16.
QWEN35_27B = ModelConfig(arch="qwen35", n_layers=64, hidden=5120, vocab=248320, n_heads=24, n_kv_heads=4,
                         head_dim=256, ffn=17408, rms_eps=1e-6, rope_theta=1e7, rope_dim=64,
                         gated_attention=True, qk_norm=True, full_attention_interval=4,
                         ssm_groups=16, ssm_v_heads=48, ssm_state=128, conv_kernel=4,
                         max_context=262144)

# MoE hybrid 35B-A3B: 40 layers, 256 experts top-8 + shared expert.
QWEN35_35B_A3B = ModelConfig(arch="qwen35moe", n_layers=40, hidden=2048, vocab=248320, n_heads=16, n_kv_heads=2,
                             head_dim=256, ffn=0, rms_eps=1e-6, rope_theta=1e7, rope_dim=64,
                             gated_attention=True, qk_norm=True, full_attention_interval=4,
                             ssm_groups=16, ssm_v_heads=32, ssm_state=128, conv_kernel=4,
                             n_experts=256, n_experts_used=8, expert_ffn=512, shared_ffn=512,
                             max_context=262144)

# Small hybrid used by tests and the smoke entry (same structure, toy widths).
TINY_HYBRID = ModelConfig(arch="qwen35", n_layers=4, hidden=512, vocab=2048, n_heads=4, n_kv_heads=2,
                          head_dim=256, ffn=1024, rope_theta=1e7, rope_dim=64, gated_attention=True,
                          qk_norm=True, full_attention_interval=4, ssm_groups=2, ssm_v_heads=4,
                          ssm_state=128, conv_kernel=4, max_context=4096)

# Small hybrid geometry whose heads / K-head groups / FFN blocks split evenly over 2 ranks.
TINY_HYBRID_TP = ModelConfig(arch="qwen35", n_layers=4, hidden=512, vocab=2048, n_heads=4, n_kv_heads=2,
                             head_dim=256, ffn=1024, rope_theta=1e7, rope_dim=64, gated_attention=True,
                             qk_norm=True, full_attention_interval=4, ssm_groups=4, ssm_v_heads=8,
                             ssm_state=128, conv_kernel=4, max_context=4096)

# The same at a geometry that splits over 2, 4 and 8 ranks (16 K-head groups -> 2 per rank at 8; 8 heads; 8 FFN blocks).
SMALL_HYBRID_TP8 = ModelConfig(arch="qwen35", n_layers=4, hidden=512, vocab=2048, n_heads=8, n_kv_heads=2,
                               head_dim=256, ffn=2048, rope_theta=1e7, rope_dim=64, gated_attention=True,
                               qk_norm=True, full_attention_interval=4, ssm_groups=16, ssm_v_heads=32,
                               ssm_state=128, conv_kernel=4, max_context=4096)

TINY_HYBRID_MOE_TP = ModelConfig(arch="qwen35moe", n_layers=4, hidden=512, vocab=2048, n_heads=4, n_kv_heads=2,
                                 head_dim=256, ffn=0, rope_theta=1e7, rope_dim=64, gated_attention=True,
                                 qk_norm=True, full_attention_interval=4, ssm_groups=4, ssm_v_heads=8,
                                 ssm_state=128, conv_kernel=4, n_experts=16, n_experts_used=4,
                                 expert_ffn=256, shared_ffn=256, max_context=4096)

TINY_HYBRID_MOE = ModelConfig(arch="qwen35moe", n_layers=4, hidden=512, vocab=2048, n_heads=4, n_kv_heads=2,
                              head_dim=256, ffn=0, rope_theta=1e7, rope_dim=64, gated_attention=True,
                              qk_norm=True, full_attention_interval=4, ssm_groups=2, ssm_v_heads=4,
                              ssm_state=128, conv_kernel=4, n_experts=16, n_experts_used=4,
                              expert_ffn=256, shared_ffn=256, max_context=4096)

# Gemma 4 26B-A4B: 30 layers, 5 sliding (window 1024) : 1 global.
GEMMA4_26B_A4B = ModelConfig(arch="gemma4", n_layers=30, hidden=2816, vocab=262144, n_heads=16, n_kv_heads=8,
                             head_dim=256, ffn=2112, rms_eps=1e-6, rope_theta=1e6, rope_dim=256,
                             qk_norm=True, attn_scale=1.0, sliding_window=1024, swa_pattern=6,
                             global_head_dim=512, global_kv_heads=2, n_experts=128, n_experts_used=8,
                             expert_ffn=704, final_softcap=30.0, embed_scale=2816 ** 0.5,
                             act="gelu_tanh", tie_embeddings=True, max_context=262144)

TINY_GEMMA4 = ModelConfig(arch="gemma4", n_layers=6, hidden=256, vocab=2048, n_heads=4, n_kv_heads=2,
                          head_dim=64, ffn=288, rope_theta=1e6, rope_dim=64, qk_norm=True, attn_scale=1.0,
                          sliding_window=32, swa_pattern=6, global_head_dim=128, global_kv_heads=1,
                          n_experts=8, n_experts_used=2, expert_ffn=128, final_softcap=30.0,
                          embed_scale=16.0, act="gelu_tanh", tie_embeddings=True, max_context=2048)

@dataclass(frozen=True)
class AssistantConfig:
    """Gemma 4 assistant (MTP) head: a separate four-block draft model with no K/V projections of its own.  Every
    block attends against the backbone's KV of one of its last two layers (a sliding block reads layer ``n - 2``, a
    full-attention block layer ``n - 1``), so head count, KV heads, head width, window and RoPE of a block are those
    of the backbone layer it reads.  Contract: the reference's ``docs/reference/GEMMA4-ASSISTANT-MTP.md:36-60``
    (hyperparameters) and ``:62-80`` (tensor layout)."""
    arch: str = "gemma4-assistant"
    n_blocks: int = 4
    hidden: int = 1024                   # the head's own width
    backbone_hidden: int = 2816          # the target's width (``embedding_length_out``)
    ffn: int = 8192
    n_heads: int = 16
    vocab: int = 262144
    swa_blocks: Tuple[bool, ...] = (True, True, True, False)
    rms_eps: float = 1e-6

    def backbone_layer(self, il: int, backbone: ModelConfig) -> int:
        return backbone.n_layers - 2 if self.swa_blocks[il] else backbone.n_layers - 1

    def check_pairing(self, backbone: ModelConfig) -> None:
        """The head is only meaningful against the backbone it was trained with: refuse a mismatch before loading."""
        errs = []
        if backbone.arch != "gemma4":
            errs.append(f"backbone arch {backbone.arch!r} is not gemma4")
        if self.backbone_hidden != backbone.hidden:
            errs.append(f"embedding_length_out {self.backbone_hidden} != backbone width {backbone.hidden}")
        if self.n_heads != backbone.n_heads:
            errs.append(f"head count {self.n_heads} != backbone's {backbone.n_heads}")
        if self.vocab != backbone.vocab:
            errs.append(f"vocabulary {self.vocab} != backbone's {backbone.vocab}")
        if len(self.swa_blocks) != self.n_blocks:
            errs.append("sliding-window pattern length != block count")
        if backbone.n_layers >= 2 and backbone.arch == "gemma4":
            if backbone.is_global_layer(backbone.n_layers - 2) or not backbone.is_global_layer(backbone.n_layers - 1):
                errs.append("backbone's last two layers are not (sliding, global)")
        if (2 * self.backbone_hidden) % 256 or self.hidden % 256 or self.ffn % 256:
            errs.append("widths must be multiples of the 256-element block")
        if errs:
            raise ValueError("assistant head does not pair with this backbone: " + "; ".join(errs))


GEMMA4_26B_ASSISTANT = AssistantConfig()
TINY_GEMMA4_ASSISTANT = AssistantConfig(hidden=256, backbone_hidden=256, ffn=512, n_heads=4, vocab=2048)

NAMED_ASSISTANTS: Dict[str, AssistantConfig] = {
    "gemma4-26b-a4b": GEMMA4_26B_ASSISTANT,
    "tiny-gemma4": TINY_GEMMA4_ASSISTANT,
}

NAMED_CONFIGS: Dict[str, ModelConfig] = {
    "tiny-dense": TINY_DENSE,
    "tiny-hybrid": TINY_HYBRID,
    "tiny-hybrid-moe": TINY_HYBRID_MOE,
    "tiny-hybrid-tp": TINY_HYBRID_TP,
    "small-hybrid-tp8": SMALL_HYBRID_TP8,
    "tiny-hybrid-moe-tp": TINY_HYBRID_MOE_TP,
    "tiny-gemma4": TINY_GEMMA4,
    "qwen35-27b": QWEN35_27B,
    # the same geometries with the checkpoint's trailing NextN (MTP) block, for speculative serving runs
    "qwen35-27b-mtp": replace(QWEN35_27B, nextn_layers=1),
    "tiny-hybrid-mtp": replace(TINY_HYBRID, nextn_layers=1),
    "qwen35-35b-a3b": QWEN35_35B_A3B,
    "gemma4-26b-a4b": GEMMA4_26B_A4B,
}
