"""Weight containers and the GGUF tensor-name map for the supported families.

Tensor slot names follow the GGUF convention the reference maps in
``hipengine/loading/qwen35_gguf.py:15-83``: per-block ``attn_norm``,
``post_attention_norm``; linear-attention blocks ``attn_qkv, attn_gate, ssm_a,
ssm_alpha, ssm_beta, ssm_conv1d, ssm_dt.bias, ssm_norm, ssm_out``; full-attention
blocks ``attn_q`` (interleaved ``[Q | gate]`` per head), ``attn_k, attn_v,
attn_output, attn_q_norm, attn_k_norm``; dense FFN ``ffn_gate/up/down``; MoE
``ffn_gate_inp, ffn_gate_inp_shexp, ffn_{gate,up,down}_exps,
ffn_{gate,up,down}_shexp``; roots ``token_embd, output_norm, output``; NextN
tensors ``nextn.eh_proj, nextn.enorm, nextn.hnorm`` (+ optional
``nextn.embed_tokens, nextn.shared_head_head, nextn.shared_head_norm``) in the
trailing block that plain decoding ignores.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..models.config import ModelConfig
from ..quant.ggml import GGMLType, dequantize_torch, layout_of, row_bytes


@dataclass
class QTensor:
    """One checkpoint tensor kept in its on-disk GGML encoding.

    ``shape`` is row-major (slowest first).  A 2-D weight is ``[N, K]`` (``y = x @ W^T``);
    stacked expert weights are ``[E, N, K]``.  ``raw`` is ``uint8 [rows, row_bytes]``.
    """
    name: str
    ggml_type: GGMLType
    shape: Tuple[int, ...]
    raw: torch.Tensor

    @property
    def n_cols(self) -> int:
        return self.shape[-1]

    @property
    def n_rows(self) -> int:
        r = 1
        for s in self.shape[:-1]:
            r *= s
        return r

    @property
    def is_quantized(self) -> bool:
        return layout_of(self.ggml_type).block_elems > 1

    def dequant(self, device=None) -> torch.Tensor:
        raw = self.raw if device is None else self.raw.to(device)
        return dequantize_torch(raw, self.ggml_type, self.n_rows, self.n_cols).reshape(self.shape)

    def float(self) -> torch.Tensor:
        return self.dequant()

    def to(self, device) -> "QTensor":
        return QTensor(self.name, self.ggml_type, self.shape, self.raw.to(device))

    def rows(self, r0: int, r1: int) -> "QTensor":
        """Row slice of a 2-D tensor (column-parallel shard)."""
        assert len(self.shape) == 2
        return QTensor(self.name, self.ggml_type, (r1 - r0, self.shape[1]), self.raw[r0:r1].contiguous())

    def cols(self, c0: int, c1: int) -> "QTensor":
        """Column slice on block boundaries (row-parallel shard)."""
        lay = layout_of(self.ggml_type)
        assert c0 % lay.block_elems == 0 and c1 % lay.block_elems == 0, "shard must fall on quant-block boundaries"
        b0 = c0 // lay.block_elems * lay.block_bytes
        b1 = c1 // lay.block_elems * lay.block_bytes
        lead = self.shape[:-1]
        return QTensor(self.name, self.ggml_type, lead + (c1 - c0,), self.raw[:, b0:b1].contiguous())

    def expert(self, e: int) -> "QTensor":
        assert len(self.shape) == 3
        n = self.shape[1]
        return QTensor(f"{self.name}[{e}]", self.ggml_type, self.shape[1:], self.raw[e * n:(e + 1) * n])


@dataclass
class ModelWeights:
    config: ModelConfig
    tensors: Dict[str, QTensor] = field(default_factory=dict)
    metadata: Dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, name: str) -> QTensor:
        try:
            return self.tensors[name]
        except KeyError:
            raise KeyError(f"weight {name!r} missing") from None

    def get(self, name: str) -> Optional[QTensor]:
        return self.tensors.get(name)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def blk(self, i: int, slot: str) -> QTensor:
        return self[f"blk.{i}.{slot}"]

    def to(self, device) -> "ModelWeights":
        return ModelWeights(self.config, {k: v.to(device) for k, v in self.tensors.items()}, dict(self.metadata))

    def nbytes(self) -> int:
        return sum(t.raw.numel() for t in self.tensors.values())

    @property
    def lm_head(self) -> QTensor:
        return self.tensors.get("output.weight") or self.tensors["token_embd.weight"]


# ----------------------------------------------------------------------------- name maps

LINEAR_SLOTS = ("attn_norm.weight", "post_attention_norm.weight", "attn_qkv.weight", "attn_gate.weight",
                "ssm_a", "ssm_alpha.weight", "ssm_beta.weight", "ssm_conv1d.weight", "ssm_dt.bias",
                "ssm_norm.weight", "ssm_out.weight")
FULL_SLOTS = ("attn_norm.weight", "post_attention_norm.weight", "attn_q.weight", "attn_k.weight",
              "attn_v.weight", "attn_output.weight")
FULL_QK_NORM_SLOTS = ("attn_q_norm.weight", "attn_k_norm.weight")
DENSE_FFN_SLOTS = ("ffn_gate.weight", "ffn_up.weight", "ffn_down.weight")
MOE_FFN_SLOTS = ("ffn_gate_inp.weight", "ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight")
MOE_SHARED_SLOTS = ("ffn_gate_inp_shexp.weight", "ffn_gate_shexp.weight", "ffn_up_shexp.weight",
                    "ffn_down_shexp.weight")
NEXTN_SLOTS = ("nextn.eh_proj.weight", "nextn.enorm.weight", "nextn.hnorm.weight")
NEXTN_OPTIONAL_SLOTS = ("nextn.embed_tokens.weight", "nextn.shared_head_head.weight",
                        "nextn.shared_head_norm.weight")
ROOT_SLOTS = ("token_embd.weight", "output_norm.weight")


def ffn_norm_slot(cfg: ModelConfig) -> str:
    """Hybrid Qwen files call the pre-FFN norm ``post_attention_norm``; plain dense ones ``ffn_norm``."""
    return "post_attention_norm.weight" if cfg.arch.startswith("qwen35") else "ffn_norm.weight"


def expected_tensor_names(cfg: ModelConfig, include_nextn: bool = True) -> List[str]:
    names: List[str] = list(ROOT_SLOTS)
    if not cfg.tie_embeddings:
        names.append("output.weight")
    n_blocks = cfg.n_layers + (cfg.nextn_layers if include_nextn else 0)
    for i in range(n_blocks):
        is_nextn = i >= cfg.n_layers
        full = True if is_nextn else cfg.is_full_attention_layer(i)
        p = f"blk.{i}."
        names.append(p + "attn_norm.weight")
        names.append(p + ffn_norm_slot(cfg))
        if full:
            names += [p + s for s in ("attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight")]
            if cfg.qk_norm:
                names += [p + s for s in FULL_QK_NORM_SLOTS]
        else:
            names += [p + s for s in LINEAR_SLOTS if s not in ("attn_norm.weight", "post_attention_norm.weight")]
        if cfg.is_moe:
            names += [p + s for s in MOE_FFN_SLOTS]
            if cfg.shared_ffn:
                names += [p + s for s in MOE_SHARED_SLOTS]
        else:
            names += [p + s for s in DENSE_FFN_SLOTS]
        if is_nextn:
            names += [p + s for s in NEXTN_SLOTS]
    return names
