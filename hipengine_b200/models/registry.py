"""Model family declarations: what each supported ``general.architecture`` is, which executor runs it, what its layer
schedule looks like, which speculative providers and KV storage modes it admits.

Pure metadata (the role of the reference's model plugins, ``hipengine/models/registry.py``, ``models/qwen35.py``,
``models/gemma4.py``: name, architectures, default quantisation, layer sequence, MTP serving and KV capability
declarations).  Used by the server's capability route and by error messages that must say what IS supported.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .config import ModelConfig


@dataclass(frozen=True)
class ModelPlugin:
    name: str
    architectures: Tuple[str, ...]
    executor: str                               # import path of the GPU executor class
    default_quant: str = "gguf_q4_k_m"
    native_block_types: Tuple[str, ...] = ("Q4_K", "Q6_K", "Q8_0", "F32", "F16", "BF16")
    widened_block_types: Tuple[str, ...] = ("Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q5_K")
    chat_template: str = "chatml"
    speculative_providers: Tuple[str, ...] = ("prompt_lookup", "ngram")
    kv_storage: Tuple[str, ...] = ("bf16",)
    tensor_parallel: bool = True
    expert_parallel: bool = False
    notes: str = ""

    def layer_sequence(self, cfg: ModelConfig) -> List[str]:
        """One word per layer of ``cfg``: ``linear`` (Gated-DeltaNet), ``full``, ``sliding`` or ``global``."""
        out = []
        for i in range(cfg.n_layers):
            if cfg.arch == "gemma4":
                out.append("global" if cfg.is_global_layer(i) else "sliding")
            elif cfg.is_hybrid:
                out.append("full" if cfg.is_full_attention_layer(i) else "linear")
            else:
                out.append("full")
        return out

    def describe(self, cfg: Optional[ModelConfig] = None) -> Dict[str, Any]:
        d: Dict[str, Any] = {"name": self.name, "architectures": list(self.architectures), "executor": self.executor,
                             "default_quant": self.default_quant, "native_block_types": list(self.native_block_types),
                             "widened_block_types": list(self.widened_block_types), "chat_template": self.chat_template,
                             "speculative_providers": list(self.speculative_providers),
                             "kv_storage": list(self.kv_storage), "tensor_parallel": self.tensor_parallel,
                             "expert_parallel": self.expert_parallel, "notes": self.notes}
        if cfg is not None:
            seq = self.layer_sequence(cfg)
            d["layers"] = {k: seq.count(k) for k in sorted(set(seq))}
            d["ffn"] = "moe" if cfg.is_moe else "dense"
            providers = list(self.speculative_providers)
            if "mtp" in providers and cfg.arch != "gemma4" and cfg.nextn_layers == 0:
                providers.remove("mtp")                         # this checkpoint carries no NextN block
            d["speculative_providers"] = providers
        return d


_HYBRID = "hipengine_b200.models.executor.HybridExecutor"
PLUGINS: Tuple[ModelPlugin, ...] = (
    ModelPlugin("qwen35-dense-hybrid", ("qwen35",), _HYBRID,
                speculative_providers=("mtp", "prompt_lookup", "ngram"),
                notes="3 Gated-DeltaNet layers : 1 gated full-attention layer; optional trailing NextN block"),
    ModelPlugin("qwen35-moe-hybrid", ("qwen35moe",), _HYBRID, expert_parallel=True,
                speculative_providers=("mtp", "prompt_lookup", "ngram"),
                notes="hybrid schedule with top-k routed experts and a gated shared expert"),
    ModelPlugin("dense-decoder", ("qwen3", "llama"), _HYBRID, notes="full attention in every layer"),
    ModelPlugin("moe-decoder", ("qwen3moe",), _HYBRID, expert_parallel=True),
    ModelPlugin("gemma4-moe", ("gemma4",), "hipengine_b200.models.gemma4.Gemma4Executor", default_quant="gguf_q4_k_xl",
                chat_template="gemma", speculative_providers=("gemma4_mtp", "prompt_lookup", "ngram"),
                tensor_parallel=False,
                notes="5 sliding-window layers : 1 global layer, dense GeGLU branch beside top-k experts; the MTP "
                      "drafter is the separate gemma4-assistant artifact"),
)


def plugin_for(arch: str) -> ModelPlugin:
    for p in PLUGINS:
        if arch in p.architectures:
            return p
    known = sorted(a for p in PLUGINS for a in p.architectures)
    raise KeyError(f"no model plugin for architecture {arch!r}; supported: {known}")


def supported_architectures() -> List[str]:
    return sorted(a for p in PLUGINS for a in p.architectures)
