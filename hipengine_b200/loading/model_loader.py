"""GGUF file -> ``ModelConfig`` + ``ModelWeights``.

Geometry comes from the ``{arch}.*`` metadata keys the reference reads in
``hipengine/loading/qwen35_gguf.py:708-767`` (block_count, embedding_length,
attention.head_count(_kv), key_length, full_attention_interval,
rope.dimension_count, rope.freq_base, ssm.*, expert_*).  Weight bytes are
copied out of the memory map into pinned host tensors (or straight to the
device) without any re-encoding, so what the kernels see is bit-identical to
the file.  Model paths are local only: a file, or a directory of ``*.gguf``;
nothing is ever downloaded (``hipengine/loading/hf_cache.py`` has the same rule).
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..models.config import ModelConfig
from ..quant.ggml import GGMLType
from .gguf import GGUFModelInfo, GGUFReader, discover_gguf_files, scan_gguf
from .weights import ModelWeights, QTensor, expected_tensor_names

SUPPORTED_ARCHS = ("qwen35", "qwen35moe", "qwen3", "qwen3moe", "llama", "gemma4")


def config_from_gguf(info: GGUFModelInfo) -> ModelConfig:
    a = info.architecture
    if a not in SUPPORTED_ARCHS:
        raise ValueError(f"unsupported GGUF architecture {a!r}; supported: {SUPPORTED_ARCHS}")
    g = lambda k, d=None: info.metadata.get(f"{a}.{k}", d)
    hidden = int(g("embedding_length"))
    n_heads = int(g("attention.head_count"))
    nextn = int(g("nextn_predict_layers", 0) or 0)
    n_blocks = int(g("block_count"))
    head_dim = int(g("attention.key_length", hidden // n_heads))
    vocab = g("vocab_size")
    if vocab is None:
        vocab = info.tensor("token_embd.weight").shape[1]
    fai = int(g("full_attention_interval", 0) or 0)
    if a.startswith("qwen35") and fai == 0:
        fai = 4
    gated = bool(g("attention.gated", a.startswith("qwen35")))
    qk_norm = bool(g("attention.qk_norm", "blk.%d.attn_q_norm.weight" % ((fai - 1) if fai else 0) in info.tensors))
    kw = dict(
        arch=a, n_layers=n_blocks - nextn, hidden=hidden, vocab=int(vocab), n_heads=n_heads,
        n_kv_heads=int(g("attention.head_count_kv", n_heads)), head_dim=head_dim,
        ffn=int(g("feed_forward_length", 0) or 0),
        rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)),
        rope_theta=float(g("rope.freq_base", 1e7 if a.startswith("qwen35") else 1e6)),
        rope_dim=int(g("rope.dimension_count", head_dim)),
        gated_attention=gated, qk_norm=qk_norm, full_attention_interval=fai,
        ssm_groups=int(g("ssm.group_count", 0) or 0), ssm_v_heads=int(g("ssm.time_step_rank", 0) or 0),
        ssm_state=int(g("ssm.state_size", 128) or 128), conv_kernel=int(g("ssm.conv_kernel", 4) or 4),
        n_experts=int(g("expert_count", 0) or 0), n_experts_used=int(g("expert_used_count", 0) or 0),
        expert_ffn=int(g("expert_feed_forward_length", 0) or 0),
        shared_ffn=int(g("expert_shared_feed_forward_length", 0) or 0),
        nextn_layers=nextn, max_context=int(g("context_length", 8192)),
        tie_embeddings="output.weight" not in info.tensors,
    )
    if a == "gemma4":
        from .gemma4 import gemma4_config_overrides
        kw.update(gemma4_config_overrides(info))
    return ModelConfig(**kw)


def describe_model_source(model) -> Dict[str, object]:
    """What ``model`` names, found without reading a tensor: a built-in random-init geometry, or a GGUF file whose
    header gives the architecture, the geometry, the histogram of block types and the bytes the weights will take.
    ``{"error": ...}`` when it is neither (nothing is ever downloaded) or when the header cannot serve this engine.
    The server's ``--info`` prints it, so a wrong path or an unsupported file shows before any load is attempted."""
    from pathlib import Path
    from ..models.config import NAMED_CONFIGS
    from ..models.registry import plugin_for

    def geometry(cfg: ModelConfig) -> Dict[str, object]:
        out = {"arch": cfg.arch, "layers": cfg.n_layers, "hidden": cfg.hidden, "vocab": cfg.vocab,
               "ffn": "moe" if cfg.is_moe else "dense", "nextn_layers": cfg.nextn_layers,
               "max_context": cfg.max_context}
        try:
            out["family"] = plugin_for(cfg.arch).describe(cfg)
        except KeyError:
            out["family"] = None
        return out

    name = str(model)
    files = discover_gguf_files(name)
    if files:
        try:
            info = scan_gguf(files[0])
            cfg = config_from_gguf(info)
        except Exception as e:                                  # a truncated header, an unsupported architecture
            return {"source": "gguf", "path": str(files[0]), "error": f"{type(e).__name__}: {e}"}
        hist: Dict[str, int] = {}
        for t in info.tensors.values():
            hist[t.ggml_type.name] = hist.get(t.ggml_type.name, 0) + t.nbytes
        return {"source": "gguf", "path": str(files[0]), "files": len(files), "file_bytes": files[0].stat().st_size,
                "gguf_version": info.version, "tensors": info.tensor_count, "weight_bytes": info.total_tensor_nbytes,
                "bytes_by_block_type": dict(sorted(hist.items(), key=lambda kv: -kv[1])),
                "name": info.get("general.name"), **geometry(cfg)}
    if Path(name).exists():
        return {"source": "path", "path": name, "error": "no *.gguf file there"}
    if name in NAMED_CONFIGS:
        return {"source": "built-in geometry (random weights)", "name": name, **geometry(NAMED_CONFIGS[name])}
    return {"source": "unknown", "error": f"{name!r} is neither a local GGUF path nor a built-in geometry "
                                          f"({sorted(NAMED_CONFIGS)})"}


def load_gguf_model(path, device="cpu", pin: bool = False, validate: bool = True) -> ModelWeights:
    files = discover_gguf_files(path)
    if not files:
        raise FileNotFoundError(f"no GGUF file at {path}")
    rd = GGUFReader(files[0])
    try:
        cfg = config_from_gguf(rd.info)
        tensors: Dict[str, QTensor] = {}
        dev = torch.device(device)
        for name, ti in rd.info.tensors.items():
            data = rd.tensor_data(name)
            host = torch.from_numpy(np.array(data, copy=True))
            if pin and torch.cuda.is_available():
                host = host.pin_memory()
            raw = host.to(dev, non_blocking=pin) if dev.type != "cpu" else host
            tensors[name] = QTensor(name, ti.ggml_type, ti.torch_shape, raw)
        if validate and cfg.arch != "gemma4":
            missing = [n for n in expected_tensor_names(cfg) if n not in tensors]
            if missing:
                raise KeyError(f"{files[0]}: missing tensors for {cfg.arch}: {missing[:6]}")
        return ModelWeights(cfg, tensors, dict(rd.info.metadata))
    finally:
        rd.close()
