"""GGUF writer -> scanner -> reader round trip, fingerprint stability, loader config recovery."""
import numpy as np
import torch

from hipengine_b200.loading.gguf import GGUFReader, execution_fingerprint, scan_gguf
from hipengine_b200.loading.model_loader import load_gguf_model
from hipengine_b200.loading.synth import build_random_model, write_gguf
from hipengine_b200.models.config import TINY_DENSE, TINY_HYBRID, TINY_HYBRID_MOE
from hipengine_b200.quant.ggml import GGMLType, dequantize_np


def test_round_trip_bit_exact(tmp_path):
    w = build_random_model(TINY_DENSE, seed=0)
    p = write_gguf(w, tmp_path / "tiny.gguf")
    info = scan_gguf(p)
    assert info.architecture == "qwen3" and info.tensor_count == len(w.tensors)
    assert info.data_offset % 32 == 0
    with GGUFReader(p) as rd:
        for name, t in w.tensors.items():
            ti = rd.tensor_info(name)
            assert ti.ggml_type == t.ggml_type and ti.torch_shape == t.shape
            assert ti.offset % 32 == 0
            raw = rd.tensor_data(name)
            assert np.array_equal(raw.reshape(-1), t.raw.numpy().reshape(-1))
        emb = rd.dequantize_tensor("token_embd.weight")
        ref = dequantize_np(w["token_embd.weight"].raw.numpy(), GGMLType.Q4_K, 4096, 256)
        assert np.array_equal(emb, ref)


def test_loader_recovers_config(tmp_path):
    for cfg in (TINY_DENSE, TINY_HYBRID, TINY_HYBRID_MOE):
        w = build_random_model(cfg, seed=1)
        p = write_gguf(w, tmp_path / f"{cfg.arch}.gguf")
        m = load_gguf_model(p)
        for f in ("n_layers", "hidden", "vocab", "n_heads", "n_kv_heads", "head_dim", "ffn", "rope_dim",
                  "full_attention_interval", "ssm_groups", "ssm_v_heads", "n_experts", "n_experts_used",
                  "expert_ffn", "shared_ffn", "gated_attention", "qk_norm"):
            assert getattr(m.config, f) == getattr(cfg, f), f
        assert abs(m.config.rope_theta - cfg.rope_theta) < 1
        for name, t in w.tensors.items():
            assert torch.equal(m[name].raw.reshape(-1), t.raw.reshape(-1))


def test_fingerprint_ignores_tokenizer_and_general(tmp_path):
    w = build_random_model(TINY_DENSE, seed=0)
    a = write_gguf(w, tmp_path / "a.gguf")
    w.metadata["general.name"] = "other"
    b = write_gguf(w, tmp_path / "b.gguf", tokenizer_vocab=["a", "b"])
    assert execution_fingerprint(scan_gguf(a)) == execution_fingerprint(scan_gguf(b))
    w.metadata["qwen3.rope.freq_base"] = 12345.0
    c = write_gguf(w, tmp_path / "c.gguf")
    assert execution_fingerprint(scan_gguf(a)) != execution_fingerprint(scan_gguf(c))
