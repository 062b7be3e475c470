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


def test_spm_tokenizer_round_trip_and_scores():
    from hipengine_b200.tokenization.gguf_tokenizer import GGUFSPMTokenizer, tokenizer_from_metadata
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + \
           ["\u2581", "h", "e", "l", "o", "w", "r", "d", "he", "ll", "llo", "hello", "\u2581hello", "\u2581w", "or", "ld",
            "\u2581world", "<start_of_turn>"]
    scores = [0.0] * 259 + [-1, -2, -2, -2, -2, -2, -2, -2, -3, -3, -4, -5, -6, -4, -4, -4, -7, 0]
    types = [2, 3, 3] + [6] * 256 + [1] * 17 + [4]
    tk = GGUFSPMTokenizer(toks, scores, types, eos_id=2, bos_id=1)
    ids = tk.encode("hello world")
    assert [toks[i] for i in ids] == ["hello", "\u2581w", "or", "ld"]      # best-scored merges win step by step
    assert tk.decode(ids) == "hello world"
    ids = tk.encode("<start_of_turn>hé")                                    # special token + byte fallback for é
    assert ids[0] == tk.special["<start_of_turn>"] and toks[ids[1]] == "h"
    assert [toks[i] for i in ids[2:]] == ["<0xC3>", "<0xA9>"] and tk.decode(ids) == "<start_of_turn>hé"
    meta = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": scores,
            "tokenizer.ggml.token_type": types, "tokenizer.ggml.eos_token_id": 2}
    assert isinstance(tokenizer_from_metadata(meta, len(toks)), GGUFSPMTokenizer)


def test_local_only_model_resolution(tmp_path, monkeypatch):
    from hipengine_b200.loading.hf_cache import ModelNotFound, resolve_model_path
    hub = tmp_path / "hub"
    snap = hub / "models--org--m" / "snapshots" / "abc"
    snap.mkdir(parents=True)
    (hub / "models--org--m" / "refs").mkdir()
    (hub / "models--org--m" / "refs" / "main").write_text("abc")
    for n in ("m-Q4_K_M-00001-of-00002.gguf", "m-Q4_K_M-00002-of-00002.gguf", "m-Q8_0.gguf", "mmproj-m.gguf"):
        (snap / n).write_bytes(b"GGUF")
    monkeypatch.setenv("HF_HUB_CACHE", str(hub))
    monkeypatch.delenv("HE_MODEL_DIR", raising=False)
    got = resolve_model_path("org/m", quant_hint="q4_k_m")
    assert [p.name for p in got] == ["m-Q4_K_M-00001-of-00002.gguf", "m-Q4_K_M-00002-of-00002.gguf"]
    assert [p.name for p in resolve_model_path("org/m", quant_hint="q8_0")] == ["m-Q8_0.gguf"]
    assert resolve_model_path(str(snap / "m-Q8_0.gguf"))[0].name == "m-Q8_0.gguf"
    import pytest
    with pytest.raises(ModelNotFound, match="never downloaded"):
        resolve_model_path("org/absent")


def test_model_source_is_described_from_the_header_alone(tmp_path, capsys):
    """The server's ``--info`` names what ``--model`` is before anything is loaded: a GGUF file by its header
    (architecture, geometry, bytes per block type), a built-in geometry by name, and an error with exit code 2 for a
    path that is neither, a directory without a GGUF file, a truncated file or an unsupported architecture."""
    import json
    from hipengine_b200.loading.gguf import GGUFWriter
    from hipengine_b200.loading.model_loader import describe_model_source
    from hipengine_b200.server.__main__ import main
    w = build_random_model(TINY_HYBRID, seed=0)
    p = write_gguf(w, tmp_path / "hy.gguf")
    d = describe_model_source(p)
    assert d["source"] == "gguf" and d["arch"] == "qwen35" and d["layers"] == TINY_HYBRID.n_layers
    assert d["tensors"] == len(w.tensors) and d["weight_bytes"] == sum(d["bytes_by_block_type"].values())
    assert d["weight_bytes"] <= d["file_bytes"] and "Q4_K" in d["bytes_by_block_type"]
    assert d["family"]["layers"] == {"full": 1, "linear": 3}
    assert describe_model_source(tmp_path)["path"].endswith("hy.gguf")          # a directory holding the file
    assert describe_model_source("tiny-dense")["source"].startswith("built-in")
    assert "error" in describe_model_source(tmp_path / "missing.gguf")
    empty = tmp_path / "empty_dir"
    empty.mkdir()
    assert "no *.gguf" in describe_model_source(empty)["error"]
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(p.read_bytes()[:100])
    assert "error" in describe_model_source(cut)
    other = GGUFWriter(tmp_path / "other.gguf", "mamba")
    other.add_tensor("x", torch.zeros(2, 32), GGMLType.F32)
    other.write()
    assert "unsupported GGUF architecture" in describe_model_source(tmp_path / "other.gguf")["error"]
    assert main(["--model", str(p), "--info"]) == 0
    assert json.loads(capsys.readouterr().out)["model"]["arch"] == "qwen35"
    assert main(["--model", str(tmp_path / "missing.gguf"), "--info"]) == 2
    assert "neither" in json.loads(capsys.readouterr().out)["model"]["error"]
