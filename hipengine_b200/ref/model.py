"""Reference forward pass (PyTorch fp32 on dequantized weights).

This is the repo's "cpu_reference backend": a complete, incremental forward of
every supported text family written with the oracle ops in ``ref/ops.py``.  It
serves three purposes: (1) the oracle the CUDA executors are compared against
(teacher-forced logits at identical contexts, the comparison style the
reference documents in ``docs/TESTING.md:116-121``); (2) the CPU generation
path for the tiny dense benchmark config; (3) executable documentation of the
layer math listed in the reference's kernel sequence
(``hipengine/runtime/qwen35_gguf_layer_attn.py:474-1147``,
``hipengine/runtime/qwen35_gguf_layer_ffn.py:301-1278``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..loading.weights import ModelWeights, ffn_norm_slot
from ..models.config import ModelConfig
from . import ops as R


@dataclass
class RefState:
    """Per-request recurrent + KV state of the reference forward."""
    pos: int = 0
    k: Dict[int, torch.Tensor] = field(default_factory=dict)      # layer -> [S, Hkv, D]
    v: Dict[int, torch.Tensor] = field(default_factory=dict)
    conv: Dict[int, torch.Tensor] = field(default_factory=dict)   # layer -> [C, K-1]
    gdn: Dict[int, torch.Tensor] = field(default_factory=dict)    # layer -> [Hv, Dk, Dv]

    def clone(self) -> "RefState":
        c = lambda d: {i: t.clone() for i, t in d.items()}
        return RefState(self.pos, c(self.k), c(self.v), c(self.conv), c(self.gdn))


class RefModel:
    def __init__(self, weights: ModelWeights, dtype=torch.float32, device="cpu", kv_storage: str = "fp32"):
        """``kv_storage``: ``fp32`` keeps K/V exact (the oracle of the kernels), ``bf16`` / ``int8`` pass every stored
        row through that storage format first (``ref/ops.py::kv_store_roundtrip``)."""
        self.cfg = weights.config
        self.kv_storage = kv_storage
        self.device = torch.device(device)
        self.w: Dict[str, torch.Tensor] = {}
        for name, t in weights.tensors.items():
            self.w[name] = t.dequant().to(device=self.device, dtype=dtype)
        self.dtype = dtype
        if self.cfg.arch == "gemma4":
            from .gemma4 import Gemma4Ref
            self._gemma = Gemma4Ref(self)
        else:
            self._gemma = None

    # -- helpers
    def W(self, i: int, slot: str) -> torch.Tensor:
        return self.w[f"blk.{i}.{slot}"]

    def lin(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return x.to(self.dtype) @ w.t()

    def new_state(self) -> RefState:
        return RefState()

    # -- layers
    def full_attention(self, i: int, x: torch.Tensor, st: RefState, pos: torch.Tensor,
                       k_store: Optional[dict] = None, v_store: Optional[dict] = None,
                       layer_key: Optional[int] = None) -> torch.Tensor:
        cfg = self.cfg
        T = x.shape[0]
        H, Hkv, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        qf = self.lin(x, self.W(i, "attn_q.weight"))
        if cfg.gated_attention:
            qg = qf.reshape(T, H, 2, D)
            q, gate = qg[:, :, 0, :], qg[:, :, 1, :]
        else:
            q, gate = qf.reshape(T, H, D), None
        k = self.lin(x, self.W(i, "attn_k.weight")).reshape(T, Hkv, D)
        v = self.lin(x, self.W(i, "attn_v.weight")).reshape(T, Hkv, D)
        if cfg.qk_norm:
            q = R.rmsnorm(q, self.W(i, "attn_q_norm.weight"), cfg.rms_eps)
            k = R.rmsnorm(k, self.W(i, "attn_k_norm.weight"), cfg.rms_eps)
        q = R.rope_neox(q, pos, cfg.rope_theta, cfg.rope_dim)
        k = R.rope_neox(k, pos, cfg.rope_theta, cfg.rope_dim)
        ks = st.k if k_store is None else k_store
        vs = st.v if v_store is None else v_store
        key = i if layer_key is None else layer_key
        if self.kv_storage != "fp32":
            k, v = R.kv_store_roundtrip(k, self.kv_storage), R.kv_store_roundtrip(v, self.kv_storage)
        ks[key] = k if key not in ks else torch.cat([ks[key], k], 0)
        vs[key] = v.to(torch.float32) if key not in vs else torch.cat([vs[key], v.to(torch.float32)], 0)
        o = R.causal_gqa_attention(q, ks[key], vs[key], pos, cfg.scale())
        if gate is not None:
            o = o * torch.sigmoid(gate.to(torch.float32))
        return self.lin(o.reshape(T, H * D), self.W(i, "attn_output.weight"))

    def linear_attention(self, i: int, x: torch.Tensor, st: RefState) -> torch.Tensor:
        cfg = self.cfg
        T = x.shape[0]
        G, Hv, S = cfg.ssm_groups, cfg.ssm_v_heads, cfg.ssm_state
        C = cfg.linear_qkv_width
        qkv = self.lin(x, self.W(i, "attn_qkv.weight"))
        z = self.lin(x, self.W(i, "attn_gate.weight")).reshape(T, Hv, S)
        a = self.lin(x, self.W(i, "ssm_alpha.weight"))
        b = self.lin(x, self.W(i, "ssm_beta.weight"))
        if i not in st.conv:
            st.conv[i] = torch.zeros(C, cfg.conv_kernel - 1, dtype=torch.float32, device=x.device)
            st.gdn[i] = torch.zeros(Hv, S, S, dtype=torch.float32, device=x.device)
        conv_out, st.conv[i] = R.causal_conv1d_silu(qkv, self.W(i, "ssm_conv1d.weight"), st.conv[i])
        q = conv_out[:, :G * S].reshape(T, G, S)
        k = conv_out[:, G * S:2 * G * S].reshape(T, G, S)
        v = conv_out[:, 2 * G * S:].reshape(T, Hv, S)
        q = R.l2norm(q) * (S ** -0.5)
        k = R.l2norm(k)
        # GGUF tiled order: V head h uses K head h % G
        idx = torch.arange(Hv, device=x.device) % G
        qh, kh = q[:, idx], k[:, idx]
        decay, beta = R.gdn_gates(a, b, self.W(i, "ssm_a").reshape(-1), self.W(i, "ssm_dt.bias").reshape(-1))
        o, st.gdn[i] = R.gdn_recurrent(qh, kh, v, decay, beta, st.gdn[i])
        o = R.gated_rmsnorm(o, self.W(i, "ssm_norm.weight").reshape(-1), z, cfg.rms_eps)
        return self.lin(o.reshape(T, Hv * S), self.W(i, "ssm_out.weight"))

    def ffn(self, i: int, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if not cfg.is_moe:
            g = self.lin(x, self.W(i, "ffn_gate.weight"))
            u = self.lin(x, self.W(i, "ffn_up.weight"))
            return self.lin(R.swiglu(g, u, cfg.act), self.W(i, "ffn_down.weight"))
        logits = self.lin(x, self.W(i, "ffn_gate_inp.weight"))
        idx, wts = R.moe_route(logits, cfg.n_experts_used)
        Wg, Wu, Wd = self.W(i, "ffn_gate_exps.weight"), self.W(i, "ffn_up_exps.weight"), self.W(i, "ffn_down_exps.weight")
        out = torch.zeros(x.shape[0], cfg.hidden, dtype=torch.float32, device=x.device)
        for t in range(x.shape[0]):
            for j in range(cfg.n_experts_used):
                e = int(idx[t, j])
                h = R.swiglu(x[t] @ Wg[e].t(), x[t] @ Wu[e].t(), cfg.act)
                out[t] += wts[t, j] * (h @ Wd[e].t())
        if cfg.shared_ffn:
            sg = torch.sigmoid(self.lin(x, self.W(i, "ffn_gate_inp_shexp.weight").reshape(1, -1)))
            h = R.swiglu(self.lin(x, self.W(i, "ffn_gate_shexp.weight")),
                         self.lin(x, self.W(i, "ffn_up_shexp.weight")), cfg.act)
            out = out + sg * self.lin(h, self.W(i, "ffn_down_shexp.weight"))
        return out

    # -- whole model
    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.w["token_embd.weight"][tokens.long()].to(torch.float32) * self.cfg.embed_scale

    def forward_hidden(self, tokens: torch.Tensor, st: RefState) -> torch.Tensor:
        """Run ``tokens`` (1-D ids) after the ``st.pos`` tokens already consumed.  Returns post-norm hidden [T, H]."""
        if self._gemma is not None:
            return self._gemma.forward_hidden(tokens, st)
        cfg = self.cfg
        T = tokens.shape[0]
        pos = torch.arange(st.pos, st.pos + T, device=self.device)
        h = self.embed(tokens.to(self.device))
        for i in range(cfg.n_layers):
            x = R.rmsnorm(h, self.W(i, "attn_norm.weight"), cfg.rms_eps)
            if cfg.is_full_attention_layer(i):
                h = h + self.full_attention(i, x, st, pos)
            else:
                h = h + self.linear_attention(i, x, st)
            x = R.rmsnorm(h, self.W(i, ffn_norm_slot(cfg)), cfg.rms_eps)
            h = h + self.ffn(i, x)
        st.pos += T
        return R.rmsnorm(h, self.w["output_norm.weight"], cfg.rms_eps)

    def logits_from_hidden(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self.w.get("output.weight", self.w["token_embd.weight"])
        lg = hidden.to(self.dtype) @ head.t()
        if self.cfg.final_softcap > 0:
            lg = self.cfg.final_softcap * torch.tanh(lg / self.cfg.final_softcap)
        return lg.to(torch.float32)

    def forward(self, tokens: torch.Tensor, st: Optional[RefState] = None) -> Tuple[torch.Tensor, RefState]:
        st = st or self.new_state()
        hidden = self.forward_hidden(tokens, st)
        return self.logits_from_hidden(hidden), st

    @torch.no_grad()
    def generate(self, prompt: List[int], max_tokens: int) -> Tuple[List[int], torch.Tensor]:
        """Greedy generation.  Returns (generated ids, logits of every generated step [max_tokens, V])."""
        st = self.new_state()
        logits, st = self.forward(torch.tensor(prompt, dtype=torch.long), st)
        out, all_logits = [], []
        cur = logits[-1]
        for _ in range(max_tokens):
            all_logits.append(cur)
            tok = int(torch.argmax(cur))
            out.append(tok)
            lg, st = self.forward(torch.tensor([tok], dtype=torch.long), st)
            cur = lg[-1]
        return out, torch.stack(all_logits)

    # -- NextN (MTP) draft block: hipengine/kernels/cpu_reference/ops.py:840-955 defines the contract
    def nextn_step(self, token: int, hidden_row: torch.Tensor, pos: int, dstate: RefState) -> Tuple[torch.Tensor, torch.Tensor]:
        """One pass of the trailing NextN block.

        input = eh_proj([RMSNorm_e(embed(token)) | RMSNorm_h(hidden_row)]) -> gated-attention block with its own
        KV -> FFN -> shared_head_norm (or output_norm) -> logits.  Returns (logits [V], new hidden row [H]).
        """
        cfg = self.cfg
        i = cfg.n_layers
        emb_table = self.w.get(f"blk.{i}.nextn.embed_tokens.weight", self.w["token_embd.weight"])
        e = R.rmsnorm(emb_table[token].to(torch.float32)[None], self.W(i, "nextn.enorm.weight"), cfg.rms_eps)
        hn = R.rmsnorm(hidden_row[None], self.W(i, "nextn.hnorm.weight"), cfg.rms_eps)
        h = self.lin(torch.cat([e, hn], -1), self.W(i, "nextn.eh_proj.weight")).to(torch.float32)
        x = R.rmsnorm(h, self.W(i, "attn_norm.weight"), cfg.rms_eps)
        p = torch.tensor([pos], device=self.device)
        h = h + self.full_attention(i, x, dstate, p)
        x = R.rmsnorm(h, self.W(i, ffn_norm_slot(cfg)), cfg.rms_eps)
        h = h + self.ffn(i, x)
        norm_w = self.w.get(f"blk.{i}.nextn.shared_head_norm.weight", self.w["output_norm.weight"])
        hid = R.rmsnorm(h, norm_w, cfg.rms_eps)
        head = self.w.get(f"blk.{i}.nextn.shared_head_head.weight",
                          self.w.get("output.weight", self.w["token_embd.weight"]))
        return (hid.to(self.dtype) @ head.t())[0].to(torch.float32), hid[0]
