"""fp32 reference forward of the Gemma 4 MoE decoder (oracle for the GPU executor).

Layer recipe (reference model card ``docs/model-cards/MODEL-GEMMA4.md:157-190``, which follows llama.cpp's
``src/models/gemma4.cpp``; the reference's own oracle is ``hipengine/kernels/cpu_reference/gemma4.py``):
attention with per-head learned Q/K RMSNorm, weightless V RMSNorm, RoPE on Q and K only, scale 1.0, a 1024-token
window on sliding layers, V = K (pre-norm) on layers without ``attn_v``; ``post_attention_norm`` on the attention
output before the residual add; a dense GeGLU branch and a top-k expert branch computed from the same residual
with separate norms, each post-normed, summed, normed again, added to the residual, and the whole scaled by
``layer_output_scale``.  The router reads the residual through a weightless RMSNorm times ``1/sqrt(hidden)`` times
``ffn_gate_inp.scale``; expert outputs are scaled by ``ffn_down_exps.scale[e]``.  Final logits are soft-capped.

RoPE: sliding layers rotate the whole head (base ``swa_rope_theta``); global layers rotate the first
``global_rope_fraction`` of the head with frequencies spaced over the whole head dim ("proportional").
"""
from __future__ import annotations

import torch

from . import ops as R


def rope_partial_proportional(x: torch.Tensor, pos: torch.Tensor, n_rot: int, theta: float, denom: int) -> torch.Tensor:
    """NeoX-style rotation of the first ``n_rot`` dims with inv_freq_i = theta^(-2i/denom).  x [T, H, D]."""
    half = n_rot // 2
    i = torch.arange(half, dtype=torch.float32, device=x.device)
    inv = theta ** (-2.0 * i / denom)
    ang = pos.to(torch.float32)[:, None] * inv[None]
    c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
    a, b = x[..., :half], x[..., half:n_rot]
    return torch.cat([a * c - b * s, a * s + b * c, x[..., n_rot:]], -1)


class Gemma4Ref:
    def __init__(self, model):
        self.m = model
        self.cfg = model.cfg

    def rope_params(self, i: int):
        cfg = self.cfg
        D = cfg.layer_head_dim(i)
        if cfg.is_global_layer(i):
            return int(D * cfg.global_rope_fraction), cfg.rope_theta, D
        return D, cfg.swa_rope_theta, D

    def attention(self, i: int, x: torch.Tensor, st, pos: torch.Tensor) -> torch.Tensor:
        m, cfg = self.m, self.cfg
        T = x.shape[0]
        H, Hkv, D = cfg.n_heads, cfg.layer_kv_heads(i), cfg.layer_head_dim(i)
        q = m.lin(x, m.W(i, "attn_q.weight")).reshape(T, H, D)
        k = m.lin(x, m.W(i, "attn_k.weight")).reshape(T, Hkv, D)
        v = m.lin(x, m.W(i, "attn_v.weight")).reshape(T, Hkv, D) if f"blk.{i}.attn_v.weight" in m.w else k
        q = R.rmsnorm(q, m.W(i, "attn_q_norm.weight"), cfg.rms_eps)
        k_n = R.rmsnorm(k, m.W(i, "attn_k_norm.weight"), cfg.rms_eps)
        v = R.rmsnorm(v, None, cfg.rms_eps)
        n_rot, theta, denom = self.rope_params(i)
        q = rope_partial_proportional(q, pos, n_rot, theta, denom)
        k_n = rope_partial_proportional(k_n, pos, n_rot, theta, denom)
        if m.kv_storage != "fp32":
            k_n, v = R.kv_store_roundtrip(k_n, m.kv_storage), R.kv_store_roundtrip(v, m.kv_storage)
        st.k[i] = k_n if i not in st.k else torch.cat([st.k[i], k_n], 0)
        st.v[i] = v if i not in st.v else torch.cat([st.v[i], v], 0)
        o = R.causal_gqa_attention(q, st.k[i], st.v[i], pos, 1.0, window=cfg.layer_window(i))
        return m.lin(o.reshape(T, H * D), m.W(i, "attn_output.weight"))

    def ffn(self, i: int, h: torch.Tensor) -> torch.Tensor:
        m, cfg = self.m, self.cfg
        eps = cfg.rms_eps
        x1 = R.rmsnorm(h, m.W(i, "ffn_norm.weight"), eps)
        dense = m.lin(R.swiglu(m.lin(x1, m.W(i, "ffn_gate.weight")), m.lin(x1, m.W(i, "ffn_up.weight")), "gelu_tanh"),
                      m.W(i, "ffn_down.weight"))
        dense = R.rmsnorm(dense, m.W(i, "post_ffw_norm_1.weight"), eps)
        r_in = R.rmsnorm(h, None, eps) * (cfg.hidden ** -0.5) * m.W(i, "ffn_gate_inp.scale")
        logits = m.lin(r_in, m.W(i, "ffn_gate_inp.weight"))
        vals, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
        vals, idx = vals[:, :cfg.n_experts_used], idx[:, :cfg.n_experts_used]
        wts = torch.softmax(vals, -1)
        x2 = R.rmsnorm(h, m.W(i, "pre_ffw_norm_2.weight"), eps)
        Wgu, Wd, sc = m.W(i, "ffn_gate_up_exps.weight"), m.W(i, "ffn_down_exps.weight"), m.W(i, "ffn_down_exps.scale")
        F = cfg.expert_ffn
        moe = torch.zeros_like(h)
        for t in range(h.shape[0]):
            for j in range(cfg.n_experts_used):
                e = int(idx[t, j])
                gu = x2[t] @ Wgu[e].t()
                a = R.swiglu(gu[:F], gu[F:], "gelu_tanh")
                moe[t] += wts[t, j] * sc[e] * (a @ Wd[e].t())
        moe = R.rmsnorm(moe, m.W(i, "post_ffw_norm_2.weight"), eps)
        return R.rmsnorm(dense + moe, m.W(i, "post_ffw_norm.weight"), eps)

    def forward_raw(self, tokens: torch.Tensor, st) -> torch.Tensor:
        """Residual rows after the last block, before the output norm (what the assistant head is seeded with)."""
        m, cfg = self.m, self.cfg
        T = tokens.shape[0]
        pos = torch.arange(st.pos, st.pos + T, device=m.device)
        h = m.embed(tokens.to(m.device))
        for i in range(cfg.n_layers):
            x = R.rmsnorm(h, m.W(i, "attn_norm.weight"), cfg.rms_eps)
            a = R.rmsnorm(self.attention(i, x, st, pos), m.W(i, "post_attention_norm.weight"), cfg.rms_eps)
            h = h + a
            h = (h + self.ffn(i, h)) * m.W(i, "layer_output_scale.weight").reshape(())
        st.pos += T
        return h

    def forward_hidden(self, tokens: torch.Tensor, st) -> torch.Tensor:
        return R.rmsnorm(self.forward_raw(tokens, st), self.m.w["output_norm.weight"], self.cfg.rms_eps)


class AssistantRef:
    """fp32 reference of the Gemma 4 assistant (MTP) head: four post-norm blocks with no K/V of their own, each
    attending with scale 1.0 against the backbone's cached K/V of layer ``n - 2`` (sliding blocks) or ``n - 1`` (the
    full-attention block).  One step maps (token, backbone hidden row) to (logits, next hidden row); every step of a
    draft uses the same position (the number of tokens the backbone has processed) and the same keys.
    Specification: the reference's ``docs/reference/GEMMA4-ASSISTANT-MTP.md:82-150`` (forward) and ``:152-200`` (KV
    binding); its implementation is ``hipengine/runtime/gemma4_assistant.py``."""

    def __init__(self, head_weights, backbone_ref: Gemma4Ref):
        self.acfg = head_weights.config
        self.bb = backbone_ref
        self.bcfg = backbone_ref.cfg
        dev = backbone_ref.m.device
        self.w = {n: t.dequant().to(device=dev, dtype=torch.float32) for n, t in head_weights.tensors.items()}

    def step(self, token: int, h_backbone: torch.Tensor, st) -> tuple:
        """``st`` is the backbone's state after it processed ``st.pos`` tokens; ``token`` is the token sampled from
        its last row and ``h_backbone`` [Hb] the raw hidden of that row (or the previous step's second result)."""
        a, b, w = self.acfg, self.bcfg, self.w
        eps = a.rms_eps
        pos = torch.tensor([st.pos], device=h_backbone.device)
        x = self.bb.m.w["token_embd.weight"][int(token)].to(torch.float32) * b.embed_scale     # the BACKBONE's table
        cur = torch.cat([x, h_backbone.to(torch.float32)])[None] @ w["nextn.pre_projection.weight"].t()
        for il in range(a.n_blocks):
            bl = a.backbone_layer(il, b)
            D = b.layer_head_dim(bl)
            p = f"blk.{il}."
            q = (R.rmsnorm(cur, w[p + "attn_norm.weight"], eps) @ w[p + "attn_q.weight"].t()).reshape(1, a.n_heads, D)
            q = R.rmsnorm(q, w[p + "attn_q_norm.weight"], eps)
            n_rot, theta, denom = self.bb.rope_params(bl)
            q = rope_partial_proportional(q, pos, n_rot, theta, denom)
            o = R.causal_gqa_attention(q, st.k[bl], st.v[bl], pos, 1.0, window=b.layer_window(bl))
            attn = o.reshape(1, a.n_heads * D) @ w[p + "attn_output.weight"].t()      # wo BEFORE the post norm
            attn_out = R.rmsnorm(attn, w[p + "post_attention_norm.weight"], eps) + cur
            f_in = R.rmsnorm(attn_out, w[p + "ffn_norm.weight"], eps)
            ffn = R.swiglu(f_in @ w[p + "ffn_gate.weight"].t(), f_in @ w[p + "ffn_up.weight"].t(), "gelu_tanh")
            ffn = R.rmsnorm(ffn @ w[p + "ffn_down.weight"].t(), w[p + "post_ffw_norm.weight"], eps)
            cur = (ffn + attn_out) * w[p + "layer_output_scale.weight"].reshape(())
        cur = R.rmsnorm(cur, w["output_norm.weight"], eps)
        logits = (cur @ w["token_embd.weight"].t())[0]          # the HEAD's table, tied output
        h_next = (cur @ w["nextn.post_projection.weight"].t())[0]
        return logits, h_next

    def draft(self, token: int, h_backbone: torch.Tensor, st, n: int) -> list:
        """Greedy chain of ``n`` proposals after ``token`` (the hidden recurs through the post-projection)."""
        out = []
        h = h_backbone
        for _ in range(n):
            lg, h = self.step(token, h, st)
            token = int(lg.argmax())
            out.append(token)
        return out
