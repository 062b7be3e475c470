"""Gemma 4 MoE executor (sliding-window + global attention, dense GeGLU branch in parallel with top-k experts).

Reuses the hybrid executor's weight store, scratch, GEMM/GEMV dispatch, output head and decode-graph plumbing and
replaces the layer walk.  Differences from the Qwen path that matter for kernels:
  * per-layer KV geometry (sliding: ``n_kv_heads`` x ``head_dim`` with a window; global: fewer, wider heads, V = K
    when the layer has no ``attn_v``), attention scale 1.0, weightless RMSNorm on V, RoPE with per-layer span and
    frequency spacing -- all arguments of the existing ``qkv_post`` / attention kernels;
  * sandwich norms: branch outputs are RMS-normed before they join the residual (``norm_add``, ``ffn_combine``);
  * experts stored as one fused gate|up tensor per layer and a down tensor whose K (704) is not a multiple of the
    256-element quant super-block: the Q8_0 rows are zero-padded to the next multiple at load, which changes no
    result (zero weights, zero scales) and lets the block kernels run unchanged;
  * router input = weightless RMSNorm(residual) / sqrt(hidden) * ``ffn_gate_inp.scale``, expressed as the norm
    weight of the router GEMV; expert outputs scaled by ``ffn_down_exps.scale[e]``, folded into the routing weight.
Layer recipe: the reference's model card ``docs/model-cards/MODEL-GEMMA4.md:157-190`` and runtime
``hipengine/runtime/gemma4.py`` (``Gemma4Runner``); oracle ``ref/gemma4.py``.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..loading.weights import ModelWeights, QTensor
from ..ops import kernels as K
from ..ops.kernels import GemvSegment
from ..quant.ggml import GGMLType
from .executor import GEMV_MAX_ROWS, PAGE, BatchDesc, HybridExecutor
from .moe import SEL_MAX_ROWS


def _pad_q8_0_cols(t: QTensor, k_pad: int) -> QTensor:
    """Append zero Q8_0 blocks (scale 0, values 0) so that the row length becomes ``k_pad``."""
    assert t.ggml_type == GGMLType.Q8_0 and k_pad % 32 == 0
    rows = t.n_rows
    raw = t.raw.reshape(rows, -1)
    extra = (k_pad - t.n_cols) // 32 * 34
    pad = torch.zeros(rows, extra, dtype=torch.uint8, device=raw.device)
    return QTensor(t.name, t.ggml_type, tuple(t.shape[:-1]) + (k_pad,), torch.cat([raw, pad], 1).contiguous())


class Gemma4Executor(HybridExecutor):
    def __init__(self, weights: ModelWeights, **kw):
        cfg = weights.config
        self.expert_k = cfg.expert_ffn
        self.expert_k_pad = (cfg.expert_ffn + 255) // 256 * 256
        tensors = dict(weights.tensors)
        for name, t in list(tensors.items()):
            if name.endswith(("ffn_down_exps.weight", "ffn_down.weight")) and t.n_cols % 256 != 0:
                if t.ggml_type != GGMLType.Q8_0:
                    raise ValueError(f"{name}: K={t.n_cols} needs a 32-element block type (Q8_0), got {t.ggml_type}")
                tensors[name] = _pad_q8_0_cols(t, (t.n_cols + 255) // 256 * 256)
        super().__init__(ModelWeights(cfg, tensors, weights.metadata), **kw)
        H = cfg.hidden
        self.router_norm: Dict[int, torch.Tensor] = {}
        self.router_hi: Dict[int, torch.Tensor] = {}
        self.router_lo: Dict[int, torch.Tensor] = {}
        for i in range(cfg.n_layers):
            self.router_norm[i] = (self.F(i, "ffn_gate_inp.scale") * (H ** -0.5)).contiguous()
            r = self.F(i, "ffn_gate_inp.weight")
            pad = (-r.shape[0]) % 8
            if pad:
                r = torch.cat([r, torch.zeros(pad, H, device=r.device)], 0)
            self.router_hi[i] = r.to(torch.bfloat16).contiguous()
            self.router_lo[i] = (r - self.router_hi[i].float()).to(torch.bfloat16).contiguous()
        self._act_pad: Optional[torch.Tensor] = None
        self.ffn_k_pad = (cfg.ffn + 255) // 256 * 256
        # dense-branch activations live in a zero-padded buffer when the FFN width is not a block multiple
        self._dense_act = torch.zeros(GEMV_MAX_ROWS, self.ffn_k_pad, dtype=torch.bfloat16, device=self.device)

    # ------------------------------------------------------------------ state: per-layer KV geometry
    def _alloc_state(self) -> None:
        cfg, dev = self.cfg, self.device
        self.kv = {}
        self.conv_state, self.gdn_state = {}, {}
        for i in range(cfg.n_layers):
            self.kv[i] = torch.zeros(self.n_pages, 2, cfg.layer_kv_heads(i), PAGE, cfg.layer_head_dim(i),
                                     dtype=torch.bfloat16, device=dev)
        mp = self.max_pages_per_slot
        bt = torch.arange(self.max_slots * mp, dtype=torch.int32).reshape(self.max_slots, mp) + 1
        if self.n_pages < self.max_slots * mp + 1:
            bt = bt.clamp(max=self.n_pages - 1)
        self.block_table = bt.to(dev)
        self.am_v = torch.empty(GEMV_MAX_ROWS * 64 * 64, dtype=torch.float32, device=dev)
        self.am_i = torch.empty(GEMV_MAX_ROWS * 64 * 64, dtype=torch.int32, device=dev)

    def _rope(self, i: int):
        cfg = self.cfg
        D = cfg.layer_head_dim(i)
        if cfg.is_global_layer(i):
            return int(D * cfg.global_rope_fraction), cfg.rope_theta, D
        return D, cfg.swa_rope_theta, D

    # ------------------------------------------------------------------ attention
    def _attention(self, i: int, h: torch.Tensor, b: BatchDesc, small: bool) -> None:
        cfg, sc = self.cfg, self.scratch
        T, H = b.T, cfg.n_heads
        Hkv, D = cfg.layer_kv_heads(i), cfg.layer_head_dim(i)
        has_v = f"blk.{i}.attn_v.weight" in self.dw
        if small:
            qf = sc.get("q_f32", (T, H * D), torch.float32)
            kf = sc.get("k_f32", (T, Hkv * D), torch.float32)
            segs = [GemvSegment(self.W(i, "attn_q.weight"), qf), GemvSegment(self.W(i, "attn_k.weight"), kf)]
            vf = kf
            if has_v:
                vf = sc.get("v_f32", (T, Hkv * D), torch.float32)
                segs.append(GemvSegment(self.W(i, "attn_v.weight"), vf))
            K.gemv(h, segs, norm_w=self.F(i, "attn_norm.weight"), eps=cfg.rms_eps)
        else:
            xn = sc.get("xn", (T, cfg.hidden), torch.bfloat16)
            K.rmsnorm_rows(h, self.F(i, "attn_norm.weight"), xn, cfg.rms_eps)
            qf = self._gemm(xn, self.W(i, "attn_q.weight"), sc.get("q_bf", (T, H * D), torch.bfloat16), tag="q")
            kf = self._gemm(xn, self.W(i, "attn_k.weight"), sc.get("k_bf", (T, Hkv * D), torch.bfloat16), tag="k")
            vf = kf
            if has_v:
                vf = self._gemm(xn, self.W(i, "attn_v.weight"), sc.get("v_bf", (T, Hkv * D), torch.bfloat16), tag="k")
        q_out = sc.get("q_out", (T, H, D), torch.bfloat16)
        n_rot, theta, denom = self._rope(i)
        K.qkv_post(qf, kf, vf, self.F(i, "attn_q_norm.weight"), self.F(i, "attn_k_norm.weight"), q_out, None,
                   self.kv[i], self.block_table, b.slot, b.pos, H, Hkv, D, PAGE, False, n_rot, theta, cfg.rms_eps,
                   v_norm=True, rope_denom=denom)
        attn = sc.get("attn_out", (T, H * D), torch.bfloat16)
        self._attend_layer(i, q_out, b, attn, H, Hkv, D, cfg.layer_window(i))
        if small:
            y = sc.get("y_f32", (T, cfg.hidden), torch.float32)
            K.gemv(attn, [GemvSegment(self.W(i, "attn_output.weight"), y, K.EPI_F32)])
        else:
            y = self._gemm(attn, self.W(i, "attn_output.weight"), sc.get("y_bf", (T, cfg.hidden), torch.bfloat16),
                           tag="o")
        K.norm_add(h, y, self.F(i, "post_attention_norm.weight"), cfg.rms_eps)

    def _attend_layer(self, i, q_out, b: BatchDesc, out, H, Hkv, D, window) -> None:
        T = b.T
        if T > GEMV_MAX_ROWS and b.segs_host is not None and os.environ.get("HE_PREFILL_ATTN", "flash") == "flash":
            from ..ops import attention as A
            if A.flash_prefill_available(D):
                r0 = 0
                for (slot, pos0, n) in b.segs_host:
                    A.flash_prefill(q_out[r0:r0 + n], None, self.kv[i], self.block_table, slot, pos0, out[r0:r0 + n],
                                    H, Hkv, D, PAGE, 1.0, window=window)
                    r0 += n
                return
        span = min(b.max_ctx, window) if window > 0 else b.max_ctx
        split_len, max_splits = K.attn_decode_split(span, T, Hkv)
        max_splits += 1 if window > 0 else 0
        part = self.scratch.get("attn_part", (K.attn_decode_scratch_floats(T, H, max_splits, D),), torch.float32)
        K.attn_decode(q_out, None, self.kv[i], self.block_table, b.slot, b.ctx_len, part, out, H, Hkv, D, PAGE,
                      split_len, max_splits, 1.0, window=window)

    # ------------------------------------------------------------------ FFN: dense branch || experts
    def _ffn_layer(self, i: int, h: torch.Tensor, b: BatchDesc, small: bool) -> None:
        from ..ops import gemm as GM
        cfg, sc = self.cfg, self.scratch
        T, H, Fd = b.T, cfg.hidden, cfg.ffn
        E, k, F, Fp = cfg.n_experts, cfg.n_experts_used, cfg.expert_ffn, self.expert_k_pad
        eps = cfg.rms_eps
        logits = sc.get("moe_logits", (T, self.router_hi[i].shape[0]), torch.float32)
        ids = sc.get("moe_ids", (T, k), torch.int32)
        wts = sc.get("moe_wts", (T, k), torch.float32)
        eo = sc.get("moe_eo", (T, H), torch.float32)
        eo.zero_()
        # ---- dense branch + router logits
        if small:
            act = self._dense_act[:T]
            K.gemv(h, [GemvSegment(self.W(i, "ffn_gate.weight"), act[:, :Fd], K.EPI_GELU_MUL,
                                   self.W(i, "ffn_up.weight"))], norm_w=self.F(i, "ffn_norm.weight"), eps=eps)
            d = sc.get("ffn_d", (T, H), torch.float32)
            K.gemv(act, [GemvSegment(self.W(i, "ffn_down.weight"), d, K.EPI_F32)])
            K.gemv(h, [GemvSegment(self.W(i, "ffn_gate_inp.weight"), logits[:, :E])], norm_w=self.router_norm[i],
                   eps=eps)
        else:
            xn = sc.get("xn", (T, H), torch.bfloat16)
            K.rmsnorm_rows(h, self.F(i, "ffn_norm.weight"), xn, eps)
            gu = sc.get("ffn_gu", (T, 2 * Fd), torch.bfloat16)
            self._gemm(xn, self.W(i, "ffn_gate.weight"), gu[:, :Fd], tag="g")
            self._gemm(xn, self.W(i, "ffn_up.weight"), gu[:, Fd:], tag="g")
            act = sc.get("ffn_act", (T, Fd), torch.bfloat16)
            K.act_mul(gu, act, "gelu_tanh")
            # the down weight's K is zero-padded to whole blocks; the GEMM reads the missing activation columns as 0
            d = GM.gemm_quant(act, self.W(i, "ffn_down.weight"), sc.get("ffn_d_bf", (T, H), torch.bfloat16), sc)
            xr = sc.get("xn_router", (T, H), torch.bfloat16)
            K.rmsnorm_rows(h, self.router_norm[i], xr, eps)
            GM.gemm_bf16(xr, self.router_hi[i], logits, epi=1)
            GM.gemm_bf16(xr, self.router_lo[i], logits, epi=2)
        K.moe_route(logits, k, ids, wts, n_experts=E, mode=1, expert_scale=self.F(i, "ffn_down_exps.scale"))
        wgu, wd = self.W(i, "ffn_gate_up_exps.weight"), self.W(i, "ffn_down_exps.weight")
        norm2 = self.F(i, "pre_ffw_norm_2.weight")
        if T <= SEL_MAX_ROWS:
            if self._act_pad is None:
                # sized once for the largest selected-expert batch: a buffer a captured graph may hold is never freed
                self._act_pad = torch.zeros(SEL_MAX_ROWS * k, Fp, dtype=torch.bfloat16, device=self.device)
            act_rows = self._act_pad[:T * k]
            K.moe_gateup_sel(h, norm2, eps, ids, wts, wgu, None, F, act_rows, "gelu_tanh", fused_gate_up=True)
            K.moe_down_sel(act_rows, ids, wts, wd, H, eo)
        else:
            x2 = sc.get("xn2", (T, H), torch.bfloat16)
            K.rmsnorm_rows(h, norm2, x2, eps)
            P = T * k
            bound = K.moe_sorted_rows_bound(P, E)
            pos = sc.get("moe_pos", (P,), torch.int32)
            tiles = sc.get("moe_tiles", (bound // 128,), torch.int32)
            meta = sc.get("moe_meta", (4,), torch.int32)
            K.moe_group(ids, E, pos, tiles, meta)
            xs = sc.get("moe_xs", (bound, H), torch.bfloat16)
            K.moe_gather(x2, pos, k, xs)
            from .moe import _grouped
            gus = sc.get("moe_gu", (bound, 2 * F), torch.bfloat16)
            _grouped(sc, xs, wgu, gus, E, tiles)
            acts = sc.get("moe_act_g", (bound, F), torch.bfloat16)
            K.act_mul(gus, acts, "gelu_tanh")
            ys = sc.get("moe_ys", (bound, H), torch.bfloat16)
            _grouped(sc, acts, wd, ys, E, tiles)
            K.moe_combine(eo, ys, pos, wts, k)
        K.ffn_combine(h, d, eo, self.F(i, "post_ffw_norm_1.weight"), self.F(i, "post_ffw_norm_2.weight"),
                      self.F(i, "post_ffw_norm.weight"), self.F(i, "layer_output_scale.weight"), eps)

    # ------------------------------------------------------------------ whole model
    def forward(self, b: BatchDesc, journal: Optional[dict] = None, h_out: Optional[torch.Tensor] = None,
                defer_resid: bool = False) -> torch.Tensor:
        cfg = self.cfg
        T = b.T
        small = T <= self.small_rows
        h = h_out if h_out is not None else self.scratch.get("h", (T, cfg.hidden), torch.float32)
        K.embed(self.dw["token_embd.weight"], b.tokens, h, cfg.embed_scale)
        for i in range(cfg.n_layers):
            self._attention(i, h, b, small)
            self._ffn_layer(i, h, b, small)
        return h
