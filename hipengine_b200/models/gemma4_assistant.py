"""Gemma 4 assistant (MTP) head on the GPU: a four-block draft model that owns no K/V.

One step maps (token, backbone hidden row) to (logits, next hidden row) for up to 8 independent requests:

    x   = backbone_token_embd[token] * sqrt(backbone width)              the BACKBONE's embedding table
    cur = pre_projection @ concat(x, h)                                  [head width]
    per block: q = rope(rmsnorm_head(attn_q @ rmsnorm(cur)))             no K/V projections
               a = attention(q, K/V of the backbone's layer n-2 (sliding block) or n-1 (full block), scale 1)
               cur = rmsnorm(attn_output @ a) + cur                      post-norm; wo BEFORE the norm
               cur = (rmsnorm(down(gelu(gate f) * up f)) + cur) * layer_output_scale,  f = rmsnorm(cur)
    cur = rmsnorm(cur, output_norm); logits = head_token_embd @ cur; h_next = post_projection @ cur

Every step of one draft uses the same position p (the number of tokens the backbone has processed: the query sits at
p, the keys are 0 .. p-1) and the same keys, so the head needs no KV allocation, no eviction and no rollback: it reads
the backbone executor's own paged KV of two layers through the same block table.  Head count, KV heads, head width,
window and RoPE of a block are those of the backbone layer it reads, so the backbone's own kernels serve it: the
quantised GEMV with the fused norm prologue, the Q-only form of the norm + RoPE kernel (zero KV heads: nothing is
written), the split-K decode attention, the sandwich-norm add.  No new kernel.

Specification: the reference's ``docs/reference/GEMMA4-ASSISTANT-MTP.md:82-200``; its implementation is
``hipengine/runtime/gemma4_assistant.py`` (``Gemma4AssistantHead``, ``Gemma4MtpDrafter``); the fp32 oracle here is
``ref/gemma4.py::AssistantRef``.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..loading.gemma4 import validate_assistant
from ..loading.weights import ModelWeights
from ..ops import kernels as K
from ..ops.kernels import DeviceWeight, GemvSegment
from ..quant.ggml import GGMLType
from .executor import GEMV_MAX_ROWS, PAGE


class Gemma4AssistantHead:
    def __init__(self, ex, weights: ModelWeights, max_rows: int = GEMV_MAX_ROWS):
        validate_assistant(weights, ex.cfg)
        self.ex, self.acfg, self.bcfg = ex, weights.config, ex.cfg
        self.device = ex.device
        self.max_rows = min(int(max_rows), GEMV_MAX_ROWS)
        self.dw: Dict[str, DeviceWeight] = {}
        self.f32: Dict[str, torch.Tensor] = {}
        for name, t in weights.tensors.items():
            raw = t.raw.to(self.device)
            if t.ggml_type == GGMLType.F32 and len(t.shape) == 1:
                self.f32[name] = raw.view(torch.float32).reshape(t.shape).contiguous()
            elif len(t.shape) == 2:
                self.dw[name] = K.to_device_weight(raw, t.ggml_type, t.n_rows, t.n_cols)
        a, b, dev = self.acfg, self.bcfg, self.device
        R, Ha, Hb = self.max_rows, a.hidden, a.backbone_hidden
        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
        bf16 = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        # persistent buffers (a captured graph may hold them)
        self.e, self.xh, self.cur = f32(R, Hb), f32(R, 2 * Hb), f32(R, Ha)
        self.y, self.d, self.act = f32(R, Ha), f32(R, Ha), bf16(R, a.ffn)
        self.logits, self.h_next = f32(R, a.vocab), f32(R, Hb)
        self.layers = [a.backbone_layer(il, b) for il in range(a.n_blocks)]
        self.qf: Dict[int, torch.Tensor] = {}
        self.q_out: Dict[int, torch.Tensor] = {}
        self.attn: Dict[int, torch.Tensor] = {}
        for bl in set(self.layers):
            D = b.layer_head_dim(bl)
            self.qf[bl], self.q_out[bl] = f32(R, a.n_heads * D), bf16(R, a.n_heads, D)
            self.attn[bl] = bf16(R, a.n_heads * D)
        self._part = None

    def nbytes(self) -> int:
        return sum(w.data.numel() * w.data.element_size() for w in self.dw.values())

    def W(self, il: int, slot: str) -> DeviceWeight:
        return self.dw[f"blk.{il}.{slot}.weight"]

    def F(self, il: int, slot: str) -> torch.Tensor:
        return self.f32[f"blk.{il}.{slot}.weight"]

    @torch.no_grad()
    def forward_batch(self, tokens: torch.Tensor, h_in: torch.Tensor, slot: torch.Tensor, n_past: torch.Tensor,
                      max_ctx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """One head step for R independent requests.

        ``tokens`` int64 [R]: the token each request just sampled (not yet fed to the backbone); ``h_in`` fp32
        [R, backbone width]: the raw hidden (before the output norm) of the backbone row that produced it, or the
        previous step's second result; ``slot`` int32 [R]: the requests' block-table rows; ``n_past`` int32 [R]: how
        many tokens the backbone has cached for each (query position = key count); ``max_ctx`` a host bound on
        them.  Returns (logits fp32 [R, vocab], next hidden fp32 [R, backbone width]) in buffers of the head that
        the next call overwrites (passing the second result back in as ``h_in`` is fine)."""
        ex, a, b = self.ex, self.acfg, self.bcfg
        R, Hb, eps = tokens.shape[0], a.backbone_hidden, a.rms_eps
        assert 1 <= R <= self.max_rows
        H = a.n_heads
        xh, cur = self.xh[:R], self.cur[:R]
        K.embed(ex.dw["token_embd.weight"], tokens, self.e[:R], b.embed_scale)
        xh[:, Hb:].copy_(h_in)                       # before anything of this step is written (h_in may be h_next)
        xh[:, :Hb].copy_(self.e[:R])
        K.gemv(xh, [GemvSegment(self.dw["nextn.pre_projection.weight"], cur)])
        for il, bl in enumerate(self.layers):
            Hkv, D, window = b.layer_kv_heads(bl), b.layer_head_dim(bl), b.layer_window(bl)
            qf, q_out, attn = self.qf[bl][:R], self.q_out[bl][:R], self.attn[bl][:R]
            K.gemv(cur, [GemvSegment(self.W(il, "attn_q"), qf)], norm_w=self.F(il, "attn_norm"), eps=eps)
            n_rot, theta, denom = ex._rope(bl)
            # zero KV heads: the kernel's grid covers the query heads only, so nothing is written to the cache
            K.qkv_post(qf, qf, qf, self.F(il, "attn_q_norm"), None, q_out, None, ex.kv[bl], ex.block_table, slot,
                       n_past, H, 0, D, PAGE, False, n_rot, theta, eps, rope_denom=denom)
            # the query at position p sees keys k <= p (all n_past of them) and, in a sliding block, k > p - window:
            # the last window - 1 keys
            win = window - 1 if window > 0 else 0
            span = min(max_ctx, win) if win > 0 else max_ctx
            split_len, max_splits = K.attn_decode_split(max(span, 1), R, Hkv)
            max_splits += 1 if win > 0 else 0
            need = K.attn_decode_scratch_floats(R, H, max_splits, D)
            if self._part is None or self._part.numel() < need:
                self._part = torch.empty(need, dtype=torch.float32, device=self.device)
            K.attn_decode(q_out, None, ex.kv[bl], ex.block_table, slot, n_past, self._part, attn, H, Hkv, D, PAGE,
                          split_len, max_splits, 1.0, window=win)
            y = self.y[:R]
            K.gemv(attn, [GemvSegment(self.W(il, "attn_output"), y)])
            K.norm_add(cur, y, self.F(il, "post_attention_norm"), eps)
            act, d = self.act[:R], self.d[:R]
            K.gemv(cur, [GemvSegment(self.W(il, "ffn_gate"), act, K.EPI_GELU_MUL, self.W(il, "ffn_up"))],
                   norm_w=self.F(il, "ffn_norm"), eps=eps)
            K.gemv(act, [GemvSegment(self.W(il, "ffn_down"), d)])
            K.norm_add(cur, d, self.F(il, "post_ffw_norm"), eps)
            cur.mul_(self.F(il, "layer_output_scale"))
        logits, h_next = self.logits[:R], self.h_next[:R]
        K.gemv(cur, [GemvSegment(self.dw["token_embd.weight"], logits),
                     GemvSegment(self.dw["nextn.post_projection.weight"], h_next)],
               norm_w=self.f32["output_norm.weight"], eps=eps)
        return logits, h_next
