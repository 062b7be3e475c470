"""Mixture-of-experts FFN block of the hybrid executor (Qwen3.5-MoE: 256 experts, top-8, shared expert).

Two routes, chosen by the number of packed rows:

* ``T <= SEL_MAX_ROWS`` (decode, verify chains, short prefill chunks): *selected-expert GEMV*.  The router
  GEMV writes logits, ``he_moe_route`` picks the experts on the device, and two kernels walk the
  (token, expert) pairs reading the experts' quantised rows in place.  No expert id is ever read by the host,
  so the whole block is CUDA-graph capturable.
* larger ``T``: *grouped tensor-core GEMM*.  Pairs are bucketed by expert (128-row padded segments), rows are
  gathered and the tcgen05 GEMM runs in grouped mode over the experts' quantised blocks (each 128-row tile
  carries its expert id; the blocks are expanded to bf16 inside the GEMM pipeline), followed by a combine kernel that applies the routing weights, the
  sigmoid-gated shared expert and the residual add.

Behaviour follows the reference MoE layer executor (``hipengine/runtime/qwen35_gguf_layer_ffn.py:719-1278``)
and its oracle (``hipengine/kernels/cpu_reference/ops.py:575-700``): softmax over all experts, stable top-k,
renormalise by ``max(sum, 6.1e-5)``, shared expert scaled by ``sigmoid(x . w_shexp_gate)``.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.kernels import GemvSegment
from ..quant.ggml import GGMLType

SEL_MAX_ROWS = 64


class _MoeLayer:
    """Per-layer derived weights: router as a GEMV weight and as bf16 hi/lo halves for the tensor-core path."""

    def __init__(self, ex, i: int):
        cfg = ex.cfg
        E = cfg.n_experts
        self.router = ex.W(i, "ffn_gate_inp.weight")
        router_f32 = ex.f32[f"blk.{i}.ffn_gate_inp.weight"]
        self.has_shared = cfg.shared_ffn > 0
        rows = [router_f32]
        self.shexp_gate = None
        if self.has_shared:
            g = ex.f32[f"blk.{i}.ffn_gate_inp_shexp.weight"].reshape(1, -1).contiguous()
            self.shexp_gate = K.to_device_weight(g.view(torch.uint8).reshape(1, -1), GGMLType.F32, 1, cfg.hidden)
            rows.append(g)
        full = torch.cat(rows, 0)
        pad = (-full.shape[0]) % 8
        if pad:
            full = torch.cat([full, torch.zeros(pad, full.shape[1], device=full.device)], 0)
        # fp32 router weights as two bf16 GEMM operands: hi + lo reproduces ~16 mantissa bits
        self.r_hi = full.to(torch.bfloat16).contiguous()
        self.r_lo = (full - self.r_hi.float()).to(torch.bfloat16).contiguous()
        self.n_logits = E + (1 if self.has_shared else 0)
        self.n_logits_pad = full.shape[0]


def _layer(ex, i: int) -> _MoeLayer:
    cache: Dict[int, _MoeLayer] = ex.__dict__.setdefault("_moe_layers", {})
    if i not in cache:
        cache[i] = _MoeLayer(ex, i)
    return cache[i]


def moe_ffn(ex, i: int, h: torch.Tensor, T: int, norm_w: torch.Tensor, small: bool) -> None:
    """h[T, hidden] (fp32 residual) += MoE(RMSNorm(h)) for layer ``i`` of executor ``ex``.

    Expert parallelism: an executor that owns only experts ``ex.expert_range = (lo, hi)`` (weights already sliced)
    computes the contributions of its own experts for every token -- the activations are replicated across ranks
    -- into a zeroed partial buffer that ``ex._moe_reduce`` sums over the ranks and adds to the residual.  The
    shared expert runs on the one rank with ``ex.owns_shared_expert``.
    """
    rng = getattr(ex, "expert_range", None)
    target = h
    if rng is not None:
        target = ex.scratch.get("moe_partial", (T, h.shape[1]), torch.float32)
        target.zero_()
    if T <= SEL_MAX_ROWS:
        _moe_selected(ex, i, h, target, T, norm_w, rng)
    else:
        _moe_grouped(ex, i, h, target, T, norm_w, rng)
    if rng is not None:
        ex._moe_reduce(h, target)


def _moe_selected(ex, i: int, h: torch.Tensor, target: torch.Tensor, T: int, norm_w: torch.Tensor, rng) -> None:
    cfg, sc = ex.cfg, ex.scratch
    L = _layer(ex, i)
    er = rng or (0, 0)
    shared_here = L.has_shared and getattr(ex, "owns_shared_expert", True)
    E, k, F = cfg.n_experts, cfg.n_experts_used, cfg.expert_ffn
    logits = sc.get("moe_logits", (T, L.n_logits_pad), torch.float32)
    ids = sc.get("moe_ids", (T, k), torch.int32)
    wts = sc.get("moe_wts", (T, k), torch.float32)
    act_rows = sc.get("moe_act", (T * k, F), torch.bfloat16)
    act_sh = sc.get("moe_act_sh", (T, max(cfg.shared_ffn, 1)), torch.bfloat16) if L.has_shared else None
    epi = K.EPI_SILU_MUL if cfg.act == "silu" else K.EPI_GELU_MUL
    # everything that reads the residual stream runs before anything that adds to it
    for r0 in range(0, T, 8):
        r1 = min(T, r0 + 8)
        segs = [GemvSegment(L.router, logits[r0:r1, :E])]
        if L.has_shared:
            segs.append(GemvSegment(L.shexp_gate, logits[r0:r1, E:E + 1]))
        K.gemv(h[r0:r1], segs, norm_w=norm_w, eps=cfg.rms_eps)
        if shared_here:
            K.gemv(h[r0:r1], [GemvSegment(ex.W(i, "ffn_gate_shexp.weight"), act_sh[r0:r1], epi,
                                          ex.W(i, "ffn_up_shexp.weight"))], norm_w=norm_w, eps=cfg.rms_eps)
    K.moe_route(logits, k, ids, wts, n_experts=E)
    K.moe_gateup_sel(h, norm_w, cfg.rms_eps, ids, wts, ex.W(i, "ffn_gate_exps.weight"),
                     ex.W(i, "ffn_up_exps.weight"), F, act_rows, cfg.act, expert_range=er)
    K.moe_down_sel(act_rows, ids, wts, ex.W(i, "ffn_down_exps.weight"), cfg.hidden, target, expert_range=er)
    if shared_here:
        K.moe_scale_rows(act_sh, logits[:, E:E + 1])
        for r0 in range(0, T, 8):
            r1 = min(T, r0 + 8)
            K.gemv(act_sh[r0:r1], [GemvSegment(ex.W(i, "ffn_down_shexp.weight"), target[r0:r1], K.EPI_ADD_F32)])


def _grouped(sc, a_sorted: torch.Tensor, w, out: torch.Tensor, n_groups: int, tile_group: torch.Tensor) -> None:
    """Grouped expert GEMM: quantised experts in place; float-typed experts through a bf16 scratch expansion."""
    from ..ops import gemm as GM
    if GM.quant_gemm_ok(w):
        GM.gemm_quant_grouped(a_sorted, w, out, n_groups, tile_group)
        return
    wb = sc.get("moe_deq", (w.n_rows, w.n_cols), torch.bfloat16)
    K.dequant_bf16(w, wb)
    GM.gemm_bf16_grouped(a_sorted, wb[:, :a_sorted.shape[1]], out, n_groups, tile_group)


def _moe_grouped(ex, i: int, h: torch.Tensor, target: torch.Tensor, T: int, norm_w: torch.Tensor, rng) -> None:
    from ..ops import gemm as GM
    cfg, sc = ex.cfg, ex.scratch
    L = _layer(ex, i)
    E, k, F, H = cfg.n_experts, cfg.n_experts_used, cfg.expert_ffn, cfg.hidden
    e_lo, e_hi = rng or (0, E)
    El = e_hi - e_lo                      # local experts (all of them without expert parallelism)
    shared_here = L.has_shared and getattr(ex, "owns_shared_expert", True)
    xn = ex._norm_rows(h, norm_w)       # sequence-parallel executors gather the rows of all ranks here
    ex._xn_ready()
    logits = sc.get("moe_logits", (T, L.n_logits_pad), torch.float32)
    GM.gemm_bf16(xn, L.r_hi, logits, epi=1)
    GM.gemm_bf16(xn, L.r_lo, logits, epi=2)
    ids = sc.get("moe_ids", (T, k), torch.int32)
    wts = sc.get("moe_wts", (T, k), torch.float32)
    K.moe_route(logits, k, ids, wts, n_experts=E)
    P = T * k
    bound = K.moe_sorted_rows_bound(P, El)
    pos = sc.get("moe_pos", (P,), torch.int32)
    tile_group = sc.get("moe_tiles", (bound // 128,), torch.int32)
    meta = sc.get("moe_meta", (4,), torch.int32)
    K.moe_group(ids, El, pos, tile_group, meta, expert_lo=e_lo)
    xs = sc.get("moe_xs", (bound, H), torch.bfloat16)
    K.moe_gather(xn, pos, k, xs)
    gu = sc.get("moe_gu", (bound, 2 * F), torch.bfloat16)
    wg, wu, wd = (ex.W(i, "ffn_gate_exps.weight"), ex.W(i, "ffn_up_exps.weight"), ex.W(i, "ffn_down_exps.weight"))
    # the experts' quantised blocks are read in place by the grouped tensor-core GEMM (no bf16 expansion)
    _grouped(sc, xs, wg, gu[:, :F], El, tile_group)
    _grouped(sc, xs, wu, gu[:, F:], El, tile_group)
    act = sc.get("moe_act_g", (bound, F), torch.bfloat16)
    K.act_mul(gu, act, cfg.act)
    ys = sc.get("moe_ys", (bound, H), torch.bfloat16)
    _grouped(sc, act, wd, ys, El, tile_group)
    ysh = None
    if shared_here:
        Fs = cfg.shared_ffn
        gus = sc.get("moe_gus", (T, 2 * Fs), torch.bfloat16)
        ex._gemm(xn, ex.W(i, "ffn_gate_shexp.weight"), gus[:, :Fs], tag="g")
        ex._gemm(xn, ex.W(i, "ffn_up_shexp.weight"), gus[:, Fs:], tag="g")
        acts = sc.get("moe_acts", (T, Fs), torch.bfloat16)
        K.act_mul(gus, acts, cfg.act)
        ysh = ex._gemm(acts, ex.W(i, "ffn_down_shexp.weight"), sc.get("y_bf", (T, H), torch.bfloat16), tag="d")
    K.moe_combine(target, ys, pos, wts, k, ysh, logits[:, E:E + 1] if shared_here else None)
