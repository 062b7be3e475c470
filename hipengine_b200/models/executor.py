"""GPU executor for the Qwen3.5-family hybrid decoders and plain dense decoders.

One object owns the device-resident weights (in kernel layouts), the paged KV
pool tensors, the per-slot recurrent state (conv window + Gated-DeltaNet state)
and all scratch.  ``forward`` runs a packed batch of rows that may mix requests
("segments"): decode rows, speculative verify chains and prefill chunks all go
through the same call, differing only in how many rows a segment has.

Kernel sequence per layer follows the reference executors
(``hipengine/runtime/qwen35_gguf_layer_attn.py:474-1147`` for linear / full
attention, ``hipengine/runtime/qwen35_gguf_layer_ffn.py:301-1278`` for dense and
MoE FFN) but the fusion boundaries are chosen for B200: for <= 8 rows each
projection is a single fused [RMSNorm + int8 quantize + dp4a GEMV + epilogue]
launch; above that the projections run on the tcgen05 GEMM.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..loading.weights import ModelWeights, QTensor, ffn_norm_slot
from ..ops import kernels as K
from ..ops.kernels import DeviceWeight, GemvSegment
from ..quant.ggml import GGMLType
from .config import ModelConfig

PAGE = 16
GEMV_MAX_ROWS = 8


@dataclass
class BatchDesc:
    """Device-side description of one packed forward batch of T rows in n_seg segments."""
    tokens: torch.Tensor      # [T] int64
    slot: torch.Tensor        # [T] int32   state/block-table slot of each row
    pos: torch.Tensor         # [T] int32   absolute position of each row
    ctx_len: torch.Tensor     # [T] int32   keys visible to the row (pos + 1)
    seg_start: torch.Tensor   # [n_seg + 1] int32
    seg_slot: torch.Tensor    # [n_seg] int32
    tok_seg: torch.Tensor     # [T] int32
    T: int
    n_seg: int
    max_ctx: int              # host upper bound of ctx_len (sizes the split-K grid)
    segs_host: Optional[List[Tuple[int, int, int]]] = None   # (slot, start_pos, n_rows) per segment, when known


def make_batch(segments: Sequence[Tuple[int, int, Sequence[int]]], device) -> BatchDesc:
    """segments: (slot, start_pos, token_ids) per request.  Builds the packed descriptor (one H2D copy each)."""
    toks: List[int] = []
    slot: List[int] = []
    pos: List[int] = []
    seg_start = [0]
    seg_slot: List[int] = []
    tok_seg: List[int] = []
    max_ctx = 1
    for si, (s, p0, ids) in enumerate(segments):
        n = len(ids)
        toks += list(ids)
        slot += [s] * n
        pos += list(range(p0, p0 + n))
        tok_seg += [si] * n
        seg_start.append(seg_start[-1] + n)
        seg_slot.append(s)
        max_ctx = max(max_ctx, p0 + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    pos_t = i32(pos)
    return BatchDesc(torch.tensor(toks, dtype=torch.int64, device=device), i32(slot), pos_t, pos_t + 1,
                     i32(seg_start), i32(seg_slot), i32(tok_seg), len(toks), len(segments), max_ctx,
                     [(s, p0, len(ids)) for (s, p0, ids) in segments])


class _Scratch:
    """Grow-only named scratch tensors (no allocation on the steady-state path).

    A buffer that has been handed out may be baked into a captured CUDA graph, so it must stay mapped for the
    life of the executor: when a name outgrows its buffer the old tensor is *retired* (kept referenced), never
    freed.  (Freed blocks go back to the caching allocator, which unmaps its cache at the next graph capture; an
    older graph replaying into such a block is an illegal access.)  Capacity at least doubles on growth, which
    bounds the retired bytes by the live bytes.
    """

    CANARY_BYTES = 256
    CANARY_BYTE = 0xA5

    def __init__(self, device, canaries: Optional[bool] = None):
        self.device = device
        self.bufs: Dict[str, torch.Tensor] = {}
        self.retired: List[torch.Tensor] = []
        # canary words behind every buffer (HE_SCRATCH_CANARY=1 or canaries=True): a kernel that writes past the
        # extent it was given lands in them, and check_canaries() names the buffer -- the host-side check that stands
        # in for a memory checker on the scratch arena
        self.canaries = (os.environ.get("HE_SCRATCH_CANARY", "0") == "1") if canaries is None else canaries
        self._raw: Dict[str, torch.Tensor] = {}

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        cur = self.bufs.get(name)
        if cur is None or cur.numel() < n or cur.dtype != dtype:
            if cur is not None:
                self.retired.append(self._raw.get(name, cur))
                if cur.dtype == dtype:
                    n_alloc = max(n, 2 * cur.numel())
                else:
                    n_alloc = n
            else:
                n_alloc = n
            n_alloc = max(n_alloc, 1)
            if self.canaries:
                esz = torch.empty(0, dtype=dtype).element_size()
                pad = -(-self.CANARY_BYTES // esz)
                raw = torch.empty(n_alloc + pad, dtype=dtype, device=self.device)
                raw[n_alloc:].view(torch.uint8).fill_(self.CANARY_BYTE)
                self._raw[name] = raw
                cur = raw[:n_alloc]
            else:
                cur = torch.empty(n_alloc, dtype=dtype, device=self.device)
            self.bufs[name] = cur
        return cur[:n].view(*shape)

    def check_canaries(self) -> List[str]:
        """Names of the buffers whose trailing canary words were overwritten (empty when clean or canaries are off)."""
        bad = []
        for name, raw in self._raw.items():
            n = self.bufs[name].numel()
            if not bool((raw[n:].view(torch.uint8) == self.CANARY_BYTE).all()):
                bad.append(name)
        return bad

    def retired_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.retired)


class HybridExecutor:
    def __init__(self, weights: ModelWeights, device="cuda", max_slots: int = 4, max_context: int = 4608,
                 n_pages: Optional[int] = None, gemm_impl: Optional[str] = None):
        self.cfg = cfg = weights.config
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.max_slots = max_slots
        self.max_context = max_context
        self.max_pages_per_slot = (max_context + PAGE - 1) // PAGE
        self.n_pages = n_pages if n_pages is not None else max_slots * self.max_pages_per_slot + 1
        self.gemm_impl = gemm_impl or os.environ.get("HE_GEMM", "tcgen05")
        self.scratch = _Scratch(self.device)
        # packed batches of up to small_rows rows take the quantised GEMV path, larger ones the tensor-core path
        # (the int8 GEMV costs ~1.65 ms per extra row on the 27B geometry; the split-K tensor-core path streams the
        # same quantised blocks once for any row count up to 128)
        # measured on the 27B: a packed step costs 7.0 / 8.7 / 10.3 / 11.7 / 14.0 / 18.5 ms at 2 / 3 / 4 / 5 / 6 / 8
        # rows on the GEMV path and 13.3 / 13.6 / 14.2 ms at 5 / 6 / 8 rows on the tensor-core path, so the switch is
        # above five rows
        self.small_rows = min(GEMV_MAX_ROWS, int(os.environ.get("HE_SMALL_ROWS", "5")))
        self.dw: Dict[str, DeviceWeight] = {}
        self.f32: Dict[str, torch.Tensor] = {}
        # per-stage device timing of the tensor-core (many rows) path, off unless HE_STAGE_TIMING=1 (the role of the
        # reference's stage timers, hipengine/runtime/qwen35_gguf_timing.py:1-80): CUDA events around each stage,
        # read back once by stage_summary()
        from ..utils.tracing import StageTimer
        self.timer = StageTimer(enabled=os.environ.get("HE_STAGE_TIMING", "0") == "1")
        self._load(weights)
        self._alloc_state()

    # ------------------------------------------------------------------ weights
    def _load(self, weights: ModelWeights) -> None:
        for name, t in weights.tensors.items():
            raw = t.raw.to(self.device)
            if t.ggml_type == GGMLType.F32 and (len(t.shape) == 1 or name.endswith(("ssm_a", "ssm_dt.bias",
                                                                                  "ssm_conv1d.weight"))):
                self.f32[name] = raw.view(torch.float32).reshape(t.shape).contiguous()
                continue
            if len(t.shape) == 3:
                E, Nn, Kk = t.shape
                self.dw[name] = K.to_device_weight(raw, t.ggml_type, E * Nn, Kk)
                continue
            if t.ggml_type == GGMLType.F32:
                self.f32[name] = raw.view(torch.float32).reshape(t.shape).contiguous()
            self.dw[name] = K.to_device_weight(raw, t.ggml_type, t.n_rows, t.n_cols)
        if "output.weight" not in self.dw:
            self.dw["output.weight"] = self.dw["token_embd.weight"]
        # prefill path: the two small F32 gate projections of a linear layer run as one bf16 tensor-core GEMM
        # ... and for decode they ride the int8 block path of the fused GEMV as one Q8_0 segment: as fp32 rows each
        # was a 20 KB dot product walked by a single warp, a latency-bound tail twice as long as the rest of the launch
        self.ab_bf16: Dict[int, torch.Tensor] = {}
        self.ab_q8: Dict[int, DeviceWeight] = {}
        from ..quant.ggml import quantize
        for i in range(self.cfg.n_layers):
            a_name, b_name = f"blk.{i}.ssm_alpha.weight", f"blk.{i}.ssm_beta.weight"
            if a_name in self.f32 and b_name in self.f32:
                ab = torch.cat([self.f32[a_name], self.f32[b_name]], 0).contiguous()
                # rows padded with zeros to a multiple of 8 so that the tensor-core GEMM takes any head count (six value
                # heads per rank at eight-way tensor parallelism would otherwise fall to the scalar kernel, which
                # walks all 4096 activation rows once per output column)
                pad = (-ab.shape[0]) % 8
                abp = torch.cat([ab, ab.new_zeros(pad, ab.shape[1])], 0) if pad else ab
                self.ab_bf16[i] = abp.to(torch.bfloat16).contiguous()
                if ab.shape[1] % 256 == 0 and os.environ.get("HE_AB_Q8", "1") != "0":
                    raw = quantize(ab, GGMLType.Q8_0).reshape(ab.shape[0], -1).contiguous()
                    self.ab_q8[i] = K.to_device_weight(raw, GGMLType.Q8_0, ab.shape[0], ab.shape[1])

    def _stage(self, name: str):
        """Context manager timing one stage (a no-op when timing is off or the stream is being captured)."""
        if self.timer.enabled and not torch.cuda.is_current_stream_capturing():
            return self.timer.stage(name)
        import contextlib
        return contextlib.nullcontext()

    def stage_summary(self) -> Dict[str, Dict[str, float]]:
        return self.timer.summary()

    def W(self, i: int, slot: str) -> DeviceWeight:
        return self.dw[f"blk.{i}.{slot}"]

    def F(self, i: int, slot: str) -> torch.Tensor:
        return self.f32[f"blk.{i}.{slot}"]

    # ------------------------------------------------------------------ state
    def _alloc_state(self) -> None:
        cfg, dev = self.cfg, self.device
        kinds = cfg.layer_kinds()
        n_blocks = cfg.n_layers + cfg.nextn_layers
        self.kv: Dict[int, torch.Tensor] = {}
        self.conv_state: Dict[int, torch.Tensor] = {}
        self.gdn_state: Dict[int, torch.Tensor] = {}
        for i in range(n_blocks):
            full = True if i >= cfg.n_layers else kinds[i] == "full"
            if full:
                self.kv[i] = torch.zeros(self.n_pages, 2, cfg.n_kv_heads, PAGE, cfg.head_dim, dtype=torch.bfloat16,
                                         device=dev)
            else:
                self.conv_state[i] = torch.zeros(self.max_slots, cfg.linear_qkv_width, cfg.conv_kernel - 1,
                                                 dtype=torch.float32, device=dev)
                self.gdn_state[i] = torch.zeros(self.max_slots, cfg.ssm_v_heads, cfg.ssm_state, cfg.ssm_state,
                                                dtype=torch.float32, device=dev)
        # default identity paging: slot s owns pages [1 + s*mp, 1 + (s+1)*mp); page 0 is a scratch sink
        mp = self.max_pages_per_slot
        bt = torch.arange(self.max_slots * mp, dtype=torch.int32).reshape(self.max_slots, mp) + 1
        if self.n_pages < self.max_slots * mp + 1:
            bt = bt.clamp(max=self.n_pages - 1)
        self.block_table = bt.to(dev)
        self.am_v = torch.empty(GEMV_MAX_ROWS * 64 * 64, dtype=torch.float32, device=dev)
        self.am_i = torch.empty(GEMV_MAX_ROWS * 64 * 64, dtype=torch.int32, device=dev)

    def reset_slot(self, slot: int) -> None:
        for t in self.conv_state.values():
            t[slot].zero_()
        for t in self.gdn_state.values():
            t[slot].zero_()

    def state_bytes(self) -> int:
        tot = 0
        for d in (self.kv, self.conv_state, self.gdn_state):
            tot += sum(t.numel() * t.element_size() for t in d.values())
        return tot

    # ------------------------------------------------------------------ linear algebra dispatch
    def _gemm(self, x: torch.Tensor, w: DeviceWeight, out: torch.Tensor, row0: int = 0, rows: Optional[int] = None,
              tag: str = "w") -> torch.Tensor:
        """out[T, rows] (bf16) = x[T, K] (bf16) @ W[row0:row0+rows, :]^T on the tensor cores."""
        rows = w.n_rows - row0 if rows is None else rows
        if self.gemm_impl == "tcgen05":
            from ..ops import gemm as G
            return G.gemm_quant(x, w, out, self.scratch, row0=row0, rows=rows)
        wb = self.scratch.get("deq_" + tag, (rows, w.n_cols), torch.bfloat16)
        K.dequant_bf16(w, wb, row0=row0, rows=rows)
        torch.matmul(x, wb.t(), out=out)
        return out

    SPLITK_MAX_ROWS = 128

    def _use_splitk(self, T: int) -> bool:
        return (self.gemm_impl == "tcgen05" and T <= self.SPLITK_MAX_ROWS and os.environ.get("HE_SPLITK", "1") != "0")

    def _proj(self, x: torch.Tensor, w: DeviceWeight, name: str, tag: str, out: Optional[torch.Tensor] = None
              ) -> torch.Tensor:
        """x[T, K] (bf16) @ W^T for the tensor-core path.  Large batches: bf16 result.  Batches of at most
        SPLITK_MAX_ROWS rows: split-K into a zeroed fp32 buffer, so that all SMs stream the weight even when the
        output is only a few tiles wide (the consumers take fp32 or bf16 rows)."""
        T = x.shape[0]
        if self._use_splitk(T):
            from ..ops import gemm as GM
            acc = out if out is not None else self.scratch.get(name + "_f32", (T, w.n_rows), torch.float32)
            return GM.gemm_quant_splitk(x, w, acc, self.scratch)
        dst = out if out is not None else self.scratch.get(name + "_bf", (T, w.n_rows), torch.bfloat16)
        return self._gemm(x, w, dst, tag=tag)

    # GEMVs whose activation rows ARE the residual stream go through this hook, and any other reader of the residual
    # calls _sync_resid first: a tensor-parallel executor defers the cross-rank sum of a row-parallel projection to
    # the next reader (folded into that GEMV's prologue, or a small stand-alone kernel).
    def _gemv_resid(self, h: torch.Tensor, segs, norm_w: torch.Tensor, eps: float) -> None:
        K.gemv(h, segs, norm_w=norm_w, eps=eps)

    def _sync_resid(self, h: torch.Tensor) -> None:
        return

    # Tensor-core (many rows) path: the normalised bf16 rows the projections read, the residual buffer of a forward
    # pass and its completion.  A sequence-parallel executor shards the residual by rows and overrides these.
    def _norm_rows(self, h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        xn = self.scratch.get("xn", (h.shape[0], self.cfg.hidden), torch.bfloat16)
        K.rmsnorm_rows(h, w, xn, self.cfg.rms_eps)
        return xn

    def _xn_ready(self) -> None:
        return

    def _resid_buffer(self, T: int) -> torch.Tensor:
        return self.scratch.get("h", (T, self.cfg.hidden), torch.float32)

    def _finish_resid(self, h: torch.Tensor) -> torch.Tensor:
        return h

    # Row-parallel ("output") projections: h += x @ W^T.  A tensor-parallel executor overrides these two to
    # reduce the partial products across ranks before the residual add.
    def _out_small(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor) -> None:
        K.gemv(x, [GemvSegment(w, h, K.EPI_ADD_F32)])

    def _out_big(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor, tag: str) -> None:
        T = x.shape[0]
        if self._use_splitk(T) and h.is_contiguous():
            # few rows against a hidden-wide output is only ~20 tiles: split K over the SMs and let the tiles add
            # themselves into the fp32 residual (which is the residual add)
            from ..ops import gemm as GM
            GM.gemm_quant_splitk(x, w, h, self.scratch, add=True)
            return
        if self.gemm_impl == "tcgen05" and h.is_contiguous():
            # accumulate straight into the fp32 residual in the GEMM epilogue (one CTA per tile: plain +=)
            from ..ops import gemm as GM
            GM.gemm_quant(x, w, h, self.scratch, epi=2)
            return
        y = self._gemm(x, w, self.scratch.get("y_bf", (T, w.n_rows), torch.bfloat16), tag=tag)
        K.resid_add_bf16(h, y)

    # ------------------------------------------------------------------ layers
    def _attention_full(self, i: int, h: torch.Tensor, b: BatchDesc, small: bool) -> None:
        cfg, sc = self.cfg, self.scratch
        T = b.T
        H, Hkv, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        qw = cfg.q_proj_width
        if small:
            qf = sc.get("q_f32", (T, qw), torch.float32)
            kf = sc.get("k_f32", (T, cfg.kv_width), torch.float32)
            vf = sc.get("v_f32", (T, cfg.kv_width), torch.float32)
            self._gemv_resid(h, [GemvSegment(self.W(i, "attn_q.weight"), qf),
                                 GemvSegment(self.W(i, "attn_k.weight"), kf),
                                 GemvSegment(self.W(i, "attn_v.weight"), vf)], self.F(i, "attn_norm.weight"),
                             cfg.rms_eps)
        else:
            self._sync_resid(h)
            with self._stage("norm"):
                xn = self._norm_rows(h, self.F(i, "attn_norm.weight"))
            with self._stage("attn_qkv_gemm"):
                qf = self._proj(xn, self.W(i, "attn_q.weight"), "q", "q")
                kf = self._proj(xn, self.W(i, "attn_k.weight"), "k", "k")
                vf = self._proj(xn, self.W(i, "attn_v.weight"), "v", "k")
        q_out = sc.get("q_out", (T, H, D), torch.bfloat16)
        gate = sc.get("gate_out", (T, H, D), torch.bfloat16) if cfg.gated_attention else None
        qn = self.f32.get(f"blk.{i}.attn_q_norm.weight") if cfg.qk_norm else None
        kn = self.f32.get(f"blk.{i}.attn_k_norm.weight") if cfg.qk_norm else None
        K.qkv_post(qf, kf, vf, qn, kn, q_out, gate, self.kv[i], self.block_table, b.slot, b.pos, H, Hkv, D, PAGE,
                   cfg.gated_attention, cfg.rope_dim, cfg.rope_theta, cfg.rms_eps)
        attn = sc.get("attn_out", (T, H * D), torch.bfloat16)
        with self._stage("attn_core"):
            self._attend(i, q_out, gate, b, attn)
        if small:
            self._out_small(attn, self.W(i, "attn_output.weight"), h)
        else:
            with self._stage("out_gemm"):
                self._out_big(attn, self.W(i, "attn_output.weight"), h, "o")

    def _attend(self, i: int, q_out: torch.Tensor, gate: Optional[torch.Tensor], b: BatchDesc,
                out: torch.Tensor) -> None:
        cfg = self.cfg
        T = b.T
        H, Hkv, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        if (T > GEMV_MAX_ROWS and b.segs_host is not None and os.environ.get("HE_PREFILL_ATTN", "flash") == "flash"):
            from ..ops import attention as A
            if A.flash_prefill_available(D):
                r0 = 0
                for (slot, pos0, n) in b.segs_host:
                    A.flash_prefill(q_out[r0:r0 + n], None if gate is None else gate[r0:r0 + n], self.kv[i],
                                    self.block_table, slot, pos0, out[r0:r0 + n], H, Hkv, D, PAGE, cfg.scale())
                    r0 += n
                return
        split_len, max_splits = K.attn_decode_split(b.max_ctx, T, Hkv)
        part = self.scratch.get("attn_part", (K.attn_decode_scratch_floats(T, H, max_splits, D),), torch.float32)
        K.attn_decode(q_out, gate, self.kv[i], self.block_table, b.slot, b.ctx_len, part, out, H, Hkv, D, PAGE,
                      split_len, max_splits, cfg.scale())

    def _attention_linear(self, i: int, h: torch.Tensor, b: BatchDesc, small: bool,
                          journal: Optional[dict] = None) -> None:
        cfg, sc = self.cfg, self.scratch
        T = b.T
        G, Hv, S, C = cfg.ssm_groups, cfg.ssm_v_heads, cfg.ssm_state, cfg.linear_qkv_width
        inner = cfg.ssm_inner
        a_p = sc.get("a_proj", (T, Hv), torch.float32)
        b_p = sc.get("b_proj", (T, Hv), torch.float32)
        if small:
            qkv = sc.get("qkv_f32", (T, C), torch.float32)
            z = sc.get("z_f32", (T, inner), torch.float32)
            if i in self.ab_q8:
                ab = sc.get("ab_proj", (T, 2 * Hv), torch.float32)
                ab_split = os.environ.get("HE_AB_SPLIT", "1" if cfg.hidden >= 4096 else "0")
                if ab_split != "0":
                    # the 2*Hv Q8_0 rows get their own (tiny) launch: in the same launch their 272-byte blocks
                    # would size every ring slot and halve the warps of the two big Q4_K projections (for narrow
                    # models the projections are so short that the extra launch costs more than it saves)
                    self._gemv_resid(h, [GemvSegment(self.W(i, "attn_qkv.weight"), qkv),
                                         GemvSegment(self.W(i, "attn_gate.weight"), z)],
                                     self.F(i, "attn_norm.weight"), cfg.rms_eps)
                    K.gemv(h, [GemvSegment(self.ab_q8[i], ab)], norm_w=self.F(i, "attn_norm.weight"), eps=cfg.rms_eps)
                else:
                    self._gemv_resid(h, [GemvSegment(self.W(i, "attn_qkv.weight"), qkv),
                                         GemvSegment(self.W(i, "attn_gate.weight"), z),
                                         GemvSegment(self.ab_q8[i], ab)],
                                     self.F(i, "attn_norm.weight"), cfg.rms_eps)
                a_p, b_p = ab[:, :Hv], ab[:, Hv:]
            else:
                self._gemv_resid(h, [GemvSegment(self.W(i, "attn_qkv.weight"), qkv),
                                     GemvSegment(self.W(i, "attn_gate.weight"), z),
                                     GemvSegment(self.W(i, "ssm_alpha.weight"), a_p),
                                     GemvSegment(self.W(i, "ssm_beta.weight"), b_p)],
                                 self.F(i, "attn_norm.weight"), cfg.rms_eps)
        else:
            self._sync_resid(h)
            with self._stage("norm"):
                xn = self._norm_rows(h, self.F(i, "attn_norm.weight"))
            with self._stage("gdn_qkvz_gemm"):
                qkv = self._proj(xn, self.W(i, "attn_qkv.weight"), "qkv", "q")
                z = self._proj(xn, self.W(i, "attn_gate.weight"), "z", "q")
            if self.gemm_impl == "tcgen05" and i in self.ab_bf16:
                from ..ops import gemm as GM
                ab = sc.get("ab_proj", (T, self.ab_bf16[i].shape[0]), torch.float32)
                GM.gemm_bf16(xn, self.ab_bf16[i], ab)
                a_p, b_p = ab[:, :Hv], ab[:, Hv:2 * Hv]
            else:
                K.small_gemm_f32(xn, self.F(i, "ssm_alpha.weight"), a_p)
                K.small_gemm_f32(xn, self.F(i, "ssm_beta.weight"), b_p)
        conv = sc.get("conv_out", (T, C), torch.float32)
        decay = sc.get("decay", (T, Hv), torch.float32)
        beta = sc.get("beta", (T, Hv), torch.float32)
        og = sc.get("gdn_og", (T, inner), torch.bfloat16)
        if (small and journal is None and b.n_seg == T and S == 128 and cfg.conv_kernel == 4
                and os.environ.get("HE_GDN_FUSED", "1") != "0"):
            # plain decode rows: two fused launches instead of five
            K.gdn_decode(qkv, self.F(i, "ssm_conv1d.weight"), self.conv_state[i], a_p, b_p,
                         self.F(i, "ssm_a").reshape(-1), self.F(i, "ssm_dt.bias").reshape(-1), b.seg_slot, conv,
                         decay, beta, self.gdn_state[i], z, self.F(i, "ssm_norm.weight").reshape(-1), og, G, Hv,
                         cfg.rms_eps)
            self._out_small(og, self.W(i, "ssm_out.weight"), h)
            return
        cj = journal["conv"][i] if journal is not None else None
        _gdn_stage = self._stage("gdn_core")
        _gdn_stage.__enter__()
        K.conv1d(qkv, self.F(i, "ssm_conv1d.weight"), self.conv_state[i], b.seg_start, b.seg_slot, b.tok_seg, conv, C,
                 update_state=journal is None, journal=cj)
        K.gdn_prepare(conv, a_p, b_p, self.F(i, "ssm_a").reshape(-1), self.F(i, "ssm_dt.bias").reshape(-1), decay, beta,
                      G, Hv, S)
        o = sc.get("gdn_o", (T, Hv, S), torch.float32)
        gj = journal["gdn"][i] if journal is not None else None
        if (journal is None and S == 128 and T >= 64 * b.n_seg and os.environ.get("HE_GDN_CHUNKED", "1") != "0"):
            # long prefill segments: 16-token chunks on the tensor cores instead of the token-serial recurrence
            K.gdn_scan_chunked(conv, decay, beta, self.gdn_state[i], b.seg_start, b.seg_slot, o, G, Hv)
        else:
            K.gdn_scan(conv, decay, beta, self.gdn_state[i], b.seg_start, b.seg_slot, o, G, Hv,
                       write_state=journal is None, journal=gj)
        K.gdn_gated_norm(o, z, self.F(i, "ssm_norm.weight").reshape(-1), og, Hv, S, cfg.rms_eps)
        _gdn_stage.__exit__(None, None, None)
        if small:
            self._out_small(og, self.W(i, "ssm_out.weight"), h)
        else:
            with self._stage("out_gemm"):
                self._out_big(og, self.W(i, "ssm_out.weight"), h, "o")

    def _ffn(self, i: int, h: torch.Tensor, b: BatchDesc, small: bool) -> None:
        cfg, sc = self.cfg, self.scratch
        T = b.T
        norm_w = self.F(i, ffn_norm_slot(cfg))
        if cfg.is_moe:
            from . import moe as M
            self._sync_resid(h)
            M.moe_ffn(self, i, h, T, norm_w, small)
            return
        Fd = cfg.ffn
        epi = K.EPI_SILU_MUL if cfg.act == "silu" else K.EPI_GELU_MUL
        if small:
            act = sc.get("ffn_act", (T, Fd), torch.bfloat16)
            self._gemv_resid(h, [GemvSegment(self.W(i, "ffn_gate.weight"), act, epi, self.W(i, "ffn_up.weight"))],
                             norm_w, cfg.rms_eps)
            self._out_small(act, self.W(i, "ffn_down.weight"), h)
        else:
            self._sync_resid(h)
            with self._stage("norm"):
                xn = self._norm_rows(h, norm_w)
            if self._use_splitk(T):
                from ..ops import gemm as GM
                gu = sc.get("ffn_gu_f32", (T, 2 * Fd), torch.float32)
                GM.gemm_quant_splitk(xn, self.W(i, "ffn_gate.weight"), gu[:, :Fd], sc)
                GM.gemm_quant_splitk(xn, self.W(i, "ffn_up.weight"), gu[:, Fd:], sc)
            else:
                gu = sc.get("ffn_gu", (T, 2 * Fd), torch.bfloat16)
                with self._stage("ffn_gateup_gemm"):
                    self._gemm(xn, self.W(i, "ffn_gate.weight"), gu[:, :Fd], tag="g")
                    self._gemm(xn, self.W(i, "ffn_up.weight"), gu[:, Fd:], tag="g")
            act = sc.get("ffn_act", (T, Fd), torch.bfloat16)
            with self._stage("act_mul"):
                K.act_mul(gu, act, cfg.act)
            with self._stage("ffn_down_gemm"):
                self._out_big(act, self.W(i, "ffn_down.weight"), h, "d")

    # ------------------------------------------------------------------ whole model
    def forward(self, b: BatchDesc, journal: Optional[dict] = None, h_out: Optional[torch.Tensor] = None,
                defer_resid: bool = False) -> torch.Tensor:
        """Runs all layers over the packed rows; returns the fp32 residual stream [T, hidden] (pre output_norm).
        With ``defer_resid`` a tensor-parallel executor may leave the last cross-rank sum pending for ``logits`` /
        ``head_greedy`` to fold in; otherwise the returned rows are complete."""
        cfg = self.cfg
        T = b.T
        small = T <= self.small_rows
        h = h_out if h_out is not None else self._resid_buffer(T)
        K.embed(self.dw["token_embd.weight"], b.tokens, h, cfg.embed_scale)
        for i in range(cfg.n_layers):
            if cfg.is_full_attention_layer(i):
                self._attention_full(i, h, b, small)
            else:
                self._attention_linear(i, h, b, small, journal)
            self._ffn(i, h, b, small)
        if not defer_resid:
            self._sync_resid(h)
        return self._finish_resid(h)

    def logits(self, h_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
               hidden_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """output_norm + lm_head over the given residual rows [R, hidden] -> fp32 logits [R, vocab]."""
        cfg = self.cfg
        R = h_rows.shape[0]
        head = self.dw["output.weight"]
        if out is None:
            out = self.scratch.get("logits", (R, cfg.vocab), torch.float32)
        if R <= GEMV_MAX_ROWS:
            self._gemv_resid(h_rows, [GemvSegment(head, out)], self.f32["output_norm.weight"], cfg.rms_eps)
        else:
            self._sync_resid(h_rows)
            xn = self.scratch.get("xn_head", (R, cfg.hidden), torch.bfloat16)
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], xn, cfg.rms_eps)
            lb = self._gemm(xn, head, self.scratch.get("logits_bf", (R, cfg.vocab), torch.bfloat16), tag="head")
            out.copy_(lb)
        if hidden_out is not None:
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], hidden_out, cfg.rms_eps)
        if cfg.final_softcap > 0:
            K.softcap_(out, cfg.final_softcap)
        return out

    def head_greedy(self, h_rows: torch.Tensor, out_ids: torch.Tensor, logits_out: Optional[torch.Tensor] = None,
                    hidden_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Greedy decode head: output norm + lm_head + argmax over the rows -> ``out_ids`` (int64).  A vocab-parallel
        executor overrides this to merge per-shard (max, id) pairs instead of gathering logits."""
        lg = self.logits(h_rows, out=logits_out, hidden_out=hidden_out)
        return self.greedy(lg, out_ids)

    # ------------------------------------------------------------------ NextN / MTP draft block
    @property
    def has_nextn(self) -> bool:
        return self.cfg.nextn_layers > 0 and f"blk.{self.cfg.n_layers}.nextn.eh_proj.weight" in self.dw

    def nextn_forward(self, b: BatchDesc, hidden_prev: torch.Tensor) -> torch.Tensor:
        """One pass of the trailing NextN block over the packed rows.

        Row input = eh_proj([RMSNorm_e(embed(token)) | RMSNorm_h(hidden_prev)]) where ``hidden_prev`` [T, hidden]
        is the post-norm hidden of the position before the row's token; then the block's own gated attention
        (its own KV planes, layer index ``n_layers``) and FFN.  Returns the fp32 residual rows [T, hidden].
        Contract: hipengine/kernels/cpu_reference/ops.py:840-955 (the reference's NextN oracle).
        """
        cfg, sc = self.cfg, self.scratch
        i = cfg.n_layers
        T, H = b.T, cfg.hidden
        small = T <= self.small_rows
        table = self.dw.get(f"blk.{i}.nextn.embed_tokens.weight", self.dw["token_embd.weight"])
        e = sc.get("nx_e", (T, H), torch.float32)
        K.embed(table, b.tokens, e, cfg.embed_scale)
        xcat = sc.get("nx_cat", (T, 2 * H), torch.float32)
        K.rmsnorm_rows(e, self.F(i, "nextn.enorm.weight"), xcat[:, :H], cfg.rms_eps)
        K.rmsnorm_rows(hidden_prev, self.F(i, "nextn.hnorm.weight"), xcat[:, H:], cfg.rms_eps)
        h = sc.get("nx_h", (T, H), torch.float32)
        w = self.W(i, "nextn.eh_proj.weight")
        if small:
            K.gemv(xcat, [GemvSegment(w, h, K.EPI_F32)])
        else:
            xb = sc.get("nx_cat_bf", (T, 2 * H), torch.bfloat16)
            xb.copy_(xcat)
            y = self._gemm(xb, w, sc.get("y_bf", (T, H), torch.bfloat16), tag="o")
            h.copy_(y)
        self._attention_full(i, h, b, small)
        self._ffn(i, h, b, small)
        return h

    def nextn_logits(self, h_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
                     hidden_out: Optional[torch.Tensor] = None, head_rows: int = 0) -> torch.Tensor:
        """Draft head: shared_head_norm (or output_norm) + shared head (or the model's head) over <= 8 rows.

        ``head_rows`` > 0 scores only the first ``head_rows`` vocabulary rows (hot-vocabulary draft head,
        ``speculative/draft_vocab.py``): rows are contiguous in every device layout, so the slice is the same buffer
        with a smaller row count and the logits come back as [R, head_rows]."""
        cfg = self.cfg
        i = cfg.n_layers
        R = h_rows.shape[0]
        norm_w = self.f32.get(f"blk.{i}.nextn.shared_head_norm.weight", self.f32["output_norm.weight"])
        head = self.dw.get(f"blk.{i}.nextn.shared_head_head.weight", self.dw["output.weight"])
        if 0 < head_rows < head.n_rows:
            head = K.DeviceWeight(head.qtype, int(head_rows), head.n_cols, head.data)
        if out is None:
            out = self.scratch.get("nx_logits" if head_rows <= 0 else "nx_logits_hot", (R, head.n_rows),
                                   torch.float32)
        if hidden_out is not None:
            K.rmsnorm_rows(h_rows, norm_w, hidden_out, cfg.rms_eps)
        for r0 in range(0, R, GEMV_MAX_ROWS):
            r1 = min(R, r0 + GEMV_MAX_ROWS)
            K.gemv(h_rows[r0:r1], [GemvSegment(head, out[r0:r1])], norm_w=norm_w, eps=cfg.rms_eps)
        return out

    def alloc_journal(self, rows: int) -> dict:
        """Per-verify-row recurrent state journals for every linear-attention layer."""
        cfg = self.cfg
        j = {"conv": {}, "gdn": {}}
        for i in self.conv_state:
            j["conv"][i] = torch.empty(rows, cfg.linear_qkv_width, cfg.conv_kernel - 1, dtype=torch.float32,
                                       device=self.device)
            j["gdn"][i] = torch.empty(rows, cfg.ssm_v_heads, cfg.ssm_state, cfg.ssm_state, dtype=torch.float32,
                                      device=self.device)
        return j

    def commit_journal(self, journal: dict, seg_slot: torch.Tensor, commit_row: torch.Tensor) -> None:
        """state[seg_slot[s]] = journal[commit_row[s]] for every linear layer (speculative commit)."""
        cfg = self.cfg
        for i, st in self.conv_state.items():
            K.state_commit(st, journal["conv"][i], seg_slot, commit_row, cfg.linear_qkv_width * (cfg.conv_kernel - 1))
            K.state_commit(self.gdn_state[i], journal["gdn"][i], seg_slot, commit_row,
                           cfg.ssm_v_heads * cfg.ssm_state * cfg.ssm_state)

    def greedy(self, logits: torch.Tensor, out_ids: torch.Tensor) -> torch.Tensor:
        return K.argmax_rows(logits, self.am_v, self.am_i, out_ids)

    # ------------------------------------------------------------------ convenience (tests, smoke, bench)
    @torch.no_grad()
    def prefill(self, slot: int, tokens: Sequence[int], start_pos: int = 0, chunk: int = 4096,
                graph: Optional[bool] = None) -> torch.Tensor:
        """Prefill one request; returns the fp32 logits of its last row [1, vocab].

        With ``graph`` (default: ``HE_PREFILL_GRAPH=1``) a single-chunk prefill is replayed from a CUDA graph keyed by
        (slot, start position, rows): the first call of a key runs eagerly, the second captures, later ones copy the
        token ids into the graph's input buffer and launch once.  The forward of a sharded model is hundreds of
        short launches per layer group; with eight ranks driven by eight Python processes the host, not the GPUs,
        sets the pace of an eager prefill, and a replayed graph takes the host out of it."""
        if graph is None:
            graph = os.environ.get("HE_PREFILL_GRAPH", "0") == "1"
        if graph and 0 < len(tokens) <= chunk:
            return self._prefill_graphed(slot, tokens, start_pos)
        last_h = None
        for c0 in range(0, len(tokens), chunk):
            ids = tokens[c0:c0 + chunk]
            b = make_batch([(slot, start_pos + c0, ids)], self.device)
            h = self.forward(b)
            last_h = h[b.T - 1:b.T]
        return self.logits(last_h)

    def _prefill_graphed(self, slot: int, tokens: Sequence[int], start_pos: int) -> torch.Tensor:
        T = len(tokens)
        key = (slot, start_pos, T)
        cache = self.__dict__.setdefault("_prefill_graphs", {})
        ent = cache.get(key)
        if ent is None:
            # first sight of the shape: eager (sizes the scratch, sets function attributes), remember it
            cache[key] = {"seen": 1}
            return self.prefill(slot, tokens, start_pos, graph=False)
        if "graph" not in ent:
            b = make_batch([(slot, start_pos, [0] * T)], self.device)
            ent["tok"] = b.tokens
            ent["stage"] = torch.empty(T, dtype=torch.int64).pin_memory()
            ent["logits"] = torch.empty(1, self.cfg.vocab, dtype=torch.float32, device=self.device)
            torch.cuda.synchronize()
            k0 = K.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                h = self.forward(b)
                self.logits(h[T - 1:T], out=ent["logits"])
            ent["kernels"] = K.launch_count() - k0
            ent["graph"], ent["batch"] = g, b
        ent["stage"].copy_(torch.as_tensor(tokens, dtype=torch.int64))
        ent["tok"].copy_(ent["stage"], non_blocking=True)
        ent["graph"].replay()
        K.add_launches(ent["kernels"])
        return ent["logits"]

    @torch.no_grad()
    def forward_logits(self, slot: int, tokens: Sequence[int], start_pos: int = 0) -> torch.Tensor:
        """All-row logits for one segment (teacher-forced comparison against the reference)."""
        b = make_batch([(slot, start_pos, tokens)], self.device)
        h = self.forward(b)
        out = torch.empty(b.T, self.cfg.vocab, dtype=torch.float32, device=self.device)
        for r0 in range(0, b.T, GEMV_MAX_ROWS):
            r1 = min(b.T, r0 + GEMV_MAX_ROWS)
            self.logits(h[r0:r1], out=out[r0:r1])
        return out
