"""Tensor-parallel executor: the single-GPU hybrid executor run on a weight shard, plus the reductions.

Column-parallel projections (QKV, gate/up, the GDN input projections) need no communication: every rank
holds the replicated fp32 residual stream and produces its own heads / FFN columns.  Row-parallel projections
(attention output, ``ssm_out``, FFN down) produce partial sums of the full hidden width that are reduced over
the ranks and added to the residual.  Two reduction back-ends:

* ``comm="nccl"``  : ``torch.distributed.all_reduce`` (captured inside the decode CUDA graphs) -- the baseline;
* ``comm="fused"`` : own kernels over peer memory.  Few rows (``csrc/comm.cu``): every rank pushes its partial
  rows into all peers' symmetric buffers and the reduction is folded into one small kernel that also applies
  the residual add, so a decode step has no library collective at all.  Many rows
  (``csrc/gemm_sm100.cu::gemm_bf16_allreduce_kernel``): the tcgen05 GEMM pushes its partial tiles to their owner
  ranks from the epilogue, owners reduce and broadcast, every rank adds into its residual -- one kernel.

The output head is vocab-parallel; logits are all-gathered (greedy decode merges per-shard (max, id) pairs
instead).  The reference engine is single-device (its ``docs/ARCHITECTURE.md`` lists multi-GPU as future work),
so this layer has no counterpart there; sharding rules follow the planning notes on its geometry
(``hipengine/kernels/policy.py:103-153``).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..loading.weights import ModelWeights
from ..models.executor import GEMV_MAX_ROWS, HybridExecutor
from ..ops import kernels as K
from ..ops.kernels import DeviceWeight, GemvSegment
from .groups import DistContext, merge_argmax
from .sharding import TPPlan, shard_weights


class TPHybridExecutor(HybridExecutor):
    def __init__(self, full_weights: ModelWeights, ctx: DistContext, comm: Optional[str] = None, **kw):
        self.ctx = ctx
        self.full_cfg = full_weights.config
        shard, self.plan = shard_weights(full_weights, ctx.world, ctx.rank)
        self.comm = comm or os.environ.get("HE_TP_COMM", "nccl")
        super().__init__(shard, device=ctx.device, **kw)
        if self.full_cfg.is_moe and ctx.world > 1:
            # expert parallelism over the replicated activations: this rank computes only its experts' share
            self.expert_range = self.plan.experts
            self.owns_shared_expert = self.plan.owns_shared_expert
        self.fused = None
        self.fgemm = None
        self.peer = None
        self.peer_head = None
        self._pending = None
        self.sp = None
        if self.comm == "fused" and ctx.world > 1:
            from .fused import FusedReducer, PeerResidual
            self.fused = FusedReducer(ctx, self.full_cfg.hidden, max_rows=GEMV_MAX_ROWS)
            # decode: the all-reduce of a row-parallel projection is folded into the GEMVs around it (push from the
            # epilogue, sum in the next prologue), and the greedy head merges (max, id) pairs over peer memory
            # Every CTA of the consumer GEMV reads the partial rows of all ranks (world x 40 KB of tagged words for the
            # 27B width), so the fold pays up to four ranks (2 ranks: 30.7 vs 33.9 us per GEMV pair) and loses at
            # eight (4.52 vs 4.19 ms per decode step), where the stand-alone push/reduce kernel stays the default.
            fold_default = "1" if ctx.world <= 4 else "0"
            if os.environ.get("HE_TP_FOLD", fold_default) != "0" and self.full_cfg.hidden % 8 == 0 \
                    and self.full_cfg.hidden <= 8192:
                self.peer = PeerResidual(ctx, self.full_cfg.hidden, max_rows=GEMV_MAX_ROWS)
                self._pending = None          # (residual tensor, rows) of a push not yet summed into the residual
            if os.environ.get("HE_TP_PEER_HEAD", "1") != "0":
                # the (max, id) merge of the greedy head does not depend on the fold: no logits gather at any world
                self.peer_head = PeerResidual(ctx, 1, max_rows=64)
            if self.gemm_impl == "tcgen05" and self.full_cfg.hidden % 8 == 0 and \
                    os.environ.get("HE_TP_FUSED_GEMM", "1") != "0":
                from .fused import FusedGemmAllReduce
                rows = min(8192, (self.max_context + 127) // 128 * 128)
                if os.environ.get("HE_TP_SEQ_PARALLEL", "1") != "0":
                    # prefill: residual sharded by rows; GEMM -> reduce-scatter and all-gather -> GEMM over peer memory
                    from .fused import SeqParallel
                    self.sp = SeqParallel(ctx, self.full_cfg.hidden, max_rows=rows)
                else:
                    self.fgemm = FusedGemmAllReduce(ctx, self.full_cfg.hidden, max_rows=rows)

    # ------------------------------------------------------------------ reductions
    def _sync_resid(self, h: torch.Tensor) -> None:
        """Finish a pending push with the stand-alone reduce kernel (readers that are not a reduce-prologue GEMV)."""
        if self._pending is not None:
            ph, rows = self._pending
            self._pending = None
            self.peer.reduce_in(ph, rows)

    def _gemv_resid(self, h: torch.Tensor, segs, norm_w: torch.Tensor, eps: float) -> None:
        if self._pending is not None:
            ph, rows = self._pending
            fold = (ph.data_ptr() == h.data_ptr() and rows == h.shape[0] and h.dtype == torch.float32
                    and norm_w is not None and h.shape[1] == self.peer.width
                    and all(s.w.qtype in (8, 12, 14) and (s.w2 is None or s.w2.qtype in (8, 12, 14)) for s in segs))
            if fold:
                self._pending = None
                K.gemv(h, segs, norm_w=norm_w, eps=eps, comm=self.peer.comm(K.COMM_REDUCE))
                return
            self._sync_resid(h)
        K.gemv(h, segs, norm_w=norm_w, eps=eps)

    def _out_small(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor) -> None:
        if self.ctx.world == 1:
            return super()._out_small(x, w, h)
        T = x.shape[0]
        if self.peer is not None and w.n_rows == self.peer.width and w.qtype in (8, 12, 14):
            self._sync_resid(h)                 # at most one push in flight per residual
            K.gemv(x, [GemvSegment(w, h, K.EPI_F32)], comm=self.peer.comm(K.COMM_PUSH))
            self._pending = (h, T)
            return
        if self.fused is not None:
            part = self.fused.local_rows(T)
            K.gemv(x, [GemvSegment(w, part, K.EPI_F32)])
            self.fused.reduce_add(h, T)
            return
        part = self.scratch.get("tp_part", (T, w.n_rows), torch.float32)
        K.gemv(x, [GemvSegment(w, part, K.EPI_F32)])
        self.ctx.all_reduce_(part)
        K.resid_add_f32(h, part)

    def _moe_reduce(self, h: torch.Tensor, part: torch.Tensor) -> None:
        """h += sum over ranks of the per-rank expert contributions ``part`` [T, hidden] fp32."""
        T = part.shape[0]
        if self._sp_on(h):
            # expert parallelism over the row-sharded residual: each rank's expert outputs are reduce-scattered to
            # the rows' owners (peer stores of bf16 rows, fp32 sums)
            self.sp.rows_rs(part, T)
            return
        if self.peer is not None and T <= self.peer.max_rows and part.is_contiguous():
            self._sync_resid(h)
            self.peer.push_rows(part, T)
            self._pending = (h, T)
            return
        if self.fused is not None and T <= self.fused.max_rows:
            self.fused.local_rows(T).copy_(part)
            self.fused.reduce_add(h, T)
            return
        self.ctx.all_reduce_(part)
        K.resid_add_f32(h, part)

    # ------------------------------------------------------------------ sequence-parallel prefill
    def _sp_on(self, h: torch.Tensor) -> bool:
        return (self.sp is not None and h.shape[0] > self.SPLITK_MAX_ROWS and h.shape[0] <= self.sp.max_rows
                and h.data_ptr() == self.sp.h.data_ptr())

    def _resid_buffer(self, T: int) -> torch.Tensor:
        if self.sp is not None and self.SPLITK_MAX_ROWS < T <= self.sp.max_rows and self.gemm_impl == "tcgen05":
            return self.sp.h[:T]
        return super()._resid_buffer(T)

    def _norm_rows(self, h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        if self._sp_on(h):
            return self.sp.norm_push(h.shape[0], w, self.cfg.rms_eps)
        return super()._norm_rows(h, w)

    def _gemm(self, x: torch.Tensor, w: DeviceWeight, out: torch.Tensor, row0: int = 0, rows=None,
              tag: str = "w") -> torch.Tensor:
        if self.sp is not None and self.sp.ag_pending and x.data_ptr() == self.sp.xn.data_ptr():
            from ..ops import gemm as GM
            if GM.quant_gemm_ok(w) and self.gemm_impl == "tcgen05":
                # the first reader of freshly pushed rows waits for their owners tile by tile inside the kernel;
                # everything after it in the stream sees complete rows
                self.sp.ag_pending = False
                rows_ = w.n_rows - row0 if rows is None else rows
                return GM.gemm_quant(x, w, out, self.scratch, row0=row0, rows=rows_, ag=self.sp.ag_args())
            self.sp.wait()
        return super()._gemm(x, w, out, row0=row0, rows=rows, tag=tag)

    def _xn_ready(self) -> None:
        """Readers of freshly pushed rows that are not the all-gather GEMM wait here (stream-ordered)."""
        if self.sp is not None and self.sp.ag_pending:
            self.sp.wait()

    def _finish_resid(self, h: torch.Tensor) -> torch.Tensor:
        if self._sp_on(h):
            return self.sp.gather_residual(h.shape[0])
        return h

    def _out_big(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor, tag: str) -> None:
        if self.ctx.world == 1:
            return super()._out_big(x, w, h, tag)
        if self._sp_on(h):
            from ..ops import gemm as GM
            if GM.quant_gemm_ok(w):
                self.sp.gemm_rs(x, w, h.shape[0])
            else:
                y = self._gemm(x, w, self.scratch.get("y_bf", (x.shape[0], w.n_rows), torch.bfloat16), tag=tag)
                self.ctx.all_reduce_(y)
                K.resid_add_bf16(h, y)
            return
        if self.fgemm is not None and self.fgemm.supports(x.shape[0], h):
            # GEMM, all-reduce over peer memory and residual add as one tcgen05 kernel per rank
            from ..ops import gemm as GM
            self.fgemm.gemm_add(x, w if GM.quant_gemm_ok(w) else GM._float_weight_bf16(w, self.scratch), h)
            return
        y = self._gemm(x, w, self.scratch.get("y_bf", (x.shape[0], w.n_rows), torch.bfloat16), tag=tag)
        self.ctx.all_reduce_(y)
        K.resid_add_bf16(h, y)

    # ------------------------------------------------------------------ vocab-parallel head
    def logits(self, h_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
               hidden_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.ctx.world == 1:
            return super().logits(h_rows, out, hidden_out)
        cfg, full = self.cfg, self.full_cfg
        R = h_rows.shape[0]
        v0, v1 = self.plan.vocab_rows
        Vl = v1 - v0
        assert full.vocab % self.ctx.world == 0, "vocab-parallel head needs an even split"
        loc = self.scratch.get("logits_local", (R, Vl), torch.float32)
        head = self.dw["output.weight"]
        if R <= GEMV_MAX_ROWS:
            self._gemv_resid(h_rows, [GemvSegment(head, loc)], self.f32["output_norm.weight"], cfg.rms_eps)
        else:
            self._sync_resid(h_rows)
            xn = self.scratch.get("xn_head", (R, cfg.hidden), torch.bfloat16)
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], xn, cfg.rms_eps)
            lb = self._gemm(xn, head, self.scratch.get("logits_bf", (R, Vl), torch.bfloat16), tag="head")
            loc.copy_(lb)
        if hidden_out is not None:
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], hidden_out, cfg.rms_eps)
        self._local_logits = loc
        gathered = self.ctx.all_gather(loc)                       # [world, R, Vl]
        if out is None:
            out = self.scratch.get("logits", (R, full.vocab), torch.float32)
        out.view(R, self.ctx.world, Vl).copy_(gathered.permute(1, 0, 2))
        if cfg.final_softcap > 0:
            K.softcap_(out, cfg.final_softcap)
        return out


    def head_greedy(self, h_rows: torch.Tensor, out_ids: torch.Tensor, logits_out: Optional[torch.Tensor] = None,
                    hidden_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Vocab-parallel greedy head without a logits gather: argmax over this rank's vocabulary shard, then the
        ranks' (max, id) pairs are exchanged over peer memory and merged (lower id wins exact ties, as one argmax
        over the concatenated logits would)."""
        R = h_rows.shape[0]
        if self.ctx.world == 1 or self.peer_head is None or R > GEMV_MAX_ROWS or self.cfg.final_softcap > 0:
            return super().head_greedy(h_rows, out_ids, logits_out, hidden_out)
        cfg = self.cfg
        v0, v1 = self.plan.vocab_rows
        loc = self.scratch.get("logits_local", (R, v1 - v0), torch.float32)
        self._gemv_resid(h_rows, [GemvSegment(self.dw["output.weight"], loc)], self.f32["output_norm.weight"],
                         cfg.rms_eps)
        if hidden_out is not None:
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], hidden_out, cfg.rms_eps)
        lv = self.scratch.get("head_val", (R,), torch.float32)
        li = self.scratch.get("head_idx", (R,), torch.int64)
        K.argmax_rows(loc, self.am_v, self.am_i, li, out_val=lv)
        self.peer_head.argmax_merge(lv, li, v0, R, out_ids)
        return out_ids

    def close_comm(self) -> None:
        for obj in (self.peer, self.peer_head, self.sp):
            if obj is not None:
                obj.close()
        self.peer = self.peer_head = self.sp = None


def build_tp_executor(cfg, seed: int, device, ctx: Optional[DistContext] = None, comm: Optional[str] = None,
                      **kw) -> TPHybridExecutor:
    """Random-init model of geometry ``cfg`` (same seed on every rank, so shards agree), sharded for this rank."""
    from ..loading.synth import build_random_model
    from .groups import init_distributed
    ctx = ctx or init_distributed()
    full = build_random_model(cfg, seed=seed, device=str(device))
    ex = TPHybridExecutor(full, ctx, comm=comm, **kw)
    del full
    torch.cuda.empty_cache()
    return ex
