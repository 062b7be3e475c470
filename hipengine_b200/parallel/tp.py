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
        if self.comm == "fused" and ctx.world > 1:
            from .fused import FusedReducer
            self.fused = FusedReducer(ctx, self.full_cfg.hidden, max_rows=GEMV_MAX_ROWS)
            if self.gemm_impl == "tcgen05" and self.full_cfg.hidden % 8 == 0 and \
                    os.environ.get("HE_TP_FUSED_GEMM", "1") != "0":
                from .fused import FusedGemmAllReduce
                rows = min(8192, (self.max_context + 127) // 128 * 128)
                self.fgemm = FusedGemmAllReduce(ctx, self.full_cfg.hidden, max_rows=rows)

    # ------------------------------------------------------------------ reductions
    def _out_small(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor) -> None:
        if self.ctx.world == 1:
            return super()._out_small(x, w, h)
        T = x.shape[0]
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
        if self.fused is not None and T <= self.fused.max_rows:
            self.fused.local_rows(T).copy_(part)
            self.fused.reduce_add(h, T)
            return
        self.ctx.all_reduce_(part)
        K.resid_add_f32(h, part)

    def _out_big(self, x: torch.Tensor, w: DeviceWeight, h: torch.Tensor, tag: str) -> None:
        if self.ctx.world == 1:
            return super()._out_big(x, w, h, tag)
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
        if hidden_out is not None:
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], hidden_out, cfg.rms_eps)
        if R <= GEMV_MAX_ROWS:
            K.gemv(h_rows, [GemvSegment(head, loc)], norm_w=self.f32["output_norm.weight"], eps=cfg.rms_eps)
        else:
            xn = self.scratch.get("xn_head", (R, cfg.hidden), torch.bfloat16)
            K.rmsnorm_rows(h_rows, self.f32["output_norm.weight"], xn, cfg.rms_eps)
            lb = self._gemm(xn, head, self.scratch.get("logits_bf", (R, Vl), torch.bfloat16), tag="head")
            loc.copy_(lb)
        self._local_logits = loc
        gathered = self.ctx.all_gather(loc)                       # [world, R, Vl]
        if out is None:
            out = self.scratch.get("logits", (R, full.vocab), torch.float32)
        out.view(R, self.ctx.world, Vl).copy_(gathered.permute(1, 0, 2))
        if cfg.final_softcap > 0:
            K.softcap_(out, cfg.final_softcap)
        return out


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
