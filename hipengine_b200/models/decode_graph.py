"""Whole-step CUDA graphs for decode buckets.

A decode step for R resident rows (embed -> all layers -> output norm -> lm_head -> sampler/argmax ->
token publish -> position advance) is captured once per bucket and replayed with one launch, so the
per-token host cost is O(1).  All per-step inputs (token ids, positions, context lengths, block-table
rows) live in persistent device tensors that in-graph kernels update, the design the reference uses for
its c=1 and packed decode graphs (``hipengine/runtime/gguf_decode_graph.py:88-110``,
``hipengine/runtime/gguf_packed_decode_graph.py``; bookkeeping kernels in
``hipengine/kernels/hip_gfx1100/runtime/state.hip``).  The split-K grid of the attention kernel is sized
for the bucket's context ceiling; spans past a row's live context exit immediately.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Sequence, Tuple

import torch

from ..core import native as N
from ..ops import kernels as K
from .executor import GEMV_MAX_ROWS, BatchDesc, HybridExecutor

CTX_BUCKETS = (1024, 4096, 8192, 16384, 32768, 65536, 131072, 262144)


def ctx_bucket(ctx: int) -> int:
    for b in CTX_BUCKETS:
        if ctx <= b:
            return b
    return ctx


class DecodeGraphRunner:
    """Persistent decode rows + captured graphs keyed by (rows, context bucket)."""

    def __init__(self, ex: HybridExecutor, max_rows: int = GEMV_MAX_ROWS, use_graphs: bool = True):
        self.ex = ex
        self.max_rows = max_rows
        self.use_graphs = use_graphs
        dev = ex.device
        R = max_rows
        self.tokens = torch.zeros(R, dtype=torch.int64, device=dev)
        self.slot = torch.zeros(R, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(R, dtype=torch.int32, device=dev)
        self.ctx_len = torch.ones(R, dtype=torch.int32, device=dev)
        self.seg_start = torch.arange(R + 1, dtype=torch.int32, device=dev)
        self.tok_seg = torch.arange(R, dtype=torch.int32, device=dev)
        self.next_ids = torch.zeros(R, dtype=torch.int64, device=dev)
        self.logits = torch.empty(R, ex.cfg.vocab, dtype=torch.float32, device=dev)
        self.hidden = torch.empty(R, ex.cfg.hidden, dtype=torch.float32, device=dev)
        self.graphs: Dict[Tuple[int, int, bool], torch.cuda.CUDAGraph] = {}
        self.stats = {"hits": 0, "misses": 0, "captures": 0, "kernels_per_graph": {}, "native_launches": 0}
        # replay through the native launcher (validated control block + cudaGraphLaunch) when torch exposes the
        # instantiated graph; otherwise through torch's own replay
        self.native_launch = os.environ.get("HE_NATIVE_GRAPH_LAUNCH", "1") != "0"
        self._execs: Dict[Tuple[int, int, bool], int] = {}

    def batch(self, rows: int, max_ctx: int) -> BatchDesc:
        return BatchDesc(self.tokens[:rows], self.slot[:rows], self.pos[:rows], self.ctx_len[:rows],
                         self.seg_start[:rows + 1], self.slot[:rows], self.tok_seg[:rows], rows, rows, max_ctx)

    def set_rows(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> None:
        """Host -> device install of the resident rows (done on admission / compaction, not per token)."""
        n = len(slots)
        dev = self.ex.device
        self.slot[:n].copy_(torch.tensor(slots, dtype=torch.int32), non_blocking=True)
        self.tokens[:n].copy_(torch.tensor(tokens, dtype=torch.int64), non_blocking=True)
        p = torch.tensor(positions, dtype=torch.int32)
        self.pos[:n].copy_(p, non_blocking=True)
        self.ctx_len[:n].copy_(p + 1, non_blocking=True)

    def _step_body(self, rows: int, max_ctx: int, greedy: bool) -> None:
        ex = self.ex
        b = self.batch(rows, max_ctx)
        h = ex.forward(b, defer_resid=True)
        if greedy:
            ex.head_greedy(h, self.next_ids[:rows], logits_out=self.logits[:rows], hidden_out=self.hidden[:rows])
            self.publish(rows)
        else:
            ex.logits(h, out=self.logits[:rows], hidden_out=self.hidden[:rows])

    def publish(self, rows: int) -> None:
        """next_ids -> tokens, advance positions (device side)."""
        self.tokens[:rows].copy_(self.next_ids[:rows])
        N.check(N.lib().he_advance_positions(C.c_void_p(self.pos.data_ptr()), C.c_void_p(self.ctx_len.data_ptr()),
                                             C.c_void_p(None), C.c_int(rows), C.c_int(1), K._stream()),
                "he_advance_positions")

    def step(self, rows: int, max_ctx: int, greedy: bool = True) -> None:
        """One decode step for the first `rows` resident rows.  Greedy steps also publish the next token."""
        if not self.use_graphs:
            self._step_body(rows, max_ctx, greedy)
            return
        key = (rows, ctx_bucket(max_ctx), greedy)
        g = self.graphs.get(key)
        if g is None:
            self.stats["misses"] += 1
            # warm-up outside capture so scratch growth and function attributes are settled;
            # save and restore the recurrent state the warm-up step mutates
            snap = self._snapshot_rows(rows)
            self._step_body(rows, key[1], greedy)
            torch.cuda.synchronize()
            self._restore_rows(rows, snap)
            k0 = K.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step_body(rows, key[1], greedy)
            self.stats["kernels_per_graph"][key] = K.launch_count() - k0
            self._restore_rows(rows, snap)
            self.graphs[key] = g
            self.stats["captures"] += 1
        else:
            self.stats["hits"] += 1
        exec_h = self._execs.get(key) if self.native_launch else None
        if exec_h is None and self.native_launch and key not in self._execs:
            from ..core import runtime as RT
            exec_h = self._execs[key] = RT.graph_exec_handle(g)
        if exec_h:
            from ..core import runtime as RT
            ctl = RT.make_control(RT.STAGE_DECODE_STEP, rows, 0)
            res = RT.cycle_launch(ctl, exec_h, torch.cuda.current_stream().cuda_stream)
            if res.rc != 0:
                raise RuntimeError(f"native graph launch failed: rc={res.rc}")
            self.stats["native_launches"] += 1
        else:
            g.replay()
        K.add_launches(self.stats["kernels_per_graph"][key])

    # -- warm-up isolation: a capture warm-up must not advance real request state
    def _snapshot_rows(self, rows: int):
        ex = self.ex
        slots = self.slot[:rows].long()
        return {
            "tokens": self.tokens.clone(), "pos": self.pos.clone(), "ctx": self.ctx_len.clone(),
            "conv": {i: t[slots].clone() for i, t in ex.conv_state.items()},
            "gdn": {i: t[slots].clone() for i, t in ex.gdn_state.items()},
            "slots": slots,
        }

    def _restore_rows(self, rows: int, snap) -> None:
        ex = self.ex
        self.tokens.copy_(snap["tokens"])
        self.pos.copy_(snap["pos"])
        self.ctx_len.copy_(snap["ctx"])
        for i, t in ex.conv_state.items():
            t[snap["slots"]] = snap["conv"][i]
        for i, t in ex.gdn_state.items():
            t[snap["slots"]] = snap["gdn"][i]
