"""Speculative decoding for Gemma 4 with its assistant (MTP) head as the drafter.

Cycle for a request whose last committed token ``t0`` sits at position ``p`` (sampled, not yet fed to the backbone):
  draft   the head is seeded with the raw hidden row of the backbone forward that produced ``t0`` and chained K
          times; every step reads the backbone's own KV of its last two layers at the same key count ``p`` (the head
          owns no KV, so a draft leaves nothing behind to roll back);
  verify  one backbone forward over rows [t0, d1 .. dK] at positions p .. p+K (``ChainVerifyCycle``);
  accept  greedy: longest matching prefix; sampled: the exact min(1, p/q) rule with a one-hot proposal;
  commit  cursors advance by accepted + 1; the seed of the next cycle is the raw hidden of the verify row that
          produced the last emitted token.  KV rows past the accepted prefix are overwritten by the next cycle.
Between 1 and K + 1 tokens are committed per cycle, and the emitted tokens are the target's own (greedy requests:
the plain greedy continuation).

Reference: ``hipengine/generation/gemma4_mtp.py`` (provider ``gemma4_mtp``: draft / verify loop) and
``hipengine/runtime/gemma4_assistant.py`` (``Gemma4MtpDrafter``: seed, shared views taken once per draft, one
position for every step of a draft); contract ``docs/reference/GEMMA4-ASSISTANT-MTP.md:226-240``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..models.executor import BatchDesc
from ..ops import kernels as K
from .contracts import SpecCycleResult, SpeculativeCapability
from .mtp import ChainVerifyCycle
from .transaction import SpecTransaction, Stage


class AssistantMTPCycle(ChainVerifyCycle):
    def __init__(self, ex, head, max_depth: int = 3, max_requests: int = 8):
        super().__init__(ex, max_depth, max_requests)
        self.head = head
        self.max_requests = min(max_requests, head.max_rows)
        # per slot: raw hidden (before the output norm) of the backbone row that produced the slot's last token
        self.h_seed = torch.zeros(ex.max_slots, ex.cfg.hidden, dtype=torch.float32, device=ex.device)
        self.picked = torch.zeros(self.max_requests, ex.cfg.hidden, dtype=torch.float32, device=ex.device)

    def capability(self) -> SpeculativeCapability:
        return SpeculativeCapability(provider="gemma4_mtp", max_depth=self.max_depth,
                                     widths=tuple(range(1, self.max_requests + 1)), attachment="assistant_head",
                                     transaction_mode="kv_overwrite")

    # ------------------------------------------------------------------ seeds
    def reset_slot(self, slot: int) -> None:
        self.h_seed[slot].zero_()

    def after_prefill(self, batch: BatchDesc, h: torch.Tensor) -> None:
        """Keep the raw hidden of every segment's last row (the last chunk of a prompt overrides earlier ones)."""
        r0 = 0
        for (slot, _pos0, n) in batch.segs_host:
            self.h_seed[slot].copy_(h[r0 + n - 1])
            r0 += n

    def _after_commit(self, slot_t: torch.Tensor, hid: torch.Tensor, R: int, raw: Optional[torch.Tensor] = None) -> None:
        K.gather_rows_f32(raw, self.hidden_row[:R], self.picked[:R])
        self.h_seed.index_copy_(0, slot_t, self.picked[:R])

    # ------------------------------------------------------------------ one cycle
    @torch.no_grad()
    def cycle(self, slots: Sequence[int], last_tokens: Sequence[int], positions: Sequence[int], depth: int,
              temperature: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
              counters: Optional[Sequence[int]] = None, draft_override: Optional[torch.Tensor] = None
              ) -> Tuple[List[SpecCycleResult], SpecTransaction]:
        """positions[r] = position of last_tokens[r] = number of tokens the backbone has cached for the request.
        ``draft_override`` (int64 [R, depth]) replaces the proposals (tests of the acceptance paths)."""
        ex, dev = self.ex, self.ex.device
        R, Kd = len(slots), depth
        assert 1 <= Kd <= self.max_depth and R <= self.max_requests and min(positions) >= 1
        txn = SpecTransaction(list(range(R)))
        for st in (Stage.RESERVED, Stage.TARGET_OPEN, Stage.PROVIDER_OPEN):
            txn.advance(st)
        slot64 = torch.tensor(list(slots), dtype=torch.int64, device=dev)
        slot32 = slot64.to(torch.int32)
        n_past = torch.tensor(list(positions), dtype=torch.int32, device=dev)
        t0 = torch.tensor(list(last_tokens), dtype=torch.int64, device=dev)
        drafts = torch.empty(R, Kd, dtype=torch.int64, device=dev)
        tok, h = t0, self.h_seed.index_select(0, slot64)
        ids = self.am_ids[:R]
        max_ctx = int(max(positions))
        for j in range(Kd):
            logits, h = self.head.forward_batch(tok, h, slot32, n_past, max_ctx)
            ex.greedy(logits, ids)
            drafts[:, j].copy_(ids)
            tok = drafts[:, j].contiguous()
        if draft_override is not None:
            drafts.copy_(draft_override.to(dev))
        txn.advance(Stage.DRAFTED)
        res = self._verify_accept_commit(txn, slots, positions, t0, drafts, temperature, seeds, counters)
        return res, txn
