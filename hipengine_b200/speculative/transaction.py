"""Speculative cycle as a transaction with explicit stages.

Same stage vocabulary as the reference (``hipengine/speculative/transaction.py``): NEW -> RESERVED ->
TARGET_OPEN -> PROVIDER_OPEN -> DRAFTED -> VERIFIED -> ACCEPTED -> READBACK -> COMMITTING -> COMMITTED, with
ROLLED_BACK / CANCELLED reachable from any non-terminal stage.  The object owns no device memory; it records the
order of operations so that a failure in any stage knows what must be undone (nothing before TARGET_OPEN, KV
cursor rewind and journal discard after it) and tests can assert the order.
"""
from __future__ import annotations

import enum
from typing import Callable, List, Optional


class Stage(enum.Enum):
    NEW = "new"
    RESERVED = "reserved"
    TARGET_OPEN = "target_open"
    PROVIDER_OPEN = "provider_open"
    DRAFTED = "drafted"
    VERIFIED = "verified"
    ACCEPTED = "accepted"
    READBACK = "readback"
    COMMITTING = "committing"
    COMMITTED = "committed"
    ROLLED_BACK = "rolled_back"
    CANCELLED = "cancelled"


_ORDER = [Stage.NEW, Stage.RESERVED, Stage.TARGET_OPEN, Stage.PROVIDER_OPEN, Stage.DRAFTED, Stage.VERIFIED,
          Stage.ACCEPTED, Stage.READBACK, Stage.COMMITTING, Stage.COMMITTED]
_TERMINAL = {Stage.COMMITTED, Stage.ROLLED_BACK, Stage.CANCELLED}


class TransactionError(RuntimeError):
    pass


class SpecTransaction:
    def __init__(self, rids: List[int], on_rollback: Optional[Callable[["SpecTransaction"], None]] = None):
        self.rids = list(rids)
        self.stage = Stage.NEW
        self.trace: List[str] = [Stage.NEW.value]
        self.on_rollback = on_rollback
        self.mutated_target = False      # verify rows were written to KV / journals
        self.mutated_provider = False    # the drafter's own KV was written

    def advance(self, to: Stage) -> None:
        if self.stage in _TERMINAL:
            raise TransactionError(f"transaction already {self.stage.value}")
        if to in (Stage.ROLLED_BACK, Stage.CANCELLED):
            raise TransactionError("use rollback() / cancel()")
        if _ORDER.index(to) != _ORDER.index(self.stage) + 1:
            raise TransactionError(f"illegal transition {self.stage.value} -> {to.value}")
        self.stage = to
        self.trace.append(to.value)
        if to == Stage.PROVIDER_OPEN:
            self.mutated_provider = True
        if to == Stage.VERIFIED:
            self.mutated_target = True

    def _abort(self, to: Stage) -> None:
        if self.stage in _TERMINAL:
            raise TransactionError(f"transaction already {self.stage.value}")
        if self.stage == Stage.COMMITTING:
            raise TransactionError("a commit in flight cannot be rolled back")
        if self.on_rollback is not None and (self.mutated_target or self.mutated_provider):
            self.on_rollback(self)
        self.stage = to
        self.trace.append(to.value)

    def rollback(self) -> None:
        self._abort(Stage.ROLLED_BACK)

    def cancel(self) -> None:
        self._abort(Stage.CANCELLED)

    @property
    def done(self) -> bool:
        return self.stage in _TERMINAL
