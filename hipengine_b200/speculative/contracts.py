"""Value types shared by drafters, verifiers and the engine loop.

Scope follows the reference's speculative contracts (``hipengine/speculative/contracts.py`` /
``interfaces.py``: capability, request plan, candidate graph rows, accept result) reduced to chain candidates,
the only shape the NextN/MTP drafter produces.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple


@dataclass(frozen=True)
class SpeculativeCapability:
    """What a runner can do: chain widths (requests per cycle), depths (draft tokens), transaction mode."""
    provider: str = "nextn_mtp"
    max_depth: int = 3
    widths: Tuple[int, ...] = (1, 2, 4, 8)
    attachment: str = "trailing_block"        # the drafter is the checkpoint's own NextN block
    transaction_mode: str = "journal"         # recurrent state is journalled per verify row and committed by copy
    sampling_modes: Tuple[str, ...] = ("greedy", "sampled")


@dataclass
class SpecRequestPlan:
    rid: int
    depth: int                  # K draft tokens this cycle
    start_position: int         # position of the chain's first token (the last committed one)
    sampling_mode: str          # greedy | sampled
    max_emit: int               # tokens the request may still emit


@dataclass
class CandidateChain:
    """One request's verify rows: ``tokens[0]`` is committed, ``tokens[1:]`` are drafts."""
    rid: int
    tokens: List[int]
    positions: List[int]

    @property
    def depth(self) -> int:
        return len(self.tokens) - 1


@dataclass
class AcceptResult:
    accepted: int               # drafts accepted (0..K)
    emitted: List[int]          # accepted drafts + the bonus token
    commit_row: int             # verify row whose recurrent state becomes live


@dataclass
class SpecCycleResult:
    tokens: List[int] = field(default_factory=list)
    drafted: int = 0
    accepted: int = 0
    stage_trace: Optional[List[str]] = None
