"""Value types shared by drafters, verifiers and the engine loop.

Scope follows the reference's speculative contracts (``hipengine/speculative/contracts.py`` /
``interfaces.py``) reduced to what chain speculation needs: the capability a provider reports (shown by the
runner's capacity and the server's readiness document) and the result of one cycle.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class SpeculativeCapability:
    """What a runner can do: chain widths (requests per cycle), depths (draft tokens), transaction mode."""
    provider: str = "nextn_mtp"
    max_depth: int = 3
    widths: Tuple[int, ...] = (1, 2, 4, 8)
    attachment: str = "trailing_block"        # the drafter is the checkpoint's own NextN block
    transaction_mode: str = "journal"         # recurrent state is journalled per verify row and committed by copy
    sampling_modes: Tuple[str, ...] = ("greedy", "sampled")
    graph_capture: bool = False               # the whole cycle replays as one captured graph (greedy chains)
    draft_head_rows: int = 0                  # hot-vocabulary draft head: rows of the head slice (0: full head only)

    def as_dict(self) -> Dict[str, Any]:
        return {"provider": self.provider, "max_depth": self.max_depth, "widths": list(self.widths),
                "attachment": self.attachment, "transaction_mode": self.transaction_mode,
                "sampling_modes": list(self.sampling_modes), "graph_capture": self.graph_capture,
                "draft_head_rows": self.draft_head_rows}


@dataclass
class SpecCycleResult:
    tokens: List[int] = field(default_factory=list)
    drafted: int = 0
    accepted: int = 0
    stage_trace: Optional[List[str]] = None
