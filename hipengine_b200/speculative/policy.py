"""Draft-depth planner (pre-mutation, deterministic), after ``hipengine/speculative/policy.py:181-480``.

Depth is the smaller of the configured budget, what the request may still emit, the room left in its context,
and -- once enough cycles have been observed -- the depth that the measured acceptance rate makes worthwhile:
a draft step costs ``draft_cost`` of a target step, and depth k pays off only while the expected number of
tokens per unit cost keeps rising.
"""
from __future__ import annotations


def expected_tokens(accept_rate: float, depth: int) -> float:
    """Expected tokens emitted by a chain of ``depth`` drafts with i.i.d. acceptance ``accept_rate`` (bonus included)."""
    a = min(max(accept_rate, 0.0), 1.0)
    return sum(a ** i for i in range(depth + 1))


def plan_draft_depth(budget: int, remaining_tokens: int, context_room: int, drafted: int = 0, accepted: int = 0,
                     draft_cost: float = 0.08, verify_row_cost: float = 0.02, min_observations: int = 64) -> int:
    hard = max(0, min(budget, remaining_tokens - 1, context_room - 1))
    if hard <= 1 or drafted < min_observations:
        return hard
    rate = accepted / max(drafted, 1)
    best_k, best_v = 0, 1.0
    for k in range(1, hard + 1):
        cost = 1.0 + k * (draft_cost + verify_row_cost)
        v = expected_tokens(rate, k) / cost
        if v > best_v:
            best_k, best_v = k, v
    return best_k
