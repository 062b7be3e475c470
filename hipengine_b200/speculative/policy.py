"""Draft-depth planner (pre-mutation, deterministic), after ``hipengine/speculative/policy.py:181-480``.

Depth is the smaller of the configured budget, what the request may still emit, the room left in its context,
and -- once enough cycles have been observed -- the depth that the measured acceptance rate makes worthwhile:
a draft pass and every extra verify row cost a measured fraction of a target step, and depth k pays off only
while the expected number of tokens per unit cost keeps rising (``adaptive=False`` keeps the hard limits only).
"""
from __future__ import annotations


def expected_tokens(accept_rate: float, depth: int) -> float:
    """Expected tokens emitted by a chain of ``depth`` drafts with i.i.d. acceptance ``accept_rate`` (bonus included)."""
    a = min(max(accept_rate, 0.0), 1.0)
    return sum(a ** i for i in range(depth + 1))


# Costs in units of one autoregressive step, measured on the 27B hybrid on one B200 (packed decode step by rows:
# 5.42 / 7.03 / 8.70 / 10.32 ms at 1 / 2 / 3 / 4 rows; a depth-3 cycle 13.0 ms): every verify row beyond the first
# adds ~0.30 of a step, every draft pass of the NextN block ~0.14.
DRAFT_COST = 0.14
VERIFY_ROW_COST = 0.30


def cycle_cost(depth: int, draft_cost: float = DRAFT_COST, verify_row_cost: float = VERIFY_ROW_COST) -> float:
    """Cost of one cycle of ``depth`` drafts in autoregressive steps (depth 3 -> 2.32; measured 2.33)."""
    return 1.0 + depth * (draft_cost + verify_row_cost)


def break_even_accept_rate(depth: int, draft_cost: float = DRAFT_COST, verify_row_cost: float = VERIFY_ROW_COST) -> float:
    """Smallest i.i.d. acceptance rate at which a chain of ``depth`` drafts emits more tokens per unit cost than
    plain decoding (bisection on ``expected_tokens(a, depth) = cycle_cost(depth)``)."""
    target = cycle_cost(depth, draft_cost, verify_row_cost)
    if expected_tokens(1.0, depth) <= target:
        return 1.0
    lo, hi = 0.0, 1.0
    for _ in range(40):
        mid = 0.5 * (lo + hi)
        if expected_tokens(mid, depth) < target:
            lo = mid
        else:
            hi = mid
    return hi


def plan_draft_depth(budget: int, remaining_tokens: int, context_room: int, drafted: int = 0, accepted: int = 0,
                     draft_cost: float = DRAFT_COST, verify_row_cost: float = VERIFY_ROW_COST,
                     min_observations: int = 64, adaptive: bool = True) -> int:
    hard = max(0, min(budget, remaining_tokens - 1, context_room - 1))
    if hard <= 1 or drafted < min_observations or not adaptive:
        return hard
    rate = accepted / max(drafted, 1)
    best_k, best_v = 0, 1.0
    for k in range(1, hard + 1):
        cost = 1.0 + k * (draft_cost + verify_row_cost)
        v = expected_tokens(rate, k) / cost
        if v > best_v:
            best_k, best_v = k, v
    return best_k
