"""Exact speculative sampling on the host (oracle for ``csrc/spec.cu`` and fallback for processed rows).

The law is the one the reference implements in ``hipengine/speculative/sampling.py:135-339``: a draft token d
drawn from q is accepted with probability ``min(1, p(d)/q(d))``; on rejection the replacement is drawn from
``normalize(max(0, p - q))``; after K acceptances a bonus token is drawn from the last target distribution.
The emitted sequence is then distributed exactly as ancestral sampling from the target.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def acceptance_probability(p: torch.Tensor, q: torch.Tensor, token: int) -> float:
    qd = float(q[token])
    if qd <= 0.0:
        return 1.0 if float(p[token]) > 0.0 else 0.0
    return min(1.0, float(p[token]) / qd)


def residual_distribution(p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    r = (p.double() - q.double()).clamp(min=0)
    s = r.sum()
    if s <= 0:
        return p.double() / p.double().sum()
    return r / s


def greedy_accept(draft: Sequence[int], target_argmax: Sequence[int]) -> Tuple[int, List[int]]:
    """Chain accept for greedy decoding: (accepted, emitted tokens = accepted drafts + bonus)."""
    n = 0
    while n < len(draft) and draft[n] == target_argmax[n]:
        n += 1
    return n, list(draft[:n]) + [int(target_argmax[n])]


def sampled_accept_from_distributions(draft: Sequence[int], p_rows: torch.Tensor, q_rows: Optional[torch.Tensor],
                                      uniforms: Sequence[float]) -> Tuple[int, List[int]]:
    """p_rows [K+1, V] target probabilities, q_rows [K, V] draft probabilities (None: greedy draft, a point mass).
    ``uniforms`` supplies 2 numbers per chain position (accept test, replacement draw)."""
    K = len(draft)
    out: List[int] = []
    for i in range(K + 1):
        p = p_rows[i].double()
        if i < K:
            d = int(draft[i])
            q = q_rows[i].double() if q_rows is not None else torch.zeros_like(p).index_fill_(0, torch.tensor([d]), 1.0)
            if uniforms[2 * i] <= acceptance_probability(p, q, d):
                out.append(d)
                continue
            w = residual_distribution(p, q)
        else:
            w = p / p.sum()
        c = torch.cumsum(w, 0)
        x = uniforms[2 * i + 1] * float(c[-1])
        tok = int(torch.searchsorted(c, torch.tensor([x], dtype=c.dtype)).clamp(max=p.numel() - 1))
        out.append(tok)
        return len(out) - 1, out
    raise AssertionError("unreachable")
