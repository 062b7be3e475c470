"""Host sampler law, logit processors and seed mixing.

Order of operations matches the reference's host sampler (``hipengine/generation/sampling.py:868-1060``):
logit bias -> history penalties (repetition / presence / frequency) -> suppression -> EOS suppression while
``min_tokens`` is unmet -> constraint masks -> temperature / top-k / top-p / min-p -> seeded draw; greedy ties
go to the lowest token id (``:1733``).  Per-row seeds are a SplitMix-style mix of (seed, row index, request
id) (``:1082-1106``).  The device sampler (``csrc/sampling.cu``) implements the same filter law and the same
counter-based uniform, so a CPU run and a GPU run draw the same token from the same distribution.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch

MASK64 = (1 << 64) - 1


def splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def mix_seed(seed: Optional[int], row_index: int, request_id: int) -> int:
    """Deterministic per-row seed; ``None`` seeds still separate rows and requests.  The scheduler passes request id
    0 for an explicitly seeded request, so that the same seed repeats the same draws in another request."""
    base = 0x5DEECE66D if seed is None else int(seed) & MASK64
    return splitmix64(splitmix64(base ^ (row_index * 0x9E3779B97F4A7C15 & MASK64)) ^ (request_id & MASK64))


def uniform01(seed: int, counter: int) -> float:
    """Same construction as ``uniform01`` in csrc/sampling.cu."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


def apply_processors(logits: torch.Tensor, *, logit_bias: Sequence[Tuple[int, float]] = (),
                     history: Sequence[int] = (), prompt: Sequence[int] = (), repetition_penalty: float = 1.0,
                     presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                     suppress: Iterable[int] = (), allowed_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns processed logits (fp32 copy).  Works on CPU or CUDA tensors."""
    lg = logits.to(torch.float32).clone()
    V = lg.shape[-1]
    if logit_bias:
        idx = torch.tensor([t for t, _ in logit_bias if 0 <= t < V], dtype=torch.long, device=lg.device)
        val = torch.tensor([b for t, b in logit_bias if 0 <= t < V], dtype=torch.float32, device=lg.device)
        lg.index_add_(0, idx, val)
    if repetition_penalty != 1.0 and (history or prompt):
        seen = torch.tensor(sorted(set(history) | set(prompt)), dtype=torch.long, device=lg.device)
        seen = seen[(seen >= 0) & (seen < V)]
        v = lg[seen]
        lg[seen] = torch.where(v > 0, v / repetition_penalty, v * repetition_penalty)
    if (presence_penalty != 0.0 or frequency_penalty != 0.0) and history:
        h = torch.tensor([t for t in history if 0 <= t < V], dtype=torch.long, device=lg.device)
        counts = torch.bincount(h, minlength=V).to(torch.float32)
        lg -= frequency_penalty * counts
        lg -= presence_penalty * (counts > 0).to(torch.float32)
    sup = [t for t in suppress if 0 <= t < V]
    if sup:
        lg[torch.tensor(sup, dtype=torch.long, device=lg.device)] = float("-inf")
    if allowed_mask is not None:
        lg = torch.where(allowed_mask.to(lg.device), lg, torch.full_like(lg, float("-inf")))
    return lg


def filter_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                        min_p: float) -> torch.Tensor:
    """Probabilities after temperature / top-k / top-p / min-p (zeros outside the kept set)."""
    x = (logits.to(torch.float64) - logits.max().to(torch.float64)) / temperature
    e = torch.exp(x)
    V = e.numel()
    keep = torch.ones(V, dtype=torch.bool, device=e.device)
    thr = None
    if (0 < top_k < V) or (0.0 < top_p < 1.0):
        vals, _ = torch.sort(e, descending=True)
        cands = []
        if 0 < top_k < V:
            cands.append(vals[top_k - 1])
        if 0.0 < top_p < 1.0:
            cum = torch.cumsum(vals, 0)
            n = int(torch.searchsorted(cum, top_p * cum[-1]).item())
            cands.append(vals[min(n, V - 1)])
        thr = max(cands)
        keep &= e >= thr * (1 - 1e-9)
    if min_p > 0.0:
        keep &= e >= min_p * (1 - 1e-9)
    p = torch.where(keep, e, torch.zeros_like(e))
    return p / p.sum()


def sample_token(logits: torch.Tensor, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 min_p: float = 0.0, seed: int = 0, counter: int = 0) -> Tuple[int, float]:
    """Returns (token id, logprob under the processed distribution)."""
    if temperature <= 0.0:
        m = logits.max()
        tok = int(torch.nonzero(logits == m)[0].item())      # lowest id among ties
        return tok, 0.0
    p = filter_distribution(logits, temperature, top_k, top_p, min_p)
    u = uniform01(seed, counter)
    cum = torch.cumsum(p, 0)
    tok = int(torch.searchsorted(cum, torch.tensor(u, dtype=cum.dtype, device=cum.device), right=True).item())
    tok = min(tok, p.numel() - 1)
    while tok > 0 and p[tok] == 0:
        tok -= 1
    return tok, float(torch.log(p[tok]).item())


def top_logprobs(logits: torch.Tensor, n: int, temperature: float = 1.0) -> List[Tuple[int, float]]:
    t = temperature if temperature > 0 else 1.0
    lp = torch.log_softmax(logits.to(torch.float64) / t, -1)
    vals, idx = torch.topk(lp, min(n, lp.numel()))
    return [(int(i), float(v)) for i, v in zip(idx.tolist(), vals.tolist())]


def token_logprob(logits: torch.Tensor, token: int, temperature: float = 1.0) -> float:
    t = temperature if temperature > 0 else 1.0
    return float(torch.log_softmax(logits.to(torch.float64) / t, -1)[token].item())


def classify_sampler_mode(req) -> str:
    """greedy | sampled | processed: what a speculative verifier must reproduce (reference ``:1489``)."""
    return req.sampler_mode
