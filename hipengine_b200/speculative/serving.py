"""Serving admission for MTP: decide per request whether the speculative path may be used.

The reference resolves this from a (backend, KV storage, sampling mode, batch width) key against recorded
evidence (``hipengine/speculative/serving.py:779`` ``resolve_speculative_mtp_serving_plan``); here the rules are
stated directly, since one backend and one kernel set exist:
  * the checkpoint must carry a NextN block and the runner must report ``supports_mtp``;
  * mode ``off`` never, ``on`` whenever legal, ``auto`` only when the circuit breaker for the scope is closed;
  * greedy and plain sampled requests are legal; requests with logit processors, forced tokens, grammar or
    logprobs run autoregressively (their sampler law is not reproduced by the device verifier).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class MTPServingDecision:
    use_mtp: bool
    reason: str
    sampling_mode: Optional[str] = None
    depth: int = 0


def resolve_mtp_serving_plan(mode: str, supports_mtp: bool, temperature: float, processed: bool, forced: bool,
                             logprobs: bool, breaker_open: bool = False, depth: int = 3,
                             requested: bool = True) -> MTPServingDecision:
    if mode == "off" or not requested:
        return MTPServingDecision(False, "disabled")
    if not supports_mtp:
        return MTPServingDecision(False, "no_nextn_block")
    if processed or forced or logprobs:
        return MTPServingDecision(False, "sampler_not_reproducible")
    if mode == "auto" and breaker_open:
        return MTPServingDecision(False, "circuit_open")
    return MTPServingDecision(True, "ok", "greedy" if temperature == 0.0 else "sampled", depth)
