"""Typed engine configuration.

The reference spreads configuration over constructor kwargs, ~500 ``HIPENGINE_*``
environment variables and per-backend capability tables (``docs/ENVS.md``,
``hipengine/execution_profiles.py:26-136``).  Here there is one dataclass tree
plus a handful of ``HE_*`` environment overrides; execution profiles keep their
public names but select numerics policy only (there is a single kernel per op).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from enum import Enum
from typing import Any, Optional


class ExecutionProfile(str, Enum):
    """Public profile names of the reference (``hipengine/execution_profiles.py:26-33``)."""
    STRICT = "strict"                    # fp32 residual stream, deterministic reductions (the default here)
    PRODUCTION = "production"
    BATCH_INVARIANT = "batch_invariant"  # decode rows never share a reduction order with their neighbours
    FAST = "fast"

    @classmethod
    def parse(cls, v) -> "ExecutionProfile":
        if isinstance(v, cls):
            return v
        if v is None:
            return cls.PRODUCTION
        return cls(str(v).lower())


@dataclass(frozen=True)
class SchedulerConfig:
    """Mirrors ``EngineLoopConfig`` (``hipengine/generation/engine_loop.py:155-213``) with this engine's defaults."""
    policy: str = "protect_decode"          # protect_decode | protect_ttft | fair | token_budget
    max_prefill_chunk_tokens: int = 4096
    round_prefill_token_budget: int = 4096
    round_decode_row_budget: int = 64
    fair_prefill_burst_chunks: int = 1
    max_pending_requests: int = 1024
    max_active_requests: int = 8
    stream_mailbox: int = 64


@dataclass(frozen=True)
class KVConfig:
    page_tokens: int = 16
    storage: str = "bf16"                   # bf16 | int8 (per token/head scales)
    pool_pages: Optional[int] = None        # None: sized from free memory
    memory_reserve_mib: int = 3072          # never admit below this free-memory floor
    pool_budget_mib: Optional[int] = None   # size the page pool from a memory budget (pool_pages wins when both are set)
    prefix_cache: str = "radix"             # off | radix
    snapshot_interval_tokens: int = 2048    # hybrid recurrent-state snapshot cadence for prefix reuse
    max_snapshots: int = 16
    cold_tier_bytes: int = 0                # > 0: evicted prefix blocks go to a host / disk tier (``kvcache/tiering.py``)
    cold_tier_dir: Optional[str] = None     # None: host memory; a path: one file per object
    cold_restore_prefill_tok_s: float = 16000.0   # recompute rate the restore economics compare against


def resolve_pool_pages(kv: "KVConfig", kv_bytes_per_token: int, n_slots: int, pages_per_slot: int) -> int:
    """Pages of the KV pool: an explicit count wins, then a memory budget, else every slot at full context (twice
    that with the prefix cache on, so cached prefixes do not starve admissions) plus the null page."""
    if kv.pool_pages:
        return int(kv.pool_pages)
    if kv.pool_budget_mib and kv_bytes_per_token > 0:
        return max(2, int(kv.pool_budget_mib * (1 << 20) // (kv.page_tokens * kv_bytes_per_token)) + 1)
    return n_slots * pages_per_slot * (2 if kv.prefix_cache != "off" else 1) + 1


@dataclass(frozen=True)
class SpeculativeConfig:
    mode: str = "off"                       # off | mtp | prompt_lookup | ngram (``speculative/providers.py``)
    draft_depth: int = 3
    adaptive_depth: bool = True             # shrink the draft depth to what the measured acceptance rate pays for
    hot_vocab: str = "off"                  # NextN draft head slice: off | auto | row count (``speculative/draft_vocab.py``)
    draft_model: Any = None                 # Gemma 4: the assistant (MTP) head artifact (path, loaded weights or "random")


@dataclass(frozen=True)
class ParallelConfig:
    tp: int = 1
    ep: int = 1
    fused_collectives: bool = True          # in-kernel P2P/NVLS paths; False = NCCL-only baseline


@dataclass(frozen=True)
class EngineConfig:
    max_sequence_length: int = 8192
    profile: ExecutionProfile = ExecutionProfile.PRODUCTION
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    kv: KVConfig = field(default_factory=KVConfig)
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    use_cuda_graphs: bool = True
    command_timeout_seconds: float = 300.0

    @staticmethod
    def from_env(base: Optional["EngineConfig"] = None) -> "EngineConfig":
        cfg = base or EngineConfig()
        e = os.environ
        if "HE_MAX_SEQ" in e:
            cfg = replace(cfg, max_sequence_length=int(e["HE_MAX_SEQ"]))
        if "HE_CUDA_GRAPHS" in e:
            cfg = replace(cfg, use_cuda_graphs=e["HE_CUDA_GRAPHS"] not in ("0", "false", "off"))
        if "HE_PREFILL_CHUNK" in e:
            cfg = replace(cfg, scheduler=replace(cfg.scheduler, max_prefill_chunk_tokens=int(e["HE_PREFILL_CHUNK"])))
        if "HE_SCHED_POLICY" in e:
            cfg = replace(cfg, scheduler=replace(cfg.scheduler, policy=e["HE_SCHED_POLICY"]))
        if "HE_PREFIX_CACHE" in e:
            cfg = replace(cfg, kv=replace(cfg.kv, prefix_cache=e["HE_PREFIX_CACHE"]))
        if "HE_COMMAND_TIMEOUT" in e:
            cfg = replace(cfg, command_timeout_seconds=float(e["HE_COMMAND_TIMEOUT"]))
        return cfg
