"""The readiness document of ``GET /ready``.

One JSON object that tells an operator (or a load balancer) whether the process can serve and why not: engine
service health, what is loaded, how start-up went (stages with their durations, checks, device memory), context
and KV capacity, what the KV path is capable of, prefix-cache and graph-cache state, queue and batcher, sessions,
parallel layout, speculative capability.  Field layout follows the reference's readiness payload
(``hipengine/server/readiness.py:89-217``); HTTP status is 200 when ``ready`` else 503.
"""
from __future__ import annotations

import time
from typing import Any, Dict, Mapping, Optional


def kv_capability(cfg, kv_cfg) -> Dict[str, Any]:
    """What the KV path of this build supports for the loaded geometry, with the evidence it rests on (the tests that
    compare each path with fp32 PyTorch).  The reference ships such a record per storage mode
    (``hipengine/kvcache/capabilities.py``)."""
    hd = int(getattr(cfg, "head_dim", 0) or 0)
    return {
        "storage": {"bf16": {"supported": True, "evidence": "tests/test_gpu_kernels.py (paged write + decode), "
                                                             "tests/test_gpu_executor.py (end to end vs fp32)"},
                    "int8": {"supported": False, "granularity": "per_token_head", "scale_dtype": "float16",
                             "reason": "no int8 writer / reader kernels for sm_100a in this build; the format is "
                                       "defined by ref/ops.py::kv_int8_quantize and served by the cpu_reference "
                                       "backend only"}},
        "selected_storage": getattr(kv_cfg, "storage", "bf16"),
        "page_tokens": int(getattr(kv_cfg, "page_tokens", 16)),
        "layout": "[pages][k|v][kv_heads][page_tokens][head_dim] bf16, block table per slot",
        "head_dim": hd,
        "decode_kernel": "tensor-core split-K (mma.sync over the query heads of a KV group)" if hd >= 128
                         else "CUDA-core split-K",
        "prefill_kernel": "flash (mma.sync)" if hd in (64, 128, 256) else "row-wise decode kernel",
        "prefix_cache": getattr(kv_cfg, "prefix_cache", "off"),
        "recurrent_state_snapshots": bool(getattr(cfg, "is_hybrid", False)),
        "sliding_window": bool(getattr(cfg, "sliding_window", 0)),
        "cold_tier": True,
    }


def build_readiness(*, model_id: str, health: Mapping[str, Any], startup: Mapping[str, Any],
                    capacity: Optional[Mapping[str, Any]], live: Optional[Mapping[str, Any]], config, server_cfg,
                    gate, sessions: Optional[Mapping[str, Any]], started: float,
                    model_cfg=None, error: Optional[str] = None) -> Dict[str, Any]:
    healthy = bool(health.get("healthy", True))
    loaded = bool(startup.get("model_loaded"))
    diagnostics = []
    if not healthy:
        diagnostics.append({"code": "engine_unhealthy", "detail": health.get("unhealthy") or "engine service closed"})
    if error:
        diagnostics.append({"code": "capacity_probe_failed", "detail": error})
    if startup.get("error"):
        diagnostics.append({"code": "startup_failed", "detail": startup["error"]})
    ready = healthy and not error and not startup.get("error")
    cap = dict(capacity or {})
    graphs = dict(((live or {}).get("runner") or live or {}).get("graphs") or {})
    hits, misses = int(graphs.get("hits", 0)), int(graphs.get("misses", 0))
    body: Dict[str, Any] = {
        "object": "hipengine.readiness",
        "status": "ready" if ready else "not_ready",
        "ready": ready,
        "diagnostics": diagnostics,
        "engine_service": dict(health),
        "engine": dict(health),
        "model": {"id": model_id, "loaded": loaded, "loaded_model_count": 1 if loaded else 0,
                  "weight_bytes": cap.get("weight_bytes"),
                  "kv_capability": kv_capability(model_cfg, config.kv) if model_cfg is not None else {}},
        "startup": {"eager_load": bool(startup.get("eager_load")),
                    "warmup_complete": bool(startup.get("warmup_complete")),
                    "stages": list(startup.get("stages", [])),
                    "last_timings_s": dict(startup.get("timings_s", {})),
                    "checks": dict(startup.get("checks", {})),
                    "memory": dict(startup.get("memory", {})),
                    "error": startup.get("error")},
        "context": {"configured_max_context_tokens": config.max_sequence_length,
                    "effective_max_context_tokens": cap.get("max_context"),
                    "max_context_tokens": cap.get("max_context"),
                    "chat_default_max_tokens": server_cfg.chat_default_max_tokens},
        "kv_capacity": {"storage": config.kv.storage, "pool": cap.get("kv_pool"),
                        "prefix_cache": cap.get("prefix_cache"),
                        "estimate": {"kv_bytes_per_token": cap.get("kv_bytes_per_token"),
                                     "recurrent_state_bytes_per_request": cap.get("recurrent_state_bytes_per_request"),
                                     "state_bytes": cap.get("state_bytes")}},
        "prefix_cache": cap.get("prefix_cache") or {},
        "resources": cap.get("resources") or {},
        "graph_cache": {"entries": int(graphs.get("captures", 0)), "hits": hits, "misses": misses,
                        "replay_hit_rate": (hits / (hits + misses)) if hits + misses else None,
                        "native_launches": graphs.get("native_launches")},
        "device": {"backend": cap.get("backend")},
        "queue": {"in_flight": gate.in_flight, "limit": gate.limit, "depth": gate.in_flight,
                  "max_depth": server_cfg.max_queued_requests,
                  "max_active_requests": config.scheduler.max_active_requests,
                  "batch_window_ms": float(getattr(server_cfg, "batch_window_ms", 0.0))},
        "batcher": gate.snapshot(),
        "sessions": dict(sessions or {}),
        "parallelism": {"world_size": config.parallel.tp * config.parallel.ep,
                        "tensor_parallel": config.parallel.tp, "expert_parallel": config.parallel.ep},
        "speculative": cap.get("speculative"),
        "uptime_seconds": time.time() - started,
    }
    if not ready:
        body["reason"] = "; ".join(str(d.get("detail")) for d in diagnostics if d.get("detail")) or "not ready"
    return body
