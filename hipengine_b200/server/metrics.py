"""Prometheus text exposition for the server (``--metrics prometheus``).

Series families mirror the reference's ``hipengine_*`` set (``hipengine/server/metrics.py:1-15``): requests,
tokens, queue depth, resident occupancy, KV pool pages / bytes, graph-bucket hits / misses / captures, MTP
accepted / rejected / acceptance rate, prefix-cache hits, latency percentiles, under the reference's names where a
series has a counterpart there.
"""
from __future__ import annotations

import threading
import time
from typing import Any, Dict, List, Tuple


class ServerMetrics:
    def __init__(self) -> None:
        self.lock = threading.Lock()
        self.counters: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], float] = {}
        self.started = time.time()

    def inc(self, name: str, value: float = 1.0, **labels: str) -> None:
        key = (name, tuple(sorted(labels.items())))
        with self.lock:
            self.counters[key] = self.counters.get(key, 0.0) + value

    def get(self, name: str, **labels: str) -> float:
        return self.counters.get((name, tuple(sorted(labels.items()))), 0.0)

    def render(self, engine_snapshot: Dict[str, Any], capacity: Dict[str, Any], queue_depth: int = 0,
               batcher: Dict[str, Any] = None) -> str:
        lines: List[str] = []

        def emit(name: str, value: Any, typ: str = "gauge", help_: str = "", labels: str = "") -> None:
            if value is None:
                return
            if help_:
                lines.append(f"# HELP {name} {help_}")
            lines.append(f"# TYPE {name} {typ}")
            lines.append(f"{name}{labels} {float(value)}")

        emit("hipengine_uptime_seconds", time.time() - self.started, help_="Seconds since server start")
        with self.lock:
            items = sorted(self.counters.items())
        seen = set()
        for (name, labels), v in items:
            if name not in seen:
                lines.append(f"# TYPE {name} counter")
                seen.add(name)
            lab = "{" + ",".join(f'{k}="{val}"' for k, val in labels) + "}" if labels else ""
            lines.append(f"{name}{lab} {v}")
        c = engine_snapshot.get("counters", {})
        b = batcher or {}
        # request / queue families
        emit("hipengine_generation_queue_depth", queue_depth, help_="HTTP requests admitted and not yet finished")
        emit("hipengine_generation_queue_max_depth", b.get("limit"))
        emit("hipengine_generation_batches_total", b.get("batches"), "counter")
        emit("hipengine_generation_batch_max_size", b.get("max_batch_seen"))
        emit("hipengine_generation_batch_window_wait_seconds_total", b.get("window_wait_seconds"), "counter")
        emit("hipengine_request_rejected_total", b.get("rejected_busy"), "counter")
        emit("hipengine_request_completed_total", c.get("finished"), "counter")
        emit("hipengine_request_cancelled_total", c.get("cancelled"), "counter")
        emit("hipengine_request_failed_total", c.get("failed"), "counter")
        emit("hipengine_prompt_tokens_total", c.get("prefill_tokens"), "counter")
        emit("hipengine_completion_tokens_total", c.get("decode_tokens"), "counter")
        emit("hipengine_resident_requests_pending", engine_snapshot.get("pending"),
             help_="Requests waiting for admission")
        emit("hipengine_resident_requests_active", engine_snapshot.get("active"), help_="Resident requests")
        emit("hipengine_resident_requests_admitted_total", c.get("admitted"), "counter")
        emit("hipengine_resident_work_prefill_total", c.get("prefill_chunks"), "counter")
        emit("hipengine_resident_work_decode_total", c.get("decode_steps"), "counter")
        emit("hipengine_resident_prefill_rows", engine_snapshot.get("prefill_rows"))
        emit("hipengine_resident_decode_rows", engine_snapshot.get("decode_rows"))
        slots = capacity.get("max_slots")
        act = engine_snapshot.get("active")
        emit("hipengine_resident_bucket_capacity", slots)
        if slots and act is not None:
            emit("hipengine_resident_bucket_occupied_slots", act)
            emit("hipengine_resident_bucket_free_slots", max(0, slots - act))
            emit("hipengine_resident_bucket_occupancy_ratio", act / slots)
        emit("hipengine_generation_scheduler_fairness_policy_info", 1,
             labels='{policy="%s"}' % engine_snapshot.get("policy", ""))
        for k in ("submitted", "cached_prompt_tokens", "spec_cycles"):
            emit(f"hipengine_engine_{k}_total", c.get(k), "counter")
        # speculative decoding
        drafted = c.get("spec_drafted", 0) or 0
        accepted = c.get("spec_accepted", 0) or 0
        emit("hipengine_mtp_draft_tokens_accepted_total", accepted, "counter")
        emit("hipengine_mtp_draft_tokens_rejected_total", drafted - accepted, "counter")
        emit("hipengine_mtp_draft_acceptance_rate", (accepted / drafted) if drafted else 0.0)
        emit("hipengine_mtp_requests_total", c.get("spec_cycles"), "counter")
        lat = engine_snapshot.get("latency", {})
        for k in ("ttft_p50_ms", "ttft_p99_ms", "itl_p50_ms", "itl_p99_ms"):
            v = lat.get(k)
            emit("hipengine_resident_request_latency_seconds", None if v is None else v / 1e3,
                 labels='{quantile="%s"}' % k[:-3])
        # KV pool / prefix cache
        pool = capacity.get("kv_pool", {})
        bpt = capacity.get("kv_bytes_per_token") or 0
        page_bytes = pool.get("page_tokens", 16) * bpt
        emit("hipengine_kv_pool_max_pages", pool.get("pages_total"))
        emit("hipengine_kv_pool_free_pages", pool.get("pages_free"))
        emit("hipengine_kv_pool_current_pages", pool.get("pages_used"))
        emit("hipengine_kv_pool_refcounted_pages", pool.get("pages_cached"))
        emit("hipengine_kv_pool_high_water_observed_pages", pool.get("peak_used"))
        if page_bytes:
            emit("hipengine_kv_pool_budget_bytes", (pool.get("pages_total") or 0) * page_bytes)
            emit("hipengine_kv_pool_current_bytes", (pool.get("pages_used") or 0) * page_bytes)
            emit("hipengine_kv_pool_high_water_observed_bytes", (pool.get("peak_used") or 0) * page_bytes)
            emit("hipengine_resident_kv_total_bytes", (pool.get("pages_total") or 0) * page_bytes)
        for k in ("pages_credit", "leases", "grants", "truncated", "evictions"):
            emit(f"hipengine_kv_pool_{k}", pool.get(k))
        pref = capacity.get("prefix_cache", {})
        for k in ("nodes", "lookups", "hits", "hit_tokens", "inserted_pages", "evicted_pages"):
            emit(f"hipengine_prefix_cache_{k}", pref.get(k))
        # decode graphs
        g = engine_snapshot.get("runner", {}).get("graphs", {})
        for k in ("hits", "misses", "captures"):
            emit(f"hipengine_graph_bucket_{k}_total", g.get(k), "counter")
        hits, misses = g.get("hits") or 0, g.get("misses") or 0
        if hits + misses:
            emit("hipengine_graph_bucket_replay_hit_rate", hits / (hits + misses))
        emit("hipengine_graph_bucket_entries", g.get("captures"))
        emit("hipengine_state_bytes", capacity.get("state_bytes"))
        emit("hipengine_max_context_tokens", capacity.get("max_context"))
        emit("hipengine_weight_bytes", capacity.get("weight_bytes"))
        return "\n".join(lines) + "\n"
