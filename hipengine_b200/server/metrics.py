"""Prometheus text exposition for the server (``--metrics prometheus``).

Series families mirror the reference's ``hipengine_*`` set (``hipengine/server/metrics.py:1-15``): requests,
tokens, queue depth, resident occupancy, KV pool pages / bytes, graph-bucket hits / misses / captures, MTP
accepted / rejected / acceptance rate, prefix-cache hits, latency percentiles.  Names use the ``he_`` prefix.
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

    def render(self, engine_snapshot: Dict[str, Any], capacity: Dict[str, Any], queue_depth: int = 0) -> str:
        lines: List[str] = []

        def emit(name: str, value: Any, typ: str = "gauge", help_: str = "", labels: str = "") -> None:
            if value is None:
                return
            if help_:
                lines.append(f"# HELP {name} {help_}")
            lines.append(f"# TYPE {name} {typ}")
            lines.append(f"{name}{labels} {float(value)}")

        emit("he_uptime_seconds", time.time() - self.started, help_="Seconds since server start")
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
        emit("he_requests_pending", engine_snapshot.get("pending"), help_="Requests waiting for admission")
        emit("he_requests_active", engine_snapshot.get("active"), help_="Resident requests")
        emit("he_resident_prefill_rows", engine_snapshot.get("prefill_rows"))
        emit("he_resident_decode_rows", engine_snapshot.get("decode_rows"))
        emit("he_http_queue_depth", queue_depth)
        for k in ("submitted", "admitted", "finished", "cancelled", "failed", "prefill_tokens", "decode_tokens",
                  "prefill_chunks", "decode_steps", "cached_prompt_tokens", "spec_cycles", "spec_drafted",
                  "spec_accepted"):
            emit(f"he_engine_{k}_total", c.get(k), "counter")
        drafted = c.get("spec_drafted", 0) or 0
        emit("he_mtp_acceptance_rate", (c.get("spec_accepted", 0) / drafted) if drafted else 0.0)
        emit("he_mtp_rejected_total", drafted - (c.get("spec_accepted", 0) or 0), "counter")
        lat = engine_snapshot.get("latency", {})
        for k in ("ttft_p50_ms", "ttft_p99_ms", "itl_p50_ms", "itl_p99_ms"):
            emit(f"he_latency_{k}", lat.get(k))
        pool = capacity.get("kv_pool", {})
        for k in ("pages_total", "pages_free", "pages_used", "pages_cached", "pages_credit", "leases", "grants",
                  "cow", "evictions", "peak_used"):
            emit(f"he_kv_pool_{k}", pool.get(k))
        if pool and capacity.get("kv_bytes_per_token"):
            emit("he_kv_pool_bytes_used", pool.get("pages_used", 0) * pool.get("page_tokens", 16)
                 * capacity["kv_bytes_per_token"])
        pref = capacity.get("prefix_cache", {})
        for k in ("nodes", "lookups", "hits", "hit_tokens", "inserted_pages", "evicted_pages"):
            emit(f"he_prefix_cache_{k}", pref.get(k))
        g = engine_snapshot.get("runner", {}).get("graphs", {})
        for k in ("hits", "misses", "captures"):
            emit(f"he_graph_bucket_{k}_total", g.get(k), "counter")
        emit("he_state_bytes", capacity.get("state_bytes"))
        emit("he_max_context_tokens", capacity.get("max_context"))
        emit("he_max_slots", capacity.get("max_slots"))
        return "\n".join(lines) + "\n"
