"""Server log formatting: one formatter (ANSI or plain), ``LOAD_TIMING`` rows for the start-up stages, and the
start-up summary printed once the engine is resident.

Counterpart of the reference's ``hipengine/server/log_style.py`` (ANSI formatter, ``LOAD_TIMING`` rows, start-up
summary).  Everything here builds strings; ``server/__main__.py`` installs the formatter and logs the rows.
"""
from __future__ import annotations

import logging
from typing import Any, Dict, Iterable, List, Optional

RESET, DIM, BOLD = "\033[0m", "\033[2m", "\033[1m"
LEVEL_COLOR = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m",
               "CRITICAL": "\033[1;31m"}


def want_color(mode: str, is_tty: bool) -> bool:
    """``--log-color always|never|auto``: ``auto`` colours only a terminal."""
    return mode == "always" or (mode == "auto" and is_tty)


class StyledFormatter(logging.Formatter):
    """``time LEVEL logger: message`` with the level coloured and time / logger dimmed when ``color`` is on."""

    def __init__(self, color: bool = False):
        super().__init__("%(asctime)s %(levelname)s %(name)s: %(message)s")
        self.color = color

    def format(self, record: logging.LogRecord) -> str:
        if not self.color:
            return super().format(record)
        msg = record.getMessage()
        if record.exc_info:
            msg += "\n" + self.formatException(record.exc_info)
        lv = record.levelname
        return (f"{DIM}{self.formatTime(record)}{RESET} {LEVEL_COLOR.get(lv, '')}{BOLD}{lv:<7}{RESET} "
                f"{DIM}{record.name}:{RESET} {msg}")


def install(level: str = "INFO", color: bool = False) -> None:
    """Route the root logger through one stream handler with the styled formatter (idempotent)."""
    root = logging.getLogger()
    for h in list(root.handlers):
        if getattr(h, "_he_styled", False):
            root.removeHandler(h)
    h = logging.StreamHandler()
    h.setFormatter(StyledFormatter(color))
    h._he_styled = True
    root.addHandler(h)
    root.setLevel(level)


def human_bytes(n: Optional[float]) -> str:
    if n is None:
        return "-"
    n = float(n)
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024.0 or unit == "TiB":
            return f"{n:.0f} {unit}" if unit == "B" else f"{n:.2f} {unit}"
        n /= 1024.0
    return f"{n:.2f} TiB"


def load_timing_rows(startup: Dict[str, Any]) -> List[str]:
    """One ``LOAD_TIMING`` row per start-up stage (name, seconds, share of the total, outcome) and a total row."""
    stages = list(startup.get("stages") or [])
    total = sum(float(s.get("seconds", 0.0)) for s in stages)
    rows = []
    for s in stages:
        sec = float(s.get("seconds", 0.0))
        share = 100.0 * sec / total if total > 0 else 0.0
        rows.append(f"LOAD_TIMING stage={s.get('name')} seconds={sec:.3f} share={share:.1f}% "
                    f"{'ok' if s.get('ok', True) else 'FAILED'}")
    rows.append(f"LOAD_TIMING total seconds={total:.3f} stages={len(stages)}"
                + (f" error={startup['error']}" if startup.get("error") else ""))
    return rows


def startup_summary(model: str, backend: str, capacity: Optional[Dict[str, Any]], startup: Dict[str, Any],
                    options: Optional[Dict[str, Any]] = None) -> List[str]:
    """The lines logged once when the engine is resident: what is served, from what memory, with which options."""
    cap = capacity or {}
    pool = cap.get("kv_pool") or {}
    spec = cap.get("speculative") or {}
    mem = startup.get("memory") or {}
    lines = [f"model {model} on {backend}",
             f"context up to {cap.get('max_context', '-')} tokens, {cap.get('max_slots', '-')} request slots"]
    if cap.get("weight_bytes"):
        lines.append(f"weights {human_bytes(cap['weight_bytes'])} resident (quantised blocks, read in place)")
    if pool.get("pages_total"):
        pages, ptok = int(pool["pages_total"]), int(pool.get("page_tokens", 16))
        lines.append(f"KV pool {pages} pages x {ptok} tokens"
                     f" ({human_bytes(cap.get('kv_bytes_per_token', 0) * ptok * pages)})")
    if spec:
        extra = f", draft head slice {spec['draft_head_rows']} rows" if spec.get("draft_head_rows") else ""
        lines.append(f"speculative provider {spec.get('provider')} depth {spec.get('max_depth')}"
                     f"{' (one graph per cycle)' if spec.get('graph_capture') else ''}{extra}")
    if mem:
        lines.append(f"device memory {human_bytes(mem.get('device_free_bytes'))} free of "
                     f"{human_bytes(mem.get('device_total_bytes'))}")
    for k, v in sorted((options or {}).items()):
        if v not in (None, "", "off", False, 0, 1):
            lines.append(f"option {k}={v}")
    lines.append("warm (start-up request went through)" if startup.get("warmup_complete")
                 else "not warmed up: the first request captures graphs and sizes scratch")
    return lines


def log_lines(log: logging.Logger, lines: Iterable[str], level: int = logging.INFO) -> None:
    for ln in lines:
        log.log(level, ln)
