"""``python -m hipengine_b200.server`` / ``hipengine-b200 serve``: start the OpenAI-compatible server.

Flag surface follows the reference's server and engine-loop flags (``hipengine/server/__main__.py:139-490``,
``hipengine/generation/engine_loop.py:2099-2215``), reduced to the knobs this engine has.
"""
from __future__ import annotations

import argparse
import logging
import sys
from dataclasses import replace
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="hipengine-b200 serve", description="OpenAI-compatible server on sm_100a")
    ap.add_argument("--model", required=True, help="GGUF file / directory, or a built-in random-init geometry name")
    ap.add_argument("--backend", default="auto", choices=["auto", "cuda_sm100a", "cpu_reference"])
    ap.add_argument("--execution-profile", default="production", choices=["strict", "production", "batch_invariant", "fast"])
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--log-level", default="info")
    ap.add_argument("--eager-load", action="store_true", help="load weights and reserve KV before accepting traffic")
    ap.add_argument("--startup-chat-smoke", action="store_true", help="run one tiny chat request at startup")
    ap.add_argument("--max-context-tokens", type=int, default=8192)
    ap.add_argument("--max-active-requests", type=int, default=8)
    ap.add_argument("--max-queued-requests", type=int, default=256)
    ap.add_argument("--max-pending-requests", type=int, default=1024)
    ap.add_argument("--max-chat-sessions", type=int, default=256)
    ap.add_argument("--chat-default-max-tokens", type=int, default=4096)
    ap.add_argument("--request-timeout-ms", type=int, default=None)
    ap.add_argument("--stream-queue-max-chunks", type=int, default=16)
    ap.add_argument("--shutdown-grace-seconds", type=float, default=5.0)
    ap.add_argument("--batch-window-ms", "--generation-batch-window-ms", dest="batch_window_ms", type=float,
                    default=0.0, help="hold compatible requests up to this long so that they enter the engine together")
    ap.add_argument("--max-batch-size", type=int, default=64, help="release a held group early at this size")
    ap.add_argument("--kv-storage", default="bf16", choices=["bf16", "int8"],
                    help="int8 (per token and head, fp16 scales) is served by the cpu_reference backend only")
    ap.add_argument("--kv-pool-pages", "--kv-pool-initial-pages", dest="kv_pool_pages", type=int, default=None)
    ap.add_argument("--kv-pool-memory-budget-mib", type=int, default=None,
                    help="size the KV page pool from a memory budget instead of a page count")
    ap.add_argument("--startup-min-free-mib", type=int, default=None,
                    help="refuse to start unless this much device memory stays free after weights, KV pool and state")
    ap.add_argument("--eager-load-prompt", default="ping", help="prompt of the start-up smoke request")
    ap.add_argument("--eager-load-max-tokens", type=int, default=4)
    ap.add_argument("--replay-dir", default=None, help="write every admitted request as a JSON line into this directory")
    ap.add_argument("--replay-redaction", default="hash", choices=["none", "hash", "drop"])
    ap.add_argument("--quant", default=None, help="expected dominant block type of the checkpoint (e.g. Q4_K); a "
                                                  "mismatch is refused by the artifact admission")
    ap.add_argument("--debug", action="store_true", help="log level debug")
    ap.add_argument("--log-color", default="auto", choices=["auto", "always", "never"])
    ap.add_argument("--prefix-cache", default="radix", choices=["off", "radix"])
    ap.add_argument("--prefix-snapshot-interval", type=int, default=2048)
    ap.add_argument("--prefix-max-snapshots", type=int, default=16)
    ap.add_argument("--prefill-decode-policy", default="protect_decode",
                    choices=["protect_decode", "protect_ttft", "fair", "token_budget"])
    ap.add_argument("--max-prefill-chunk-tokens", type=int, default=4096)
    ap.add_argument("--round-prefill-token-budget", type=int, default=4096)
    ap.add_argument("--round-decode-row-budget", type=int, default=64)
    ap.add_argument("--fair-prefill-burst-chunks", type=int, default=1)
    ap.add_argument("--speculative-mtp-serving", default="off", choices=["off", "auto", "on"])
    ap.add_argument("--speculative-candidate-budget", type=int, default=3)
    ap.add_argument("--speculative-provider", default="mtp", choices=["mtp", "gemma4_mtp", "prompt_lookup", "ngram"])
    ap.add_argument("--draft-model", default=None,
                    help="Gemma 4: path of the assistant (MTP) head GGUF (general.architecture gemma4-assistant), or "
                         "'random' for a random-init head of the matching geometry")
    ap.add_argument("--mtp-hot-vocab", default="off",
                    help="NextN draft head slice: off | auto (98304 rows) | row count; verification keeps the full head")
    ap.add_argument("--kv-cold-tier-gib", type=float, default=0.0,
                    help="keep evicted prefix blocks in a compressed host/disk tier of this size (0 = off)")
    ap.add_argument("--kv-cold-tier-dir", default=None, help="directory for cold-tier objects (default: host memory)")
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--expert-parallel", type=int, default=1)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--metrics", default=None, choices=["prometheus"])
    ap.add_argument("--info", action="store_true", help="print the resolved configuration and exit")
    return ap


def configs_from_args(a):
    from ..config import EngineConfig, KVConfig, SchedulerConfig
    from .api import ServerConfig
    eng = EngineConfig(
        max_sequence_length=a.max_context_tokens, use_cuda_graphs=not a.no_cuda_graphs,
        scheduler=SchedulerConfig(policy=a.prefill_decode_policy, max_prefill_chunk_tokens=a.max_prefill_chunk_tokens,
                                  round_prefill_token_budget=a.round_prefill_token_budget,
                                  round_decode_row_budget=a.round_decode_row_budget,
                                  fair_prefill_burst_chunks=a.fair_prefill_burst_chunks,
                                  max_pending_requests=a.max_pending_requests,
                                  max_active_requests=a.max_active_requests,
                                  stream_mailbox=max(16, a.stream_queue_max_chunks * 4)),
        kv=KVConfig(storage=a.kv_storage, pool_pages=a.kv_pool_pages, prefix_cache=a.prefix_cache,
                    memory_reserve_mib=(a.startup_min_free_mib if a.startup_min_free_mib is not None
                                        else KVConfig().memory_reserve_mib),
                    pool_budget_mib=a.kv_pool_memory_budget_mib,
                    snapshot_interval_tokens=a.prefix_snapshot_interval, max_snapshots=a.prefix_max_snapshots))
    srv = ServerConfig(served_model_name=a.served_model_name or str(a.model).rstrip("/").split("/")[-1],
                       api_key=a.api_key, chat_default_max_tokens=a.chat_default_max_tokens,
                       max_queued_requests=a.max_queued_requests, request_timeout_ms=a.request_timeout_ms,
                       stream_queue_max_chunks=a.stream_queue_max_chunks, metrics=a.metrics,
                       max_chat_sessions=a.max_chat_sessions, shutdown_grace_seconds=a.shutdown_grace_seconds,
                       batch_window_ms=a.batch_window_ms, max_batch_size=a.max_batch_size,
                       replay_dir=a.replay_dir, replay_redaction=a.replay_redaction)
    srv.validate()
    return eng, srv


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    eng, srv = configs_from_args(a)
    if a.info:
        import json
        from dataclasses import asdict
        from ..loading.model_loader import describe_model_source
        model = describe_model_source(a.model)
        print(json.dumps({"model": model, "engine": asdict(eng), "server": asdict(srv)}, indent=1, default=str))
        return 2 if "error" in model else 0
    from . import log_style
    level = "DEBUG" if a.debug else a.log_level.upper()
    log_style.install(level, log_style.want_color(a.log_color, sys.stderr.isatty()))
    log = logging.getLogger("hipengine_b200.server")
    from ..llm import LLM
    from .api import create_app
    import time
    t0 = time.time()
    llm = LLM(a.model, backend=a.backend, execution_profile=a.execution_profile,
              max_active_requests=a.max_active_requests, max_sequence_length=a.max_context_tokens,
              prefix_cache=a.prefix_cache, speculative_mtp_serving=a.speculative_mtp_serving,
              speculative_candidate_budget=a.speculative_candidate_budget,
              speculative_provider=a.speculative_provider, mtp_hot_vocab=a.mtp_hot_vocab, draft_model=a.draft_model,
              kv_cold_tier_bytes=int(a.kv_cold_tier_gib * (1 << 30)), kv_cold_tier_dir=a.kv_cold_tier_dir,
              tensor_parallel=a.tensor_parallel,
              expert_parallel=a.expert_parallel, engine_config=eng, expected_quant=a.quant)
    import os
    rank = int(os.environ.get("RANK", "0"))
    if max(a.tensor_parallel, a.expert_parallel) > 1 and rank != 0:
        # one HTTP server in front of the group: rank 0 serves, this rank follows its command batches
        log.info("rank %d follows rank 0 (tensor_parallel=%d expert_parallel=%d)", rank, a.tensor_parallel,
                 a.expert_parallel)
        llm.follow()
        return 0
    if a.eager_load or a.startup_chat_smoke or max(a.tensor_parallel, a.expert_parallel) > 1:
        info = llm.prepare()
        log_style.log_lines(log, log_style.load_timing_rows(llm.startup))
        log.info("LOAD_TIMING prepare=%.2fs", time.time() - t0)
        log_style.log_lines(log, log_style.startup_summary(
            srv.served_model_name, llm.backend, info if isinstance(info, dict) else None, llm.startup,
            {"tensor_parallel": a.tensor_parallel, "expert_parallel": a.expert_parallel,
             "prefix_cache": a.prefix_cache, "speculative": a.speculative_mtp_serving,
             "mtp_hot_vocab": a.mtp_hot_vocab, "draft_model": a.draft_model, "kv_storage": a.kv_storage}))
    if a.startup_chat_smoke:
        from ..llm import SamplingParams
        out = llm.chat([{"role": "user", "content": a.eager_load_prompt}],
                       SamplingParams(max_tokens=a.eager_load_max_tokens))
        log.info("startup chat smoke: %d tokens, finish=%s", len(out.token_ids), out.finish.reason)
        llm.mark_warm()
    app = create_app(llm, srv)
    import uvicorn
    uvicorn.run(app, host=a.host, port=a.port, log_level=a.log_level)
    return 0


if __name__ == "__main__":
    sys.exit(main())
