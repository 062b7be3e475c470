"""Serving load benchmark: Poisson arrivals against the OpenAI-compatible server over HTTP with SSE streaming.

Scenario (the reference's served-load protocol, ``benchmarks/README.md`` "served ShareGPT" rows, with synthetic
prompts): ``--requests`` requests arrive as a Poisson stream of ``--rate`` per second, at most ``--concurrency``
in flight; prompt lengths are uniform in [--min-prompt, --max-prompt] random token ids, half of the prompts start
with one common ``--shared-prefix``-token prefix (exercises the paged prefix cache); every request streams
``--output-tokens`` tokens.  Reports request throughput, generated tokens/s, p50/p99 TTFT and inter-token latency
measured at the client from the SSE frames, and the server's prefix-cache counters.

    python -m hipengine_b200.benchmark.serving_load --model qwen35-27b --requests 256 --concurrency 64

The server runs in this process (uvicorn on a background thread, 127.0.0.1) unless ``--url`` points at one that is
already running.  ``--endpoint completions`` sends token-id prompts to ``/v1/completions`` (no tokenizer noise in the
timing); ``--endpoint chat`` sends one user message of random text to ``/v1/chat/completions`` (prompt length is then
approximate: the template adds a few tokens).

A tensor-parallel group is served by launching this module under ``torch.distributed.run`` with
``--tensor-parallel N``: rank 0 runs the HTTP server, the scheduler and the load generator, the other ranks follow
its command batches; ``--mtp on`` turns speculative decoding (NextN block, ``--mtp-depth`` drafts) on.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
        -m hipengine_b200.benchmark.serving_load --model qwen35-27b-mtp --tensor-parallel 8 --mtp on --endpoint chat
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import threading
import time
from typing import Any, Dict, List, Optional

from ..generation.simulator import poisson_arrivals


def build_prompts(n: int, vocab: int, min_len: int, max_len: int, shared_prefix: int, seed: int = 0) -> List[List[int]]:
    rng = random.Random(seed)
    common = [rng.randrange(vocab) for _ in range(shared_prefix)]
    out = []
    for i in range(n):
        total = rng.randint(min_len, max_len)
        if i % 2 == 0 and shared_prefix and total > shared_prefix:
            out.append(common + [rng.randrange(vocab) for _ in range(total - shared_prefix)])
        else:
            out.append([rng.randrange(vocab) for _ in range(total)])
    return out


def _as_text(ids: List[int]) -> str:
    """Random lower-case text with one character per requested token (a byte-level tokenizer maps it 1:1)."""
    return "".join(chr(97 + (t % 26)) for t in ids)


async def _one(session, url: str, model: str, prompt: List[int], max_tokens: int, rec: Dict[str, Any],
               endpoint: str = "completions") -> None:
    body = {"model": model, "max_tokens": max_tokens, "stream": True, "temperature": 0.0,
            "ignore_eos": True, "stream_options": {"include_usage": True}}
    if endpoint == "chat":
        body["messages"] = [{"role": "user", "content": _as_text(prompt)}]
        path = "/v1/chat/completions"
    else:
        body["prompt"] = prompt
        path = "/v1/completions"
    t0 = time.perf_counter()
    stamps: List[float] = []
    try:
        async with session.post(url + path, json=body) as resp:
            rec["status"] = resp.status
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                if ev.get("usage"):
                    rec["usage"] = ev["usage"]
                ch = ev["choices"][0] if ev.get("choices") else None
                d = (ch.get("delta") or {}) if ch is not None else {}
                if ch is not None and (ch.get("text") is not None or d.get("content") or d.get("reasoning_content")):
                    stamps.append(time.perf_counter())
    except Exception as exc:
        rec["error"] = f"{type(exc).__name__}: {exc}"
    rec["t_submit"], rec["stamps"] = t0, stamps


async def run_load(url: str, model: str, prompts: List[List[int]], arrivals: List[float], concurrency: int,
                   max_tokens: int, endpoint: str = "completions") -> List[Dict[str, Any]]:
    import aiohttp
    sem = asyncio.Semaphore(concurrency)
    recs: List[Dict[str, Any]] = [{} for _ in prompts]
    start = time.perf_counter()
    timeout = aiohttp.ClientTimeout(total=3600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def task(i: int) -> None:
            await asyncio.sleep(max(0.0, arrivals[i] - (time.perf_counter() - start)))
            async with sem:
                await _one(session, url, model, prompts[i], max_tokens, recs[i], endpoint)
        await asyncio.gather(*[task(i) for i in range(len(prompts))])
    for r in recs:
        r["t0"] = start
    return recs


def summarise(recs: List[Dict[str, Any]], wall_s: float) -> Dict[str, Any]:
    def pct(xs, p):
        if not xs:
            return None
        s = sorted(xs)
        return s[min(len(s) - 1, int(p * len(s)))]
    ok = [r for r in recs if r.get("status") == 200 and r.get("stamps")]
    ttft = [1e3 * (r["stamps"][0] - r["t_submit"]) for r in ok]
    itl: List[float] = []
    for r in ok:
        s = r["stamps"]
        itl += [1e3 * (b - a) for a, b in zip(s, s[1:])]
    gen = sum((r.get("usage") or {}).get("completion_tokens", len(r["stamps"])) for r in ok)
    cached = sum(((r.get("usage") or {}).get("prompt_tokens_details") or {}).get("cached_tokens", 0) for r in ok)
    prompt_toks = sum((r.get("usage") or {}).get("prompt_tokens", 0) for r in ok)
    return {"requests": len(recs), "completed": len(ok), "failed": len(recs) - len(ok), "wall_s": round(wall_s, 3),
            "requests_per_s": round(len(ok) / wall_s, 3), "generated_tok_per_s": round(gen / wall_s, 2),
            "prompt_tok_per_s": round(prompt_toks / wall_s, 2),
            "ttft_p50_ms": pct(ttft, 0.5), "ttft_p99_ms": pct(ttft, 0.99),
            "itl_p50_ms": pct(itl, 0.5), "itl_p99_ms": pct(itl, 0.99),
            "cached_prompt_tokens": cached, "prompt_tokens": prompt_toks}


def _serve_in_thread(llm, served_name: str, port: int, batch_window_ms: float = 0.0):
    import uvicorn
    from ..server.api import ServerConfig, create_app
    app = create_app(llm, ServerConfig(served_model_name=served_name, max_queued_requests=4096,
                                       batch_window_ms=batch_window_ms))
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    return server, th


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen35-27b")
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--url", default=None)
    ap.add_argument("--port", type=int, default=8011)
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--rate", type=float, default=8.0, help="mean arrivals per second")
    ap.add_argument("--min-prompt", type=int, default=512)
    ap.add_argument("--max-prompt", type=int, default=8192)
    ap.add_argument("--shared-prefix", type=int, default=2048)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--max-active", type=int, default=64)
    ap.add_argument("--mtp", default="off", choices=["off", "on"])
    ap.add_argument("--mtp-depth", type=int, default=3)
    ap.add_argument("--endpoint", default="completions", choices=["completions", "chat"])
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--batch-window-ms", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--gpu-sampler", action="store_true",
                    help="sample device memory, SM clock, power and throttle reasons over NVML (read-only) during the load")
    a = ap.parse_args(argv)
    llm = server = None
    url = a.url
    vocab = 32000
    import os
    rank = int(os.environ.get("RANK", "0"))
    if url is None:
        from ..llm import LLM
        llm = LLM(a.model, backend=a.backend, max_active_requests=a.max_active,
                  max_sequence_length=a.max_prompt + a.output_tokens + 128, prefix_cache="radix",
                  speculative_mtp_serving=a.mtp, speculative_candidate_budget=a.mtp_depth,
                  tensor_parallel=a.tensor_parallel)
        if a.tensor_parallel > 1 and rank != 0:
            llm.follow()            # returns when rank 0 closes the group
            return 0
        llm.prepare()
        vocab = llm.vocab_size
        server, _ = _serve_in_thread(llm, a.model, a.port, a.batch_window_ms)
        url = f"http://127.0.0.1:{a.port}"
    prompts = build_prompts(a.requests, vocab, a.min_prompt, a.max_prompt, a.shared_prefix, a.seed)
    arrivals = poisson_arrivals(a.requests, a.rate, a.seed)
    sampler = None
    if a.gpu_sampler:
        from ..utils.nvml_sampler import NvmlSampler
        sampler = NvmlSampler(device_index=int(os.environ.get("LOCAL_RANK", "0"))).start()
    t0 = time.perf_counter()
    recs = asyncio.run(run_load(url, a.model, prompts, arrivals, a.concurrency, a.output_tokens, a.endpoint))
    out = summarise(recs, time.perf_counter() - t0)
    if sampler is not None:
        sampler.stop()
        out["gpu"] = sampler.summary()
    if llm is not None:
        try:
            snap = llm.live_loop_snapshot()
            run = snap.get("runner") or snap
            out["server"] = {k: run.get(k) for k in ("prefix_hits", "prefix_hit_tokens", "spec_cycles", "spec_drafted",
                                                     "spec_accepted") if k in run}
            mtp = getattr(getattr(llm._engine.loop, "runner", None), "mtp", None)
            if mtp is not None:
                out["server"]["mtp"] = dict(mtp.stats)
        except Exception as exc:        # the load figures stand on their own
            out["server"] = {"error": str(exc)}
    out["config"] = {"model": a.model, "concurrency": a.concurrency, "rate_per_s": a.rate,
                     "prompt_range": [a.min_prompt, a.max_prompt], "shared_prefix": a.shared_prefix,
                     "output_tokens": a.output_tokens, "mtp": a.mtp, "mtp_depth": a.mtp_depth, "page_tokens": 16,
                     "endpoint": a.endpoint, "tensor_parallel": a.tensor_parallel}
    errs = [r.get("error") for r in recs if r.get("error")]
    if errs:
        out["first_error"] = errs[0]
    print(json.dumps(out))
    if server is not None:
        server.should_exit = True
    if llm is not None:
        llm.close()
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
