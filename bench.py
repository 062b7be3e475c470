"""Headline benchmark: dense hybrid 27B decoder, GGUF Q4_K_M weights, bf16 KV, batch 1,
4096-token prefill then 256 decode tokens.  With N GPUs: one replica and one request stream per GPU (the
headline, weak scaling), plus the same request as a single stream sharded tensor-parallel over the N GPUs.

One "step" is one complete request (prefill + decode).  `value` is decode tokens/s (whole job); prefill
tokens/s, TTFT and ITL are reported beside it.  Weights are random N(0, 0.02) quantized on the device
(no network for checkpoints), prompts are uniform random ids.  The weight stream of one decode step
(~15 GB) is far larger than L2, so no explicit L2 flush is needed between iterations.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference (prints why it is unavailable here)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_DECODE_TOK_S = 30.8     # reference README: Qwen3.8-27B Q4_K_M TG on Radeon Pro W7900
BASELINE_PREFILL_TOK_S = 898.6   # same row, PP
# (decode tok/s, prefill tok/s, label) published by the reference for each model family on the W7900
BASELINES = {
    "qwen35-27b": (30.8, 898.6, "27B dense hybrid Q4_K_M"),
    "qwen35-35b-a3b": (95.0, 2924.5, "35B-A3B MoE hybrid Q4_K_M"),
    "gemma4-26b-a4b": (75.8, 3805.6, "Gemma 4 26B-A4B MoE Q4_K_XL-style"),
}


def reference_arm(args) -> int:
    reason = ("reference cannot run here: pip install needs the hatchling build backend, which is not in the "
              "offline wheelhouse, and its GGUF kernels are HIP gfx1100/gfx1151 only (its CUDA backend is "
              "sm_120a Maple/Moonshine with no GGUF consumer, no sm_100 path, no NCCL)")
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen35-27b")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--gen-len", type=int, default=256)
    ap.add_argument("--parallelism", default="tp", choices=["dp", "tp"],
                    help="N > 1: tp = the one batch-1 request stream sharded tensor-parallel over the GPUs (the named "
                         "config, strong scaling); dp = one replica and one request stream per GPU (weak scaling)")
    ap.add_argument("--tp-comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-extra", action="store_true", help="N > 1: skip the measurement of the other parallelism")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the layer stack (marks the run invalid)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-prefill-graphs", action="store_true",
                    help="issue the prefill forward eagerly instead of replaying it from a CUDA graph per shape")
    ap.add_argument("--batch", type=int, default=1,
                    help="concurrent sequences per stream: each is prefilled on its own, then all decode together as one "
                         "packed step per token (continuous-batching steady state)")
    ap.add_argument("--no-mtp", action="store_true", help="N = 1: skip the speculative (NextN depth 3) cycle figures")
    ap.add_argument("--mtp-depth", type=int, default=3)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3 and not args.layers:
        args.warmup = 3

    if not args.no_prefill_graphs and not args.no_graphs:
        os.environ.setdefault("HE_PREFILL_GRAPH", "1")
    import torch
    import torch.distributed as dist
    from hipengine_b200.core import native
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import NAMED_CONFIGS
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.groups import init_distributed

    ctx = init_distributed()
    world, rank, local_rank, dev = ctx.world, ctx.rank, ctx.local_rank, ctx.device
    if not native.lib_available():
        raise SystemExit("native library missing: run `python -c 'import __graft_entry__ as g; g.build()'` first")

    cfg = NAMED_CONFIGS[args.model]
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    ctx_max = args.prompt_len + args.gen_len + 16
    mode = args.parallelism if world > 1 else "single"
    gen = torch.Generator().manual_seed(1234 + (rank if mode == "dp" else 0))
    prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=gen).tolist()
               for _ in range(max(args.steps + args.warmup, args.batch))]
    B = max(1, args.batch)
    if B > 1:
        ctx_max = args.prompt_len + args.gen_len + 16
    from hipengine_b200.models.decode_graph import DecodeGraphRunner

    def build(tp: bool, comm=None):
        if tp:
            from hipengine_b200.parallel.tp import build_tp_executor
            e = build_tp_executor(cfg, seed=0, device=dev, ctx=ctx, comm=comm or args.tp_comm, max_slots=B,
                                  max_context=ctx_max)
        else:
            from hipengine_b200.models import make_executor
            weights = build_random_model(cfg, seed=0, device=dev, recipe="q4_k_m")
            e = make_executor(weights, device=dev, max_slots=B, max_context=ctx_max)
            del weights
        return e, DecodeGraphRunner(e, max_rows=B, use_graphs=not args.no_graphs)

    def barrier():
        ctx.barrier()
        torch.cuda.synchronize()

    def measure(ex, runner, n_warm, n_steps, sample_clocks):
        """n_warm untimed requests, then n_steps timed ones; device times are max over ranks."""
        tok_log = torch.zeros(args.gen_len, dtype=torch.int64, device=dev)

        def one_batch(step_i, ev, log=False):
            """B sequences: prefill each (its own slot), then gen_len - 1 packed decode steps of B rows."""
            for sl in range(B):
                ex.reset_slot(sl)
            ev[0].record()
            for sl in range(B):
                logits = ex.prefill(sl, prompts[(step_i + sl) % len(prompts)])
                ex.greedy(logits, runner.next_ids[sl:sl + 1])
            runner.slot[:B].copy_(torch.arange(B, dtype=torch.int32, device=dev))
            runner.pos[:B].fill_(args.prompt_len - 1)
            runner.ctx_len[:B].fill_(args.prompt_len)
            runner.publish(B)
            ev[1].record()
            for j in range(args.gen_len - 1):
                runner.step(B, ctx_max)
                if log:
                    tok_log[j].copy_(runner.tokens[0])
            ev[2].record()

        def one_request(prompt, ev, log=False):
            if B > 1:
                return one_batch(prompts.index(prompt) if prompt in prompts else 0, ev, log)
            ex.reset_slot(0)
            ev[0].record()
            logits = ex.prefill(0, prompt)
            ex.greedy(logits, runner.next_ids[:1])
            runner.slot[:1].zero_()
            runner.pos[:1].fill_(len(prompt) - 1)
            runner.ctx_len[:1].fill_(len(prompt))
            runner.publish(1)                       # first token -> tokens[0], pos -> len(prompt)
            ev[1].record()
            for j in range(args.gen_len - 1):
                runner.step(1, ctx_max)
                if log:
                    tok_log[j].copy_(runner.tokens[0])
            ev[2].record()

        mk = lambda: [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for i in range(n_warm):
            # the last warm-up request (untimed) records its tokens: tensor-parallel ranks must generate the same ones
            one_request(prompts[i % len(prompts)], mk(), log=(i == n_warm - 1))
        barrier()
        agree = None
        if world > 1 and mode == "tp":
            allt = ctx.all_gather(tok_log)
            agree = bool((allt == allt[0]).all())
        sampler = ClockSampler(local_rank)
        if rank == 0 and sample_clocks:
            sampler.start()
        k0 = K.launch_count()
        evs = [mk() for _ in range(n_steps)]
        barrier()
        t0 = time.time()
        for i in range(n_steps):
            one_request(prompts[(n_warm + i) % len(prompts)], evs[i])
        barrier()
        wall_s = time.time() - t0
        launches = K.launch_count() - k0
        clocks = sampler.stop() if (rank == 0 and sample_clocks) else {}
        K.check_status(dev)
        t = torch.tensor([sum(e[0].elapsed_time(e[1]) for e in evs), sum(e[1].elapsed_time(e[2]) for e in evs)],
                         dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms, decode_ms = t.tolist()
        return {"prefill_ms": prefill_ms, "decode_ms": decode_ms, "wall_s": wall_s, "launches": launches,
                "clocks": clocks, "ranks_agree": agree}

    t_build0 = time.time()
    ex, runner = build(tp=(mode == "tp"))
    torch.cuda.synchronize()
    build_s = time.time() - t_build0
    m = measure(ex, runner, args.warmup, args.steps, True)
    streams = (world if mode == "dp" else 1) * B    # independent sequences in flight
    n_dec = (args.gen_len - 1) * args.steps * streams
    decode_tok_s = n_dec / (m["decode_ms"] / 1e3)
    prefill_tok_s = args.prompt_len * args.steps * streams / (m["prefill_ms"] / 1e3)

    e2e = None
    if not args.no_e2e and B == 1:
        try:
            mine = run_e2e(args, cfg, ex, prompts)
            # replicas run side by side: tokens add up, the slowest replica sets the time
            t = torch.tensor([mine["decode_s"], mine["prefill_s"]], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dec_s, pre_s = t.tolist()
            e2e = {"value": round(n_dec / dec_s, 3), "unit": "tok/s",
                   "prefill_tok_s": round(args.prompt_len * args.steps * streams / pre_s, 2),
                   "h2d_bytes_per_step": mine["h2d_bytes_per_step"] * streams,
                   "d2h_bytes_per_step": mine["d2h_bytes_per_step"] * streams}
        except Exception as exc:  # the device-timed line must still be printed
            e2e = {"error": f"{type(exc).__name__}: {exc}"}
            if world > 1:
                raise

    mtp = None
    if world == 1 and B == 1 and not args.no_mtp and not args.no_graphs and cfg.is_hybrid and not getattr(cfg, "n_experts", 0):
        # speculative decoding on the same geometry with a NextN block appended: cost of one captured cycle in units
        # of an autoregressive step, tokens per cycle with the block's own drafts (random weights: near zero
        # acceptance) and with the true continuation as drafts (every draft accepted: the upper bound)
        runner.graphs.clear()
        runner = ex = None
        torch.cuda.empty_cache()
        try:
            mtp = run_mtp(args, cfg, dev, prompts[0], ctx_max)
        except Exception as exc:
            mtp = {"error": f"{type(exc).__name__}: {exc}"}

    nccl_base = None
    if world > 1 and mode == "tp" and args.tp_comm == "fused" and not args.no_extra:
        # the same tensor-parallel engine with every collective done by the library (NCCL all-reduce / all-gather
        # after the kernels, nothing fused): the baseline the fused peer-memory paths are measured against
        if runner is not None:
            runner.graphs.clear()
        close = getattr(ex, "close_comm", None)
        if close is not None:
            close()
        runner = ex = None
        torch.cuda.empty_cache()
        try:
            ex, runner = build(tp=True, comm="nccl")
            mb = measure(ex, runner, 2, 1, False)
            nccl_base = {"steps": 1, "warmup": 2, "decode_tok_s": round((args.gen_len - 1) / (mb["decode_ms"] / 1e3), 3),
                         "prefill_tok_s": round(args.prompt_len / (mb["prefill_ms"] / 1e3), 2),
                         "itl_ms": round(mb["decode_ms"] / (args.gen_len - 1), 4),
                         "ttft_ms": round(mb["prefill_ms"], 3), "ranks_agree": mb["ranks_agree"]}
        except Exception as exc:
            nccl_base = {"error": f"{type(exc).__name__}: {exc}"}

    extra = None
    if world > 1 and not args.no_extra:
        # the other way to use the N GPUs, measured briefly for context: tp -> N independent replicas (aggregate
        # tokens/s, weak scaling); dp -> the single stream sharded over all GPUs
        other_tp = mode == "dp"
        if runner is not None:
            runner.graphs.clear()
        runner = ex = None
        torch.cuda.empty_cache()
        try:
            ex, runner = build(tp=other_tp)
            mt = measure(ex, runner, 2, 1, False)
            k = 1 if other_tp else world
            extra = {"parallelism": f"tp{world}" if other_tp else f"dp{world}", "steps": 1, "warmup": 2,
                     "decode_tok_s": round(k * (args.gen_len - 1) / (mt["decode_ms"] / 1e3), 3),
                     "prefill_tok_s": round(k * args.prompt_len / (mt["prefill_ms"] / 1e3), 2),
                     "itl_ms": round(mt["decode_ms"] / (args.gen_len - 1), 4), "ttft_ms": round(mt["prefill_ms"], 3)}
            if other_tp:
                extra["comm"] = args.tp_comm
        except Exception as exc:
            extra = {"error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        par = {"single": "single", "dp": f"dp{world}", "tp": f"tp{world}"}[mode]
        if mode == "tp" and getattr(cfg, "n_experts", 0):
            par += f"+ep{world}"              # attention / GDN tensor-parallel, experts dealt out by rank
        base_dec, base_pre, label = BASELINES.get(args.model, (None, None, args.model))
        if B > 1:
            base_dec = base_pre = None          # the published figures are single-sequence runs
        line = {
            "metric": f"decode_tok_s ({label}, bf16 KV, batch {B} per stream, {args.prompt_len} prefill + "
                      f"{args.gen_len} decode)",
            "value": round(decode_tok_s, 3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round((m["prefill_ms"] + m["decode_ms"]) / args.steps, 3),
            "higher_is_better": True, "scaling": "weak" if mode == "dp" else "strong",
            "vs_baseline": round(decode_tok_s / base_dec, 3) if base_dec else None, "dtype": "bf16",
            "data": "synthetic (random-init N(0,0.02) weights quantized to Q4_K_M-style GGUF blocks, uniform random prompt ids)",
            "config": {"model": args.model, "global_batch": streams, "seq_len": args.prompt_len,
                       "gen_len": args.gen_len, "parallelism": par, "layers": cfg.n_layers,
                       "l2": "inputs larger than L2 (weight stream ~15 GB/step)", "cuda_graphs": not args.no_graphs,
                       "prefill_graph": os.environ.get("HE_PREFILL_GRAPH", "0") == "1"},
            "prefill_tok_s": round(prefill_tok_s, 2),
            "prefill_vs_baseline": round(prefill_tok_s / base_pre, 3) if base_pre else None,
            "ttft_ms": round(m["prefill_ms"] / args.steps, 3),
            "itl_ms": round(m["decode_ms"] / ((args.gen_len - 1) * args.steps), 4),
            "batch": B,
            "wall_s": round(m["wall_s"], 3), "build_s": round(build_s, 2),
            "clocks": m["clocks"], "gpu_launches": int(m["launches"]) * (world if mode == "dp" else 1),
        }
        if e2e is not None:
            line["e2e"] = e2e
        if mtp is not None:
            line["mtp"] = mtp
        if extra is not None:
            line["other_parallelism"] = extra
        if mode == "tp":
            line["config"]["tp_comm"] = args.tp_comm
            line["ranks_agree"] = m["ranks_agree"]
        if nccl_base is not None:
            line["nccl_baseline"] = nccl_base
        if args.layers:
            line["invalid"] = "truncated layer stack (debug run)"
        print(json.dumps(line))
    sys.stdout.flush()
    if world > 1:
        # Captured graphs hold library collectives: drop them before the process group goes away.  The number is
        # already printed; a watchdog ends the process if the library's teardown stalls anyway.
        import gc
        dog = threading.Timer(45.0, lambda: os._exit(0))
        dog.daemon = True
        dog.start()
        if runner is not None:
            runner.graphs.clear()
        runner = ex = None
        gc.collect()
        barrier()
        dist.destroy_process_group()
        dog.cancel()
    return 0


def run_mtp(args, cfg, dev, prompt, ctx_max):
    """NextN speculative cycle on the benchmark geometry (one request, greedy): device-timed figures."""
    import torch
    from dataclasses import replace
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models import make_executor
    from hipengine_b200.models.decode_graph import DecodeGraphRunner
    from hipengine_b200.models.executor import make_batch
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.speculative.mtp import GraphedMTPCycle
    depth = args.mtp_depth
    cfgm = replace(cfg, nextn_layers=1)
    weights = build_random_model(cfgm, seed=0, device=dev, recipe="q4_k_m")
    ex = make_executor(weights, device=dev, max_slots=1, max_context=ctx_max)
    del weights
    from hipengine_b200.speculative.draft_vocab import resolve_hot_vocab_rows
    hot_rows = resolve_hot_vocab_rows("auto", cfgm.vocab)
    cyc = GraphedMTPCycle(ex, max_depth=depth, max_requests=1, draft_head_rows=hot_rows)
    runner = DecodeGraphRunner(ex, max_rows=1)
    b = make_batch([(0, 0, prompt)], dev)
    h = ex.forward(b)
    cyc.after_prefill(b, h)
    last = int(ex.logits(h[b.T - 1:b.T]).argmax(-1))
    pos = len(prompt)                                   # position of `last`
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def cycles(n, override=None, small=False):
        nonlocal last, pos
        toks = 0
        for i in range(n):
            ov = None if override is None else torch.tensor([override[toks:toks + depth]])
            res, _ = cyc.cycle([0], [last], [pos], depth, draft_override=ov, small_head=small)
            toks += len(res[0].tokens)
            last, pos = res[0].tokens[-1], pos + len(res[0].tokens)
        return toks

    cycles(4)
    n_cyc = 24
    e0, e1 = ev(), ev()
    torch.cuda.synchronize()
    e0.record()
    got = cycles(n_cyc)
    e1.record()
    torch.cuda.synchronize()
    cycle_ms = e0.elapsed_time(e1) / n_cyc
    # the same cycle drafting with the leading slice of the head (hot-vocabulary draft head; verification unchanged)
    hot_ms = None
    if cyc.draft_head_rows > 0:
        cycles(3, small=True)
        e4, e5 = ev(), ev()
        torch.cuda.synchronize()
        e4.record()
        cycles(n_cyc, small=True)
        e5.record()
        torch.cuda.synchronize()
        hot_ms = e4.elapsed_time(e5) / n_cyc
    # autoregressive steps from the same state (graph replay), recorded: they are the true continuation
    snap = {"conv": {i: t[0].clone() for i, t in ex.conv_state.items()},
            "gdn": {i: t[0].clone() for i, t in ex.gdn_state.items()}, "hp": cyc.h_prev[0].clone()}
    n_ar = 8 * (depth + 1)
    runner.set_rows([0], [last], [pos])
    cont = torch.zeros(n_ar + 4, dtype=torch.int64, device=dev)
    for j in range(4):
        runner.step(1, ctx_max)
        cont[j].copy_(runner.tokens[0])
    e2, e3 = ev(), ev()
    e2.record()
    for j in range(n_ar):
        runner.step(1, ctx_max)
        cont[4 + j].copy_(runner.tokens[0])
    e3.record()
    torch.cuda.synchronize()
    ar_ms = e2.elapsed_time(e3) / n_ar
    # every draft accepted: rewind the recurrent state and feed the recorded continuation as drafts (eager cycle)
    for i, t in ex.conv_state.items():
        t[0].copy_(snap["conv"][i])
    for i, t in ex.gdn_state.items():
        t[0].copy_(snap["gdn"][i])
    cyc.h_prev[0].copy_(snap["hp"])
    forced = cycles(6, override=cont.tolist() + [0] * depth)
    K.check_status(dev)
    units = cycle_ms / ar_ms
    return {"depth": depth, "ar_step_ms": round(ar_ms, 4), "cycle_ms": round(cycle_ms, 4),
            "cycle_cost_ar_units": round(units, 3), "tokens_per_cycle_own_drafts": round(got / n_cyc, 3),
            "tokens_per_cycle_all_accepted": round(forced / 6, 3),
            "speedup_all_accepted": round((forced / 6) / units, 3),
            "kernels_per_cycle_graph": list(cyc.graph_stats["kernels_per_graph"].values())[:1],
            "graph": cyc.graph_stats["captures"],
            "hot_vocab": None if hot_ms is None else {"rows": cyc.draft_head_rows, "cycle_ms": round(hot_ms, 4),
                                                      "cycle_cost_ar_units": round(hot_ms / ar_ms, 3)},
            "note": "random weights: own drafts are almost never accepted"}


def run_e2e(args, cfg, ex, prompts):
    """Same request through the public API: pinned-host prompt -> LLM.generate -> token ids read back."""
    import torch
    from hipengine_b200.llm import LLM, SamplingParams
    llm = LLM.from_executor(ex) if hasattr(LLM, "from_executor") else None
    if llm is None:
        return {"error": "public API not wired"}
    sp = SamplingParams(max_tokens=args.gen_len, temperature=0.0, ignore_eos=True)
    pinned = [torch.tensor(p, dtype=torch.int64).pin_memory() for p in prompts]
    try:
        for i in range(min(2, args.warmup)):
            llm.generate_detailed(pinned[i].tolist(), sp)
        dec_s = pre_s = 0.0
        h2d = d2h = 0
        for i in range(args.steps):
            out = llm.generate_detailed(pinned[args.warmup + i].tolist(), sp)[0]
            dec_s += out.telemetry.decode_seconds
            pre_s += out.telemetry.prefill_seconds
            h2d += out.telemetry.h2d_bytes
            d2h += out.telemetry.d2h_bytes
    finally:
        # the engine's decode graphs may hold library collectives: release them with the engine
        try:
            llm._engine.loop.runner.graphs.graphs.clear()
        except Exception:
            pass
        llm.close()
    return {"decode_s": dec_s, "prefill_s": pre_s,
            "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps}


if __name__ == "__main__":
    sys.exit(main())
