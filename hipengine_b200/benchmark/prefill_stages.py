"""Device-timed stage breakdown of a prefill on the 27B geometry (CUDA events around every stage of the executor,
``HE_STAGE_TIMING=1``), single GPU or one rank per GPU under ``torch.distributed.run``.

    python -m hipengine_b200.benchmark.prefill_stages --layers 8 --tokens 4096
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29531 \
        -m hipengine_b200.benchmark.prefill_stages --layers 8 --tokens 4096

Prints rank 0's stage totals in ms (norm = RMSNorm, plus the all-gather push when the residual is sequence-parallel;
out / down GEMMs include their reduce-scatter) and the event-timed total of the whole prefill call.  The role of the
reference's stage timers (``hipengine/runtime/qwen35_gguf_timing.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen35-27b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--tp-comm", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args()
    os.environ["HE_STAGE_TIMING"] = "1"
    import torch
    from dataclasses import replace
    from ..models.config import NAMED_CONFIGS
    from ..ops import kernels as K
    from ..parallel.groups import init_distributed
    ctx = init_distributed()
    cfg = replace(NAMED_CONFIGS[a.model], n_layers=a.layers)
    toks = torch.randint(0, cfg.vocab, (a.tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    if ctx.world > 1:
        from ..parallel.tp import build_tp_executor
        ex = build_tp_executor(cfg, 0, ctx.device, ctx=ctx, comm=a.tp_comm, max_slots=1, max_context=a.tokens + 512)
    else:
        from ..loading.synth import build_random_model
        from ..models.executor import HybridExecutor
        ex = HybridExecutor(build_random_model(cfg, seed=0, device="cuda"), device="cuda", max_slots=1,
                            max_context=a.tokens + 512)
    tot = 0.0
    for _ in range(3):
        ex.reset_slot(0)
        ex.timer.reset()
        torch.cuda.synchronize()
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ex.prefill(0, toks, graph=False)
        e1.record()
        torch.cuda.synchronize()
        tot = e0.elapsed_time(e1)
    summ = ex.stage_summary()
    if ctx.rank == 0:
        print(json.dumps({"world": ctx.world, "layers": a.layers, "tokens": a.tokens, "total_ms": round(tot, 2),
                          "stages": {k: round(v["total_ms"], 2) for k, v in summ.items()}}))
    K.check_status(ctx.device)
    ctx.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
