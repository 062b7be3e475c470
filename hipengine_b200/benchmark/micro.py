"""Per-kernel micro-benchmarks with roofline fractions.

    python -m hipengine_b200.benchmark.micro gemm --m 4096 --n 17408 --k 5120
    python -m hipengine_b200.benchmark.micro gemmq --m 4096 --n 17408 --k 5120 --qtype q4_k
    python -m hipengine_b200.benchmark.micro gemv --n 17408 --k 5120 --qtype q4_k --rows 1
    python -m hipengine_b200.benchmark.micro all

Timing: CUDA events on the launching stream, >= 3 warm-up launches, inputs rotated through a pool larger
than L2 (126 MB) so every timed launch reads its operands from HBM.  Fractions are "of measured": the
denominators come from MEASURED_PEAKS.json at the repository root when present (copy bandwidth and cuBLAS
bf16 throughput measured on this pool), else the stated fallback.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


def time_launches(fn, n_variants: int, iters: int = 5, warmup: int = 3) -> float:
    """Median milliseconds per launch of fn(i).

    The n_variants launches (each touching different operands, together larger than L2) are captured into
    one CUDA graph and the graph is replayed, so the figure is device time per launch with no host launch
    overhead between kernels.
    """
    for i in range(max(warmup, 1)):
        fn(i % n_variants)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_variants):
            fn(i)
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) / n_variants)
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(M, N, K, impl="tcgen05"):
    from hipengine_b200.ops import gemm as G
    pk = peaks()
    nvar = max(2, int(200e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device="cuda") * 0.05).bfloat16() for _ in range(nvar)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    if impl == "tcgen05":
        fn = lambda i: G.gemm_bf16(x, ws[i], out)
    else:
        fn = lambda i: torch.matmul(x, ws[i].t(), out=out)
    ms = time_launches(fn, nvar)
    if impl == "tcgen05":
        G.check_status()
    tf = 2.0 * M * N * K / ms / 1e9
    return {"kernel": f"gemm_bf16[{impl}]", "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
            f"frac_of_{pk['src']}_bf16": round(tf / pk["bf16_tflops"], 3)}


def bench_gemm_quant(M, N, K, qtype="q4_k"):
    """Tensor-core GEMM over a quantised weight read in its device layout (dequantised inside the pipeline).
    M > 128: plain tiling, reported against the tensor-core peak; M <= 128: split-K, reported against HBM bandwidth
    (the weight bytes are what has to move)."""
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as Kn
    from hipengine_b200.quant import ggml as Q
    pk = peaks()
    t = {"q4_k": Q.GGMLType.Q4_K, "q6_k": Q.GGMLType.Q6_K, "q8_0": Q.GGMLType.Q8_0}[qtype]
    wbytes = N * Q.row_bytes(t, K)
    nvar = max(2, int(260e6 // wbytes) + 1)
    w = torch.randn(N, K, device="cuda") * 0.02
    raw = Q.quantize(w, t)
    dws = [Kn.to_device_weight(raw.clone(), t, N, K) for _ in range(nvar)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    sc = _Scratch(torch.device("cuda", torch.cuda.current_device()))
    if M > 128:
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = lambda i: G.gemm_quant(x, dws[i], out, sc)
    else:
        out = torch.empty(M, N, device="cuda")
        fn = lambda i: G.gemm_quant_splitk(x, dws[i], out, sc)
    ms = time_launches(fn, nvar)
    G.check_status()
    tf = 2.0 * M * N * K / ms / 1e9
    gbs = wbytes / ms / 1e6
    return {"kernel": f"gemm_quant[{qtype}]", "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
            f"frac_of_{pk['src']}_bf16": round(tf / pk["bf16_tflops"], 3), "weight_GBps": round(gbs, 1),
            f"frac_of_{pk['src']}_hbm": round(gbs / pk["hbm_gbs"], 3)}


def bench_gemv(N, K, qtype="q4_k", rows=1):
    from hipengine_b200.ops import kernels as Kn
    from hipengine_b200.quant import ggml as Q
    pk = peaks()
    t = {"q4_k": Q.GGMLType.Q4_K, "q6_k": Q.GGMLType.Q6_K, "q8_0": Q.GGMLType.Q8_0}[qtype]
    wbytes = N * Q.row_bytes(t, K)
    nvar = max(2, int(260e6 // wbytes) + 1)
    dws = []
    for i in range(nvar):
        w = torch.randn(N, K, device="cuda") * 0.02
        dws.append(Kn.to_device_weight(Q.quantize(w, t), t, N, K))
    x = torch.randn(rows, K, device="cuda")
    nw = torch.ones(K, device="cuda")
    out = torch.empty(rows, N, device="cuda")
    fn = lambda i: Kn.gemv(x, [Kn.GemvSegment(dws[i], out)], norm_w=nw)
    ms = time_launches(fn, nvar)
    gbs = wbytes / ms / 1e6
    return {"kernel": f"gemv[{qtype}]", "N": N, "K": K, "rows": rows, "ms": round(ms, 4), "GBps": round(gbs, 1),
            f"frac_of_{pk['src']}_hbm": round(gbs / pk["hbm_gbs"], 3)}


def bench_gdn_scan(T, Hv=48, G=16, n_seg=1, chunked=False):
    """Prefill scan of one gated delta-net layer: T tokens in n_seg segments (27B geometry by default)."""
    from hipengine_b200.ops import kernels as Kn
    pk = peaks()
    S = 128
    C = 2 * G * S + Hv * S
    qkv = torch.randn(T, C, device="cuda") * 0.1
    decay = torch.rand(T, Hv, device="cuda") * 0.2 + 0.8
    beta = torch.rand(T, Hv, device="cuda")
    state = torch.zeros(n_seg, Hv, S, S, device="cuda")
    seg_start = torch.arange(0, T + 1, T // n_seg, device="cuda", dtype=torch.int32)[:n_seg + 1].contiguous()
    seg_slot = torch.arange(n_seg, device="cuda", dtype=torch.int32)
    out = torch.empty(T, Hv, S, device="cuda")
    if chunked:
        fn = lambda i: Kn.gdn_scan_chunked(qkv, decay, beta, state, seg_start, seg_slot, out, G, Hv)
    else:
        fn = lambda i: Kn.gdn_scan(qkv, decay, beta, state, seg_start, seg_slot, out, G, Hv)
    ms = time_launches(fn, 1)
    flops = 6.0 * T * Hv * S * S          # decay, k.S, rank-1 update, q.S: about 6 flop per state element per token
    bytes_ = (qkv.numel() + out.numel()) * 4.0 + 2.0 * state.numel() * 4
    return {"kernel": "gdn_scan_chunked" if chunked else "gdn_scan", "T": T, "Hv": Hv, "n_seg": n_seg, "ms": round(ms, 4),
            "tflops_fp32": round(flops / ms / 1e9, 2), "us_per_token": round(1e3 * ms / (T / n_seg), 3),
            "GBps": round(bytes_ / ms / 1e6, 1), f"frac_of_{pk['src']}_hbm": round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)}


def bench_conv(T, C=10240):
    from hipengine_b200.ops import kernels as Kn
    pk = peaks()
    x = (torch.randn(T, C, device="cuda") * 0.1).bfloat16()
    w = torch.randn(C, 4, device="cuda")
    state = torch.zeros(1, C, 3, device="cuda")
    seg_start = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    seg_slot = torch.zeros(1, device="cuda", dtype=torch.int32)
    tok_seg = torch.zeros(T, device="cuda", dtype=torch.int32)
    out = torch.empty(T, C, device="cuda")
    fn = lambda i: Kn.conv1d(x, w, state, seg_start, seg_slot, tok_seg, out, C)
    ms = time_launches(fn, 1)
    bytes_ = T * C * (2.0 + 4.0)
    return {"kernel": "conv1d+state", "T": T, "C": C, "ms": round(ms, 4), "GBps": round(bytes_ / ms / 1e6, 1),
            f"frac_of_{pk['src']}_hbm": round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)}


def bench_attn_decode(ctx, H=24, Hkv=4, D=256, rows=1):
    from hipengine_b200.ops import kernels as Kn
    pk = peaks()
    page = 16
    n_pages = (ctx + page - 1) // page
    nvar = max(2, int(260e6 // (rows * n_pages * 2 * Hkv * page * D * 2)) + 1)
    caches = [(torch.randn(rows * n_pages + 1, 2, Hkv, page, D, device="cuda") * 0.3).bfloat16() for _ in range(nvar)]
    bt = (torch.arange(rows * n_pages, device="cuda", dtype=torch.int32) + 1).reshape(rows, n_pages).contiguous()
    slot = torch.arange(rows, device="cuda", dtype=torch.int32)
    ctx_len = torch.full((rows,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(rows, H, D, device="cuda").bfloat16()
    gate = torch.randn(rows, H, D, device="cuda").bfloat16()
    split_len, max_splits = Kn.attn_decode_split(ctx, rows, Hkv)
    part = torch.empty(Kn.attn_decode_scratch_floats(rows, H, max_splits, D), device="cuda")
    out = torch.empty(rows, H * D, device="cuda", dtype=torch.bfloat16)
    fn = lambda i: Kn.attn_decode(q, gate, caches[i], bt, slot, ctx_len, part, out, H, Hkv, D, page, split_len,
                                  max_splits, D ** -0.5)
    ms = time_launches(fn, nvar)
    bytes_ = ctx * 2.0 * Hkv * D * 2 * rows
    return {"kernel": "attn_decode(split+reduce)", "ctx": ctx, "rows": rows, "ms": round(ms, 4),
            "GBps": round(bytes_ / ms / 1e6, 1), f"frac_of_{pk['src']}_hbm": round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)}


def bench_fused_allreduce_gemm(M, N, K, phases=7):
    """Single-rank run of the fused GEMM -> all-reduce -> residual-add kernel (every tile goes through the stage,
    reduce and add phases in local memory) against the plain GEMM followed by the residual add: the difference is
    what the collective phases cost on top of the tensor-core work when no link is involved."""
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as K_
    from hipengine_b200.parallel.fused import FusedGemmAllReduce
    from hipengine_b200.parallel.groups import DistContext
    nvar = max(2, int(200e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(nvar)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    h = torch.zeros(M, N, device="cuda")
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ctx = DistContext(0, 1, 0, torch.device("cuda", torch.cuda.current_device()), None, "none")
    fg = FusedGemmAllReduce(ctx, N, max_rows=M)

    def plain(i):
        G.gemm_bf16(x, ws[i], y)
        K_.resid_add_bf16(h, y)

    ms_f = time_launches(lambda i: fg.gemm_add(x, ws[i], h, phases=phases), nvar)
    G.check_status()
    ms_p = time_launches(plain, nvar)
    fg.close()
    tf = 2.0 * M * N * K / 1e9
    return {"kernel": "gemm_bf16_allreduce[world=1]", "M": M, "N": N, "K": K, "phases": phases,
            "fused_ms": round(ms_f, 4), "gemm_plus_add_ms": round(ms_p, 4), "fused_tflops": round(tf / ms_f, 1)}


def bench_seq_parallel_loopback(M, N, K, qtype="q4_k"):
    """The sequence-parallel prefill kernels on the 1-rank loopback form (world = 1: this GPU is the owner of every
    tile and its own peer): GEMM -> reduce-scatter -> residual add in one tcgen05 kernel, RMSNorm + all-gather push,
    and the consumer GEMM with the all-gather wait in its TMA producer -- the form an ncu capture may run on."""
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as Kn
    from hipengine_b200.parallel.fused import SeqParallel
    from hipengine_b200.quant import ggml as Q
    t = {"q4_k": Q.GGMLType.Q4_K, "q6_k": Q.GGMLType.Q6_K, "q8_0": Q.GGMLType.Q8_0}[qtype]
    sp = SeqParallel.emulated_group("cuda", N, 1, max_rows=M)[0]
    raw = Q.quantize(torch.randn(N, K, device="cuda") * 0.02, t)
    nvar = max(2, int(260e6 // (N * Q.row_bytes(t, K))) + 1)
    dws = [Kn.to_device_weight(raw.clone(), t, N, K) for _ in range(nvar)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    sp.h[:M].normal_()
    ms_rs = time_launches(lambda i: sp.gemm_rs(x, dws[i], M), nvar)
    nw = torch.ones(N, device="cuda")
    ms_np = time_launches(lambda i: sp.norm_push(M, nw, 1e-6), nvar)
    sp.wait()
    raw2 = Q.quantize(torch.randn(K, N, device="cuda") * 0.02, t) if N % 256 == 0 else None
    out = []
    tf = 2.0 * M * N * K / 1e9
    out.append({"kernel": f"gemm_q_reduce_scatter[{qtype}, world=1]", "M": M, "N": N, "K": K, "ms": round(ms_rs, 4),
                "tflops": round(tf / ms_rs, 1)})
    out.append({"kernel": "rmsnorm_allgather_push[world=1]", "T": M, "H": N, "ms": round(ms_np, 4),
                "GBps": round(M * N * (4 + 2) / ms_np / 1e6, 1)})
    if raw2 is not None:
        dw2 = [Kn.to_device_weight(raw2.clone(), t, K, N) for _ in range(nvar)]
        sc = _Scratch(torch.device("cuda", torch.cuda.current_device()))
        y = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)

        def ag(i):
            sp.norm_push(M, nw, 1e-6)
            sp.ag_pending = False
            G.gemm_quant(sp.xn[:M], dw2[i], y, sc, ag=sp.ag_args())
        ms_ag = time_launches(ag, nvar)
        out.append({"kernel": f"norm_push + allgather_wait_gemm_q[{qtype}, world=1]", "M": M, "N": K, "K": N,
                    "ms": round(ms_ag, 4), "tflops_of_the_gemm": round(tf / max(ms_ag - ms_np, 1e-6), 1)})
    Kn.check_status()
    sp.close()
    return out


def bench_sustained(M, N, K, qtype="q4_k", secs=2.5):
    """Seconds-long loops of the quantised GEMM, the bf16 tcgen05 GEMM and cuBLAS on one shape with the SM clock and
    board power sampled (read-only nvidia-smi query) every 100 ms: what the kernels sustain under the power cap."""
    import statistics
    import subprocess
    import time
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as Kn
    from hipengine_b200.quant import ggml as Q
    t = {"q4_k": Q.GGMLType.Q4_K, "q6_k": Q.GGMLType.Q6_K, "q8_0": Q.GGMLType.Q8_0}[qtype]
    raw = Q.quantize(torch.randn(N, K, device="cuda") * 0.02, t)
    dws = [Kn.to_device_weight(raw.clone(), t, N, K) for _ in range(8)]
    wb = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(3)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    sc = _Scratch(torch.device("cuda", torch.cuda.current_device()))
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

    def run(name, fn):
        for i in range(5):
            fn(i)
        torch.cuda.synchronize()
        p = subprocess.Popen(["nvidia-smi", f"--id={torch.cuda.current_device()}", "--query-gpu=clocks.sm,power.draw",
                              "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
        time.sleep(0.3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.time()
        e0.record()
        while time.time() - t0 < secs:
            for i in range(50):
                fn(n + i)
            n += 50
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        p.terminate()
        rows = [l.split(",") for l in p.communicate()[0].strip().splitlines()[3:] if "," in l]
        ck = [float(r[0]) for r in rows]
        pw = [float(r[1]) for r in rows]
        return {"kernel": name, "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1),
                "sm_mhz_median": statistics.median(ck) if ck else None,
                "power_w_median": statistics.median(pw) if pw else None, "launches": n}

    res = [run(f"sustained gemm_quant[{qtype}]", lambda i: G.gemm_quant(x, dws[i % 8], out, sc)),
           run("sustained gemm_bf16 (tcgen05)", lambda i: G.gemm_bf16(x, wb[i % 3], out)),
           run("sustained torch.matmul (cuBLAS)", lambda i: torch.matmul(x, wb[i % 3].t(), out=out))]
    G.check_status()
    return res


def gemm_role_counters(M, N, K, qtype="q4_k"):
    """Cycle counters of CTA 0's roles in the quantised GEMM (library variant `prof`: HE_NATIVE_VARIANT=prof after
    `python -m hipengine_b200.core.build --variant=prof`); a no-op table in the product build."""
    import ctypes as C
    from hipengine_b200.core import native as Nn
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as Kn
    from hipengine_b200.quant import ggml as Q
    t = {"q4_k": Q.GGMLType.Q4_K, "q6_k": Q.GGMLType.Q6_K, "q8_0": Q.GGMLType.Q8_0}[qtype]
    raw = Q.quantize(torch.randn(N, K, device="cuda") * 0.02, t)
    dws = [Kn.to_device_weight(raw.clone(), t, N, K) for _ in range(3)]
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    sc = _Scratch(torch.device("cuda", torch.cuda.current_device()))
    if M > 128:
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = lambda i: G.gemm_quant(x, dws[i], out, sc)
    else:
        out = torch.empty(M, N, device="cuda")
        fn = lambda i: G.gemm_quant_splitk(x, dws[i], out, sc)
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    dbg = torch.zeros(32, dtype=torch.int64, device="cuda")
    Nn.lib().he_gemm_q_debug_counters(C.c_void_p(dbg.data_ptr()))
    fn(0)
    torch.cuda.synchronize()
    Nn.lib().he_gemm_q_debug_counters(C.c_void_p(0))
    d = dbg.tolist()
    return {"kernel": f"gemm_quant[{qtype}] role cycles of CTA 0", "M": M, "N": N, "K": K,
            "unpack_warp": {"raw_block_wait": d[0], "expand": d[1], "operand_stage_wait": d[2], "tmem_store": d[3],
                            "super_blocks": d[4]},
            "mma_issuer": {"operand_wait": d[8], "activation_wait": d[9], "accumulator_wait": d[10], "total": d[11],
                           "k_blocks": d[12]},
            "raw_block_producer": {"free_stage_wait": d[16], "total": d[17], "stages": d[18]}}


def bench_decode_step(rows_list, model="qwen35-27b", ctx=1024, small_rows=None):
    """Whole-model packed decode step (captured graph) at R concurrent rows, each at context `ctx`: the cost a
    continuous-batching round or a verify chain pays.  `small_rows` overrides the row count up to which the int8 GEMV
    path is taken (above it the split-K tensor-core path streams the quantised blocks once for all rows)."""
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models import make_executor
    from hipengine_b200.models.config import NAMED_CONFIGS
    from hipengine_b200.models.decode_graph import DecodeGraphRunner
    cfg = NAMED_CONFIGS[model]
    R = max(rows_list)
    w = build_random_model(cfg, seed=0, device="cuda", recipe="q4_k_m")
    ex = make_executor(w, device="cuda", max_slots=R, max_context=ctx + 64)
    del w
    if small_rows is not None:
        ex.small_rows = small_rows
    runner = DecodeGraphRunner(ex, max_rows=R)
    out = []
    for r in rows_list:
        runner.set_rows(list(range(r)), [7] * r, [ctx - 1] * r)
        for _ in range(3):
            runner.step(r, ctx + 48)
        torch.cuda.synchronize()
        n = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            runner.step(r, ctx + 48)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        out.append({"kernel": f"decode_step[{model}]", "rows": r, "ctx": ctx, "small_rows": ex.small_rows,
                    "ms_per_step": round(ms, 3), "tok_s_aggregate": round(r * 1e3 / ms, 1)})
        runner.set_rows(list(range(r)), [7] * r, [ctx - 1] * r)
    from hipengine_b200.ops import kernels as Kn
    Kn.check_status()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemmq", "gemv", "gdn", "conv", "attn", "fusedar", "seqpar", "step",
                                     "sustained", "roles", "all"])
    ap.add_argument("--rows-list", default="1,2,4,8,16,32,64")
    ap.add_argument("--model", default="qwen35-27b")
    ap.add_argument("--small-rows", type=int, default=None)
    ap.add_argument("--t", type=int, default=4096)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=17408)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--qtype", default="q4_k")
    ap.add_argument("--impl", default="tcgen05")
    ap.add_argument("--phases", type=int, default=0, help="fusedar: phase mask to time (0 = 1, 3 and 7 in turn)")
    a = ap.parse_args()
    out = []
    if a.what == "gemm":
        out.append(bench_gemm(a.m, a.n, a.k, a.impl))
    elif a.what == "gemmq":
        out.append(bench_gemm_quant(a.m, a.n, a.k, a.qtype))
    elif a.what == "gemv":
        out.append(bench_gemv(a.n, a.k, a.qtype, a.rows))
    elif a.what == "gdn":
        out.append(bench_gdn_scan(a.t))
        out.append(bench_gdn_scan(a.t, chunked=True))
    elif a.what == "conv":
        out.append(bench_conv(a.t))
    elif a.what == "attn":
        out.append(bench_attn_decode(a.ctx, rows=a.rows))
    elif a.what == "seqpar":
        out += bench_seq_parallel_loopback(a.m, a.n, a.k, a.qtype)
    elif a.what == "sustained":
        out += bench_sustained(a.m, a.n, a.k, a.qtype)
    elif a.what == "roles":
        out.append(gemm_role_counters(a.m, a.n, a.k, a.qtype))
    elif a.what == "step":
        out += bench_decode_step([int(x) for x in a.rows_list.split(",")], a.model, a.ctx, a.small_rows)
    elif a.what == "fusedar":
        for ph in ([1, 3, 7] if a.phases == 0 else [a.phases]):
            out.append(bench_fused_allreduce_gemm(a.m, a.n, a.k, ph))
    else:
        for (m, n, k) in [(4096, 10240, 5120), (4096, 34816, 5120), (4096, 5120, 17408), (4096, 5120, 6144)]:
            out.append(bench_gemm(m, n, k, "tcgen05"))
            out.append(bench_gemm(m, n, k, "cublas"))
            out.append(bench_gemm_quant(m, n, k, "q4_k"))
        out.append(bench_gemm_quant(4096, 5120, 17408, "q6_k"))
        out.append(bench_gemm_quant(4096, 5120, 5120, "q8_0"))
        for m in (16, 64, 128):
            for (n, k, q) in [(34816, 5120, "q4_k"), (5120, 17408, "q6_k"), (10240, 5120, "q4_k")]:
                out.append(bench_gemm_quant(m, n, k, q))
        for (n, k, q) in [(34816, 5120, "q4_k"), (5120, 17408, "q4_k"), (5120, 17408, "q6_k"), (16384, 5120, "q4_k"),
                          (5120, 6144, "q4_k"), (62080, 5120, "q6_k"), (8192, 5120, "q8_0")]:
            for r in (1, 4):
                out.append(bench_gemv(n, k, q, r))
        out.append(bench_gdn_scan(4096))
        out.append(bench_gdn_scan(4096, chunked=True))
        out.append(bench_conv(4096))
        for c in (4096, 32768):
            out.append(bench_attn_decode(c))
    for o in out:
        print(json.dumps(o))


if __name__ == "__main__":
    sys.path.insert(0, str(ROOT))
    main()
