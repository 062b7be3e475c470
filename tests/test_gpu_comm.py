"""Peer-memory reduction kernel on one GPU: the single-rank case, and the bounded wait giving up cleanly."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_world_of_one_reduces_to_residual_add():
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import FusedReducer
    red = FusedReducer.loopback("cuda", width=512, world=1, rank=0)
    try:
        h = torch.arange(3 * 512, dtype=torch.float32, device="cuda").reshape(3, 512).clone()
        want = h.clone()
        for it in range(5):                                # several calls: phases alternate, epochs advance
            red.local_rows(3).copy_(torch.full((3, 512), float(it + 1), device="cuda"))
            red.reduce_add(h, 3)
            want += it + 1
        torch.cuda.synchronize()
        K.check_status("cuda")
        torch.testing.assert_close(h, want)
    finally:
        red.close()


def test_wait_for_absent_peer_times_out_with_status():
    """Rank 1 never runs, so its stamp never arrives: the kernel must stop polling after its limit, set the status
    word, leave the residual alone and leave the context usable."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import FusedReducer
    red = FusedReducer.loopback("cuda", width=256, world=2, rank=0, wait_limit=500)
    try:
        h = torch.ones(2, 256, device="cuda")
        red.local_rows(2).fill_(5.0)
        red.reduce_add(h, 2)
        torch.cuda.synchronize()                           # returns: the wait was bounded
        with pytest.raises(RuntimeError, match="status 1"):
            K.check_status("cuda")
        assert torch.equal(h, torch.ones(2, 256, device="cuda"))
        K.check_status("cuda")                             # the word was cleared; the context still works
        assert float((h * 2).sum()) == 2 * 2 * 256
    finally:
        red.close()


def _ref_add(h, xs, ws):
    acc = torch.zeros_like(h, dtype=torch.float64)
    for x, w in zip(xs, ws):
        # each rank's partial tile is rounded to bf16 before the fp32 sum, and the sum is rounded to bf16 once more
        acc += (x.double() @ w.double().t()).float().bfloat16().double()
    return h + acc.float().bfloat16().float()


@pytest.mark.parametrize("direct", [True, False], ids=["one_hop", "owner"])
@pytest.mark.parametrize("n", [512, 640])
def test_fused_gemm_allreduce_world_of_one(n, direct):
    """One rank: the single kernel runs GEMM, stage, reduce and residual add with its own CTAs waiting on each
    other's stamps; several calls with different row counts advance the device-side epoch."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import FusedGemmAllReduce
    from hipengine_b200.parallel.groups import DistContext
    ctx = DistContext(0, 1, 0, torch.device("cuda", torch.cuda.current_device()), None, "none")
    fg = FusedGemmAllReduce(ctx, width=n, max_rows=1024, direct=direct)
    try:
        g = torch.Generator(device="cuda").manual_seed(3)
        w = (torch.randn(n, 384, device="cuda", generator=g) * 0.05).bfloat16()
        for rows in (300, 1000, 64, 300):
            x = torch.randn(rows, 384, device="cuda", generator=g).bfloat16()
            h = torch.randn(rows, n, device="cuda", generator=g)
            want = _ref_add(h, [x], [w])
            fg.gemm_add(x, w, h)
            torch.cuda.synchronize()
            K.check_status("cuda")
            torch.testing.assert_close(h, want, rtol=2e-2, atol=2e-2)
        assert int(fg.sync[0].item()) == 4 and int(fg.sync[1].item()) == 0
    finally:
        fg.close()


@pytest.mark.parametrize("world,direct", [(2, True), (2, False), (4, False), (4, True), (8, False)])
def test_fused_gemm_allreduce_emulated_ranks(world, direct):
    """Several ranks emulated on one GPU: the phases of both ranks run as separate launches in an order in which no
    launch waits for a later one (all phase 1, all phase 2, all phase 3); each rank holds a slice of K."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import FusedGemmAllReduce
    ranks = FusedGemmAllReduce.emulated_group("cuda", width=768, world=world, max_rows=512, direct=direct)
    try:
        g = torch.Generator(device="cuda").manual_seed(5)
        ws = [(torch.randn(768, 256, device="cuda", generator=g) * 0.05).bfloat16() for _ in range(world)]
        for rows in (200, 512):
            xs = [torch.randn(rows, 256, device="cuda", generator=g).bfloat16() for _ in range(world)]
            h0 = torch.randn(rows, 768, device="cuda", generator=g)
            hs = [h0.clone() for _ in range(world)]
            want = _ref_add(h0, xs, ws)
            for phase in (1, 2, 4):
                for r in range(world):
                    ranks[r].gemm_add(xs[r], ws[r], hs[r], phases=phase)
            torch.cuda.synchronize()
            K.check_status("cuda")
            torch.testing.assert_close(hs[0], want, rtol=2e-2, atol=3e-2)
            for r in range(1, world):                      # replicated residual streams stay bit-identical
                assert torch.equal(hs[0], hs[r])
    finally:
        for r in ranks[1:]:
            r.close()
        ranks[0].close()


def test_fused_gemm_allreduce_absent_peer_times_out():
    """Only rank 0 of two runs: the stamps of rank 1 never arrive, every wait gives up after its limit, the status
    word is set, the residual is untouched and the context stays usable."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import FusedGemmAllReduce
    ranks = FusedGemmAllReduce.emulated_group("cuda", width=512, world=2, max_rows=256)
    try:
        ranks[0].wait_limit = 500
        x = torch.ones(256, 128, device="cuda").bfloat16()
        w = torch.ones(512, 128, device="cuda").bfloat16()
        h = torch.ones(256, 512, device="cuda")
        ranks[0].gemm_add(x, w, h)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="status 1"):
            K.check_status("cuda")
        assert torch.equal(h, torch.ones(256, 512, device="cuda"))
        K.check_status("cuda")
    finally:
        for r in ranks[1:]:
            r.close()
        ranks[0].close()


def _q4k(n, k, seed):
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.quant import ggml as Q
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(n, k, generator=g, device="cuda") * 0.05
    raw = Q.quantize(w, Q.GGMLType.Q4_K)
    return K.to_device_weight(raw, Q.GGMLType.Q4_K, n, k)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_folded_decode_allreduce_push_epilogue_and_reduce_prologue(world):
    """Tensor-parallel decode without a stand-alone reduction: each emulated rank's row-parallel GEMV pushes its
    partial rows from the epilogue, the next GEMV's prologue sums them into the residual.  All ranks' pushes are
    launched before any reduce, so no launch waits for a later one.  Three rounds exercise both slot parities."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import PeerResidual
    width, kq, n2, R = 1024, 512, 768, 3
    group = PeerResidual.emulated_group("cuda", width, world)
    w_out = [_q4k(width, kq, 10 + q) for q in range(world)]
    w_next = _q4k(n2, width, 99)
    nw = torch.rand(width, device="cuda") + 0.5
    h_ref = torch.randn(R, width, device="cuda")
    hs = [h_ref.clone() for _ in range(world)]
    for rnd in range(3):
        xs = [torch.randn(R, kq, device="cuda") for _ in range(world)]
        parts = []
        for q in range(world):
            p = torch.zeros(R, width, device="cuda")
            K.gemv(xs[q], [K.GemvSegment(w_out[q], p)])
            parts.append(p)
        for q in range(world):
            K.gemv(xs[q], [K.GemvSegment(w_out[q], hs[q])], comm=group[q].comm(K.COMM_PUSH))
        before = [h.clone() for h in hs]
        for p in parts:                       # rank order, like the kernel
            h_ref = h_ref + p
        outs = []
        for q in range(world):
            o = torch.zeros(R, n2, device="cuda")
            K.gemv(hs[q], [K.GemvSegment(w_next, o)], norm_w=nw, comm=group[q].comm(K.COMM_REDUCE))
            outs.append(o)
        torch.cuda.synchronize()
        K.check_status()
        want = torch.zeros(R, n2, device="cuda")
        K.gemv(h_ref, [K.GemvSegment(w_next, want)], norm_w=nw)
        # the reference rows come from the plain multi-row kernel, whose lanes split the blocks differently from the
        # communicating kernel's: equal up to fp32 summation order; the replicas themselves are bit-identical
        tol_h = 1e-5 * h_ref.abs().max().item()
        tol_o = 1e-4 * want.abs().max().item()
        for q in range(world):
            assert not torch.equal(hs[q], before[q])
            assert torch.equal(hs[q], hs[0]) and torch.equal(outs[q], outs[0]), (rnd, q)
            assert torch.allclose(hs[q], h_ref, atol=tol_h, rtol=1e-5), (rnd, q, (hs[q] - h_ref).abs().max())
            assert torch.allclose(outs[q], want, atol=tol_o, rtol=1e-3), (rnd, q, (outs[q] - want).abs().max())
        h_ref = hs[0].clone()                 # the next round starts from what the ranks hold
    # stand-alone producer / consumer on the same regions
    part = [torch.randn(2, width, device="cuda") for _ in range(world)]
    for q in range(world):
        group[q].push_rows(part[q], 2)
    for q in range(world):
        group[q].reduce_in(hs[q], 2)
    torch.cuda.synchronize()
    K.check_status()
    want = h_ref.clone()
    for p in part:
        pass
    acc = part[0].clone()
    for p in part[1:]:
        acc = acc + p
    want[:2] += acc
    for q in range(world):
        assert torch.equal(hs[q], want)
    for g in group:
        g.close()


def test_vocab_parallel_argmax_merge_and_bounded_wait():
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import PeerResidual
    world, R, shard = 4, 5, 1000
    vals = torch.randn(world, R, device="cuda")
    vals[2, 1] = vals[0, 1] = vals[:, 1].max() + 1.0          # exact tie between ranks 0 and 2: lower id wins
    idx = torch.randint(0, shard, (world, R), device="cuda", dtype=torch.int64)
    # one CTA per rank pushes and then waits for the others: emulated ranks would wait for later launches, so the
    # pairs of the other ranks are put in place by running every rank once (bounded waits run out, status is
    # cleared), after which a second pass over the same sequence numbers' slots finds all stamps present
    group = PeerResidual.emulated_group("cuda", 1, world, max_rows=64, wait_limit=200)
    outs = [torch.zeros(R, dtype=torch.int64, device="cuda") for _ in range(world)]
    for q in range(world):
        group[q].argmax_merge(vals[q].contiguous(), idx[q].contiguous(), q * shard, R, outs[q])
    torch.cuda.synchronize()
    st = K.status_tensor("cuda")
    assert int(st[0].item()) == 1                              # the first ranks gave up waiting, as designed
    st.zero_()
    # the last rank saw every stamp: its result is the true merge
    gid = idx + torch.arange(world, device="cuda").view(-1, 1) * shard
    best = vals.max(0).values
    cand = torch.where(vals == best, gid, torch.full_like(gid, 1 << 40))
    assert torch.equal(outs[world - 1], cand.min(0).values)
    for g in group:
        g.close()


@pytest.mark.parametrize("world,T", [(2, 400), (4, 400), (8, 1700)])
def test_sequence_parallel_gemm_reduce_scatter_norm_allgather_emulated(world, T):
    """Sequence-parallel prefill on emulated ranks of one GPU, phase by phase: GEMM -> reduce-scatter -> residual add
    (quantised weight read in place), RMSNorm + all-gather push, the all-gather wait of the consumer GEMM, and the
    final residual gather -- each against plain fp32 PyTorch."""
    from hipengine_b200.models.executor import _Scratch
    from hipengine_b200.ops import gemm as G
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import SeqParallel
    from hipengine_b200.quant import ggml as Q
    H, Kq, N2 = 512, 512, 384
    group = SeqParallel.emulated_group("cuda", H, world, max_rows=2048)
    g = torch.Generator(device="cuda").manual_seed(world)
    h0 = torch.randn(T, H, device="cuda", generator=g)
    xs, dws, deqs = [], [], []
    for q in range(world):
        w = torch.randn(H, Kq, device="cuda", generator=g) * 0.05
        raw = Q.quantize(w, Q.GGMLType.Q4_K)
        deqs.append(Q.dequantize_torch(raw, Q.GGMLType.Q4_K, H, Kq))
        dws.append(K.to_device_weight(raw, Q.GGMLType.Q4_K, H, Kq))
        xs.append((torch.randn(T, Kq, device="cuda", generator=g) * 0.5).bfloat16())
        group[q].h[:T].copy_(h0)
    for ph in (1, 2):
        for q in range(world):
            group[q].gemm_rs(xs[q], dws[q], T, phases=ph)
    torch.cuda.synchronize()
    K.check_status()
    want = h0.clone()
    for q in range(world):
        want += xs[q].float() @ deqs[q].t()
    full = torch.zeros_like(want)
    for q in range(world):
        own = torch.tensor(group[q].owned_rows(T), device="cuda", dtype=torch.long)
        other = torch.ones(T, dtype=torch.bool, device="cuda")
        other[own] = False
        got = group[q].h[:T]
        assert torch.equal(got[other], h0[other])                      # rows of other owners untouched
        if own.numel():
            err = (got[own] - want[own]).abs().max() / want.abs().max()
            assert err < 6e-3, (q, err)                                 # bf16 partials, fp32 sum
            full[own] = got[own]
    # RMSNorm + all-gather: every rank ends up with the same normalised rows of ALL owners
    nw = torch.rand(H, device="cuda", generator=g) + 0.5
    for q in range(world):
        group[q].norm_push(T, nw, 1e-6)
    for q in range(world):
        group[q].wait()
    torch.cuda.synchronize()
    K.check_status()
    ref_xn = (full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-6) * nw)
    for q in range(world):
        assert torch.equal(group[q].xn[:T], group[0].xn[:T])
        assert (group[q].xn[:T].float() - ref_xn).abs().max() < 0.02 * ref_xn.abs().max()
    # consumer GEMM with the all-gather wait inside its TMA producer (stamps already present here)
    w2 = torch.randn(N2, H, device="cuda", generator=g) * 0.05
    raw2 = Q.quantize(w2, Q.GGMLType.Q4_K)
    dw2 = K.to_device_weight(raw2, Q.GGMLType.Q4_K, N2, H)
    out = torch.zeros(T, N2, device="cuda")
    G.gemm_quant(group[1].xn[:T], dw2, out, _Scratch(torch.device("cuda")), ag=group[1].ag_args())
    torch.cuda.synchronize()
    K.check_status()
    ref = group[1].xn[:T].float() @ Q.dequantize_torch(raw2, Q.GGMLType.Q4_K, N2, H).t()
    assert (out - ref).norm() / ref.norm() < 6e-3
    # a consumer whose owner never stamps gives up (bounded) and reports it
    group[0].sp_state[0] += 1
    out.zero_()
    lim_args = list(group[0].ag_args())
    lim_args[3] = 50
    G.gemm_quant(group[0].xn[:T], dw2, out, _Scratch(torch.device("cuda")), ag=tuple(lim_args))
    torch.cuda.synchronize()
    assert int(K.status_tensor("cuda")[0].item()) == 1
    K.status_tensor("cuda").zero_()
    group[0].sp_state[0] -= 1
    # final gather of the residual itself
    for q in range(world):
        group[q]._push(T, None, 0.0, 1)
    for q in range(world):
        group[q].wait()
    torch.cuda.synchronize()
    K.check_status()
    for q in range(world):
        assert torch.equal(group[q].h[:T], full)
    for gq in group:
        gq.close()


@pytest.mark.parametrize("world,T", [(2, 450), (4, 450), (8, 1650)])
def test_rows_reduce_scatter_for_expert_parallel_combine_emulated(world, T):
    """Token-ordered fp32 partial rows of every emulated rank are reduce-scattered into the row-sharded residual:
    owned rows get h + sum over ranks (bf16 on the wire for remote rows), other rows stay untouched."""
    from hipengine_b200.ops import kernels as K
    from hipengine_b200.parallel.fused import SeqParallel
    H = 512
    group = SeqParallel.emulated_group("cuda", H, world, max_rows=2048)
    g = torch.Generator(device="cuda").manual_seed(3)
    h0 = torch.randn(T, H, device="cuda", generator=g)
    parts = [torch.randn(T, H, device="cuda", generator=g) for _ in range(world)]
    for q in range(world):
        group[q].h[:T].copy_(h0)
    for ph in (1, 2):
        for q in range(world):
            group[q].rows_rs(parts[q], T, phases=ph)
    torch.cuda.synchronize()
    K.check_status()
    for q in range(world):
        own = torch.tensor(group[q].owned_rows(T), device="cuda", dtype=torch.long)
        other = torch.ones(T, dtype=torch.bool, device="cuda")
        other[own] = False
        got = group[q].h[:T]
        assert torch.equal(got[other], h0[other])
        if own.numel():
            want = h0[own].clone()
            for r in range(world):
                want += parts[r][own] if r == q else parts[r][own].bfloat16().float()
            assert torch.allclose(got[own], want, atol=1e-5, rtol=1e-5)
    for gq in group:
        gq.close()
