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
