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
