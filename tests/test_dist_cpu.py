"""Host-side distributed plumbing on CPU ranks (gloo, world size 2)."""
import os

import torch
import torch.multiprocessing as mp


def _worker(rank: int, world: int, port: int, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from hipengine_b200.parallel.groups import init_distributed, max_over_ranks, merge_argmax
    ctx = init_distributed(backend="gloo", timeout_s=60)
    try:
        assert ctx.world == world and ctx.rank == rank and ctx.backend == "gloo"
        t = torch.full((4,), float(rank + 1))
        ctx.all_reduce_(t)
        assert torch.equal(t, torch.full((4,), 3.0))
        assert max_over_ranks(ctx, 10.0 + rank) == 11.0
        # vocab-parallel greedy: every rank owns half of a 10-token vocabulary
        logits = torch.tensor([[0.1, 0.9, 0.3, 0.9, 0.2, 0.0, 0.9, -1.0, 0.5, 0.4],
                               [0.0, 0.0, 0.0, 0.0, 0.0, 2.0, 0.0, 0.0, 0.0, 2.0]])
        lo = rank * 5
        loc = logits[:, lo:lo + 5]
        v, i = loc.max(-1)
        vals, ids = ctx.all_gather(v), ctx.all_gather(i + lo)
        merged = merge_argmax(vals, ids)
        assert merged.tolist() == [1, 5], merged            # ties resolve to the lower global id
        g = ctx.all_gather(torch.tensor([rank]))
        assert g.flatten().tolist() == [0, 1]
        ctx.barrier()
        q.put((rank, "ok"))
    except Exception as exc:  # surfaced by the parent
        q.put((rank, repr(exc)))
    finally:
        torch.distributed.destroy_process_group()


def test_gloo_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
