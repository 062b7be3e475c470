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


def _group_worker(rank: int, world: int, port: int, q, drop_rank: int):
    """One rank of a serving group on the CPU reference runner: rank 0 takes the requests (at its own pace), the
    others only follow rank 0's command batches."""
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import time
    from hipengine_b200.config import EngineConfig
    from hipengine_b200.generation.engine_service import engine_from_runner
    from hipengine_b200.generation.runner import CpuReferenceRunner
    from hipengine_b200.generation.types import GenerationRequest
    from hipengine_b200.loading.synth import build_random_model
    from hipengine_b200.models.config import TINY_DENSE
    from hipengine_b200.parallel.groups import init_distributed
    from hipengine_b200.parallel.serving import GroupCoordinator
    ctx = init_distributed(backend="gloo", timeout_s=60)
    try:
        cfg = EngineConfig()
        w = build_random_model(TINY_DENSE, seed=0, std=0.05)
        coord = GroupCoordinator(rank, world, follower_timeout_s=2.0, leader_timeout_s=20.0)
        svc = engine_from_runner(CpuReferenceRunner(w, cfg, None), cfg, coordinator=coord)
        reqs = [GenerationRequest(request_id=i + 1, prompt_token_ids=[3 + i, 5, 7, 11 + i], max_tokens=4 + i,
                                  ignore_eos=True) for i in range(3)]
        if rank == 0:
            cols = []
            for r in reqs:                                   # arrivals spread over several scheduling rounds
                cols.append(svc.submit(r))
                time.sleep(0.03)
            outs = []
            for c in cols:
                svc._wait(c)
                outs.append(list(c.output.token_ids))
            if drop_rank < 0:
                svc.close()
                q.put((rank, outs))
            else:
                # a follower is gone: its acknowledgements stop, rank 0 notices on the host within the follower
                # timeout (2 s here) and the service turns unhealthy before it launches another step
                time.sleep(4.5)
                try:
                    c = svc.submit(GenerationRequest(request_id=99, prompt_token_ids=[1, 2, 3], max_tokens=2))
                    svc._wait(c)
                    q.put((rank, "no failure seen"))
                except Exception as exc:
                    q.put((rank, "unhealthy" if svc.unhealthy is not None or "stopped" in str(exc) else repr(exc)))
        else:
            if rank == drop_rank:
                # leave between steps, once the three requests are through (nothing of this rank is in flight)
                t0 = time.time()
                while len(svc.orphans) < 3 and time.time() - t0 < 30:
                    time.sleep(0.01)
                q.put((rank, [list(svc.orphans[i + 1].token_ids) for i in range(3)]))
                q.close()
                q.join_thread()
                os._exit(0)
            svc.thread.join(timeout=60)                      # returns when rank 0 publishes the stop batch
            q.put((rank, [list(svc.orphans[i + 1].token_ids) for i in range(3)]))
    except Exception as exc:
        q.put((rank, repr(exc)))
    finally:
        try:
            torch.distributed.destroy_process_group()
        except Exception:
            pass


def _run_group(drop_rank: int):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 200 + (50 if drop_rank >= 0 else 0)
    procs = [ctx.Process(target=_group_worker, args=(r, 2, port, q, drop_rank)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return res


def test_serving_group_rank0_decides_followers_mirror():
    res = _run_group(-1)
    assert isinstance(res[0], list) and res[0] == res[1], res
    assert [len(t) for t in res[0]] == [4, 5, 6]


def test_serving_group_follower_loss_turns_leader_unhealthy():
    res = _run_group(1)
    assert isinstance(res[1], list) and len(res[1]) == 3, res
    assert res[0] == "unhealthy", res
