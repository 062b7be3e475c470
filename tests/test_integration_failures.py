"""Failure detection and containment, injected on the host (no GPU is faulted, trapped or hung).

* a runner failure naming some requests fails only those (containment);
* a fatal error in the driver thread marks the service unhealthy and later calls are refused, not blocked;
* a rank that never joins a collective is detected by the process-group timeout on the surviving rank (gloo).
"""
import os
import time

import pytest
import torch
import torch.multiprocessing as mp

from hipengine_b200.config import EngineConfig, SchedulerConfig
from hipengine_b200.generation.engine_service import EngineUnavailable, engine_from_runner
from hipengine_b200.generation.simulator import SimulatedRunner
from hipengine_b200.generation.types import GenerationRequest


def _cfg():
    return EngineConfig(max_sequence_length=1024, scheduler=SchedulerConfig(max_active_requests=4))


def test_contained_failure_spares_other_requests():
    cfg = _cfg()
    runner = SimulatedRunner(cfg, fail_decode_admission=[1])
    eng = engine_from_runner(runner, cfg, None)
    try:
        reqs = [GenerationRequest(prompt_token_ids=list(range(10 + i)), max_tokens=6, ignore_eos=True) for i in range(3)]
        outs = eng.generate(reqs)
        errs = [o for o in outs if o.error]
        assert len(errs) == 1 and "execution_failed" in errs[0].error
        assert all(len(o.token_ids) == 6 for o in outs if not o.error)
        # the failed request's slot and pages were reclaimed: a new request still runs
        again = eng.generate([GenerationRequest(prompt_token_ids=[1, 2, 3], max_tokens=3, ignore_eos=True)])
        assert again[0].error is None and len(again[0].token_ids) == 3
    finally:
        eng.close()


class _Exploding(SimulatedRunner):
    def decode(self, rows):
        raise ValueError("driver-thread bug")


def test_fatal_error_marks_service_unhealthy():
    cfg = _cfg()
    eng = engine_from_runner(_Exploding(cfg), cfg, None)
    try:
        out = eng.generate([GenerationRequest(prompt_token_ids=[1, 2, 3], max_tokens=4, ignore_eos=True)])[0]
        assert out.error and "engine_unavailable" in out.error
        t0 = time.time()
        with pytest.raises(EngineUnavailable):
            eng.generate([GenerationRequest(prompt_token_ids=[1], max_tokens=1)])
        assert time.time() - t0 < 5.0                      # refused at once, not after a timeout
        assert eng.unhealthy["exception_type"] == "ValueError"
    finally:
        eng.close()


def _rank(rank, world, port, q):
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                                     # step 1: everyone present
    if rank == 1:
        q.put((rank, "left"))                              # leaves between steps, nothing in flight
        q.close()
        q.join_thread()
        os._exit(0)
    t0 = time.time()
    try:
        dist.all_reduce(t)                                 # step 2: the peer is gone
        q.put((rank, "no error"))
    except Exception as exc:
        q.put((rank, f"detected after {time.time() - t0:.1f}s: {type(exc).__name__}"))
    q.close()
    q.join_thread()
    os._exit(0)


def test_missing_rank_is_detected_by_collective_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 100
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=60) for _ in ps)
    for p in ps:
        p.join(timeout=30)
    assert res[1] == "left"
    assert res[0].startswith("detected"), res


def test_unhealthy_report_carries_recent_engine_events():
    """The flight recorder rides on the unhealthy report: a failed engine says what it was doing."""
    cfg = _cfg()
    eng = engine_from_runner(_Exploding(cfg), cfg, None)
    try:
        out = eng.generate([GenerationRequest(prompt_token_ids=[1, 2, 3], max_tokens=4, ignore_eos=True)])[0]
        assert out.error
        assert eng.unhealthy is not None
        kinds = [e["kind"] for e in eng.unhealthy["recent_events"]]
        assert "submit" in kinds and kinds[-1] == "fatal"
    finally:
        eng.close()


class _Stuck(SimulatedRunner):
    """A runner whose decode blocks the driver thread (a wedged device from the front end's point of view)."""
    def __init__(self, cfg, gate):
        super().__init__(cfg)
        self.gate = gate

    def decode(self, rows):
        self.gate.wait(timeout=20)
        return super().decode(rows)


def test_command_that_is_not_served_in_time_raises_instead_of_blocking():
    import threading
    from dataclasses import replace
    from hipengine_b200.generation.engine_service import EngineCommandTimeout
    gate = threading.Event()
    cfg = replace(_cfg(), command_timeout_seconds=0.3)
    eng = engine_from_runner(_Stuck(cfg, gate), cfg, None)
    try:
        col = eng.submit(GenerationRequest(prompt_token_ids=[1, 2, 3], max_tokens=3, ignore_eos=True))
        time.sleep(0.2)                                        # the driver is now inside the stuck decode
        t0 = time.time()
        with pytest.raises(EngineCommandTimeout, match="snapshot"):
            eng.snapshot()
        assert 0.25 < time.time() - t0 < 3.0                   # after the liveness budget, not forever
        gate.set()
        assert col.done.wait(timeout=10) and len(col.output.token_ids) == 3      # the engine itself was fine
        assert isinstance(eng.snapshot(), dict)
    finally:
        gate.set()
        eng.close()


def test_stream_many_interleaves_requests_and_delivers_every_token_once():
    cfg = _cfg()
    eng = engine_from_runner(SimulatedRunner(cfg), cfg, None)
    try:
        reqs = [GenerationRequest(prompt_token_ids=list(range(5 + i)), max_tokens=4 + i, ignore_eos=True) for i in range(3)]
        want = [o.token_ids for o in eng.generate([GenerationRequest(prompt_token_ids=list(r.prompt_token_ids),
                                                                     max_tokens=r.max_tokens, ignore_eos=True)
                                                   for r in reqs])]
        got = {0: [], 1: [], 2: []}
        order = []
        finished = set()
        for i, ch in eng.stream_many(reqs):
            assert i not in finished
            got[i] += ch.token_ids
            order.append(i)
            if ch.finished:
                finished.add(i)
        assert [got[i] for i in range(3)] == want and finished == {0, 1, 2}
        assert order != sorted(order)                          # chunks of different requests interleave
    finally:
        eng.close()


@pytest.mark.parametrize("policy", ["protect_decode", "protect_ttft", "fair", "token_budget"])
@pytest.mark.parametrize("prefix,spec_depth", [("radix", 0), ("off", 0), ("radix", 3)])
def test_churn_of_submits_cancels_and_contained_failures_leaves_the_books_balanced(policy, prefix, spec_depth):
    """Sixty requests with shared prefixes arrive at random, a third are cancelled at random moments (pending, in
    prefill, in decode), three fail inside decode (or inside a speculative cycle's verify), the pool is small enough to evict cached prefixes and to make
    admissions wait.  When the loop runs dry every request has finished exactly once, every slot is back, no lease or
    page credit is left, the only pages in use are the prefix cache's, and clearing the cache frees the whole pool."""
    import random
    from hipengine_b200.config import EngineConfig, KVConfig, SchedulerConfig, SpeculativeConfig
    from hipengine_b200.generation.engine_loop import EngineLoop
    from hipengine_b200.generation.scheduler import GenerationAdmissionRejected
    from hipengine_b200.generation.simulator import SimulatedRunner
    from hipengine_b200.generation.types import GenerationRequest
    rng = random.Random(7)
    cfg = EngineConfig(max_sequence_length=256, kv=KVConfig(prefix_cache=prefix),
                       scheduler=SchedulerConfig(max_active_requests=4, policy=policy, max_pending_requests=16),
                       speculative=SpeculativeConfig(mode="mtp" if spec_depth else "off", draft_depth=max(1, spec_depth)))
    runner = SimulatedRunner(cfg, kv_capacity_tokens=1024, fail_decode_admission=[3, 11, 17], spec_depth=spec_depth,
                             spec_accept_rate=0.6)
    loop = EngineLoop(runner, cfg)
    finished = []
    loop.on_event = lambda rs: finished.append(rs.rid) if rs.finish is not None else None
    shared = [rng.randrange(5, 900) for _ in range(48)]
    live, refused = [], 0
    for _ in range(400):
        r = rng.random()
        if r < 0.35 and len(live) + refused < 60:
            head = shared[:rng.choice([16, 32, 48])] if rng.random() < 0.5 else []
            prompt = head + [rng.randrange(5, 900) for _ in range(rng.randrange(1, 40))]
            try:
                live.append(loop.submit(GenerationRequest(prompt_token_ids=prompt, max_tokens=rng.randrange(1, 60),
                                                          ignore_eos=True)).rid)
            except GenerationAdmissionRejected:
                refused += 1                                   # the pending queue was full
        elif r < 0.45 and live:
            loop.cancel(rng.choice(live))                      # may name a finished request: a no-op
        loop.tick()
        runner.kv.radix.assert_consistent()
    for _ in range(5000):
        if loop.idle():
            break
        loop.tick()
    assert loop.idle() and sorted(finished) == sorted(live)    # each exactly once
    c = loop.sched.counters
    assert c["finished"] == len(live) and c["failed"] == 3 and c["cancelled"] >= 5
    assert (c["spec_cycles"] > 0) == (spec_depth > 0)        # failures inside a verify are contained the same way
    assert (c["cached_prompt_tokens"] > 0) == (prefix == "radix")
    assert sorted(runner.free_slots) == [0, 1, 2, 3]
    snap = runner.kv.pool.snapshot()
    assert snap["leases"] == 0 and snap["pages_credit"] == 0 and snap["pages_used"] == snap["pages_cached"]
    assert (snap["pages_cached"] > 0) == (prefix == "radix")
    runner.kv.radix.clear()                                    # hands its pages back through the release hook
    snap = runner.kv.pool.snapshot()
    assert snap["pages_free"] == snap["pages_total"] and snap["pages_used"] == 0


def test_posted_cancel_ends_a_stream_without_the_caller_waiting_for_a_tick():
    """``cancel(..., wait=False)`` only posts the command (what the HTTP routes do from the event loop when a client
    disconnects); the driver serves it before its next tick, the stream ends with the cancel reason, nothing stays
    active, and the context fit used by the stream pre-check is asked from the driver only once."""
    from hipengine_b200 import LLM, SamplingParams
    llm = LLM("tiny-dense", backend="cpu_reference", max_active_requests=2, max_sequence_length=512)
    try:
        eng = llm._get_engine()
        req = llm._request(list(range(5, 25)), SamplingParams(max_tokens=400, ignore_eos=True), 0)
        seen, last = 0, None
        for ch in eng.stream(req):
            seen += len(ch.token_ids)
            last = ch
            if seen == 3:
                assert eng.cancel(req.request_id, wait=False) is True
        assert last.finished and last.finish.reason == "cancelled" and 3 <= seen < 400
        snap = llm.live_loop_snapshot()
        assert snap["active"] == 0 and snap["pending"] == 0 and snap["counters"]["cancelled"] == 1
        assert eng.cancel(req.request_id) is False                      # already gone: the waiting form says so
        calls = []
        real = llm.resident_capacity_estimate
        llm.resident_capacity_estimate = lambda: calls.append(1) or real()
        llm._served_context = None
        assert [llm.fit_context([1] * n, 10)["fits_with_max_tokens"] for n in (10, 502, 503)] == [True, True, False]
        assert len(calls) == 1
    finally:
        llm.close()
