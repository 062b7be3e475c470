"""One engine over a tensor/expert-parallel group: rank 0 decides, every rank executes.

The ranks of a group must launch the same kernels in the same order (their collectives pair up by position).  The
engine loop's decisions depend on when requests arrive, so they are taken once, on rank 0: every tick, rank 0
publishes the batch of commands it drained from its own queue (new requests, cancellations -- including the deadlines
and cancellation tokens it probed itself) and whether to run a scheduling round; every rank, rank 0 included,
applies that batch and runs the round.  Followers never look at a clock.  This is the division of labour the
reference plans for its own tensor-parallel serving (``docs/reference/TENSOR_PARALLEL.md:28-40``: rank 0 owns HTTP,
the scheduler and the sampler; workers follow a broadcast work descriptor); the transport here is a key-value store on rank 0's
host, so that control messages never queue behind device work and rank 0 never blocks on a follower.
"""
from __future__ import annotations

import datetime
import pickle
import time
from dataclasses import replace
from typing import Any, Dict, Optional

import torch.distributed as dist


class GroupFailure(RuntimeError):
    """A rank of the serving group stopped answering (follower heartbeats stale, or rank 0 silent)."""


class GroupCoordinator:
    """Command batches from rank 0 to the other ranks through a key-value store on rank 0's host.

    Rank 0 ``publish``es batch n under its own key and never blocks on a follower; followers ``receive`` by waiting
    for the key and acknowledge with their own counter key.  Rank 0 checks the acknowledgements a few times per
    second: a follower that has not acknowledged within ``follower_timeout_s`` is reported as lost *on the host*,
    before rank 0 launches the next step whose collectives would wait for it; a follower that sees no batch (rank 0
    also publishes an idle heartbeat every second) for ``leader_timeout_s`` gives up likewise.
    """

    def __init__(self, rank: int, world: int, store=None, follower_timeout_s: float = 10.0,
                 leader_timeout_s: float = 30.0, port: Optional[int] = None):
        import os
        self.rank, self.world = rank, world
        self.follower_timeout_s, self.leader_timeout_s = follower_timeout_s, leader_timeout_s
        if store is None:
            host = os.environ.get("MASTER_ADDR", "127.0.0.1")
            port = port or int(os.environ.get("MASTER_PORT", "29500")) + 7
            store = dist.TCPStore(host, port, world, is_master=(rank == 0),
                                  timeout=datetime.timedelta(seconds=max(60.0, leader_timeout_s)))
        self.store = store
        self.batches = 0
        self._last_check = 0.0
        self._progress = {r: (0, time.time()) for r in range(1, world)}
        if rank == 0:
            for r in range(1, world):
                self.store.set(f"he/a/{r}", "0")

    @property
    def is_leader(self) -> bool:
        return self.rank == 0

    def publish(self, batch: Dict[str, Any]) -> None:
        assert self.is_leader
        self.batches += 1
        self.store.set(f"he/b/{self.batches}", pickle.dumps(batch))
        if self.batches > 64:
            try:
                self.store.delete_key(f"he/b/{self.batches - 64}")
            except Exception:
                pass

    def receive(self) -> Dict[str, Any]:
        assert not self.is_leader
        key = f"he/b/{self.batches + 1}"
        try:
            self.store.wait([key], datetime.timedelta(seconds=self.leader_timeout_s))
        except Exception as exc:
            raise GroupFailure(f"rank 0 published nothing for {self.leader_timeout_s:.0f}s: {exc}") from None
        batch = pickle.loads(self.store.get(key))
        self.batches += 1
        self.store.set(f"he/a/{self.rank}", str(self.batches))
        return batch

    def check_followers(self, force: bool = False) -> None:
        """Rank 0, at most four times per second: raise ``GroupFailure`` for a follower whose acknowledgements
        stopped while batches were outstanding."""
        now = time.time()
        if not force and now - self._last_check < 0.25:
            return
        self._last_check = now
        for r in range(1, self.world):
            ack = int(self.store.get(f"he/a/{r}"))
            seen, since = self._progress[r]
            if ack > seen or ack >= self.batches:
                self._progress[r] = (ack, now)
            elif now - since > self.follower_timeout_s:
                raise GroupFailure(f"rank {r} has not acknowledged batch {seen + 1} of {self.batches} for "
                                   f"{now - since:.1f}s")


def portable_request(req):
    """The request as the followers get it: no cancellation token, no deadline (rank 0 turns both into explicit
    cancel commands), nothing that cannot be pickled."""
    return replace(req, cancellation_token=None, deadline_at=None)
