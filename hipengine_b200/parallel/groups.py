"""Process-group setup and small host-side collectives.

One process per GPU, launched by ``torchrun`` (``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` from the
environment).  ``nccl`` on GPUs, ``gloo`` for CPU tests.  The reference engine is single-device; this layer has
no counterpart there.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistContext:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    group: Optional[object] = None
    backend: str = "none"

    @property
    def is_distributed(self) -> bool:
        return self.world > 1

    def barrier(self) -> None:
        if self.is_distributed:
            if self.backend == "nccl":
                dist.barrier(group=self.group, device_ids=[self.local_rank])
            else:
                dist.barrier(group=self.group)

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.is_distributed:
            dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, *t.shape] gathered along a new leading axis."""
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        if self.is_distributed:
            dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=self.group)
        else:
            out[0].copy_(t)
        return out

    def broadcast_(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.is_distributed:
            dist.broadcast(t, src=src, group=self.group)
        return t


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> DistContext:
    """Join the default process group described by the environment (no-op context for a single process)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world == 1:
        return DistContext(0, 1, local, device, None, "none")
    backend = backend or ("nccl" if use_cuda else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if not dist.is_initialized():
        kw = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return DistContext(rank, world, local, device, dist.group.WORLD, backend)


def max_over_ranks(ctx: DistContext, value: float) -> float:
    """Largest ``value`` on any rank (device-timed numbers are reported as the max over ranks)."""
    if not ctx.is_distributed:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=ctx.device if ctx.backend == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.group)
    return float(t.item())


def merge_argmax(vals: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Vocab-parallel argmax merge: ``vals``/``ids`` are [world, R] per-shard maxima and *global* token ids;
    the lower id wins exact ties, as a single-device argmax over the concatenated logits would."""
    best = vals.max(dim=0, keepdim=True).values
    cand = torch.where(vals == best, ids, torch.full_like(ids, torch.iinfo(ids.dtype).max))
    return cand.min(dim=0).values
