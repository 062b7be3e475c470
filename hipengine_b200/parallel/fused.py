"""Symmetric peer-mapped buffers and the fused push all-reduce + residual add (``csrc/comm.cu``).

Set-up (once per executor): every rank allocates one region with ``cudaMalloc`` through the native library,
exports a CUDA IPC handle, the handles are exchanged with ``all_gather_object`` and every rank opens its peers'
regions.  After that a reduction is one kernel launch with no host involvement, safe to capture in a CUDA
graph.  Single node only (IPC handles do not cross hosts).
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from ..core import native as N
from ..ops import kernels as K
from .groups import DistContext

_MAX_WORLD = 8


class _CommArgs(C.Structure):
    _fields_ = [("data", C.c_void_p * _MAX_WORLD), ("flags", C.c_void_p * _MAX_WORLD), ("epoch", C.c_void_p),
                ("partial", C.c_void_p), ("resid", C.c_void_p), ("out", C.c_void_p),
                ("ld_resid", C.c_longlong), ("ld_out", C.c_longlong),
                ("rows", C.c_int), ("width", C.c_int), ("slot_floats", C.c_int),
                ("world", C.c_int), ("rank", C.c_int), ("status", C.c_void_p), ("wait_limit", C.c_uint)]


class FusedReducer:
    """All-reduce of up to ``max_rows x width`` fp32 rows across the ranks of ``ctx``, added into a residual."""

    def __init__(self, ctx: DistContext, width: int, max_rows: int = 8, n_ctas: int = 16,
                 wait_limit: int = 1 << 22):
        L = N.lib()
        assert L.he_comm_args_size() == C.sizeof(_CommArgs), "ABI mismatch for CommArgs"
        assert ctx.world <= _MAX_WORLD and width % 4 == 0
        self.ctx, self.width, self.max_rows = ctx, width, max_rows
        self.n_ctas = min(n_ctas, L.he_comm_max_ctas())
        self.wait_limit = wait_limit
        self.slot_floats = max_rows * width
        self.data_bytes = 2 * ctx.world * self.slot_floats * 4
        self.flag_bytes = 2 * ctx.world * L.he_comm_max_ctas() * 4
        total = self.data_bytes + self.flag_bytes
        base = C.c_void_p()
        N.check(L.he_comm_alloc(C.c_longlong(total), C.byref(base)), "he_comm_alloc")
        self._local = base.value
        hsz = L.he_comm_ipc_handle_size()
        handle = (C.c_char * hsz)()
        N.check(L.he_comm_ipc_get(C.c_void_p(self._local), handle), "he_comm_ipc_get")
        handles: List[bytes] = [b""] * ctx.world
        dist.all_gather_object(handles, bytes(handle.raw), group=ctx.group)
        self._peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r in range(ctx.world):
            if r == ctx.rank:
                self._peer_ptrs.append(self._local)
                continue
            p = C.c_void_p()
            buf = (C.c_char * hsz).from_buffer_copy(handles[r])
            N.check(L.he_comm_ipc_open(buf, C.byref(p)), "he_comm_ipc_open")
            self._peer_ptrs.append(p.value)
            self._opened.append(p.value)
        self.epoch = torch.zeros(L.he_comm_max_ctas(), dtype=torch.int32, device=ctx.device)
        self.partial = torch.zeros(max_rows, width, dtype=torch.float32, device=ctx.device)
        ctx.barrier()           # every rank has zeroed and mapped its region before the first kernel runs
        self.calls = 0

    @classmethod
    def loopback(cls, device, width: int, world: int = 2, rank: int = 0, max_rows: int = 8, n_ctas: int = 4,
                 wait_limit: int = 2000) -> "FusedReducer":
        """Single-process instance whose "peers" all alias this process's own region.  Only rank ``rank`` ever
        runs, so the other ranks' stamps never arrive: used to exercise the bounded wait (it must give up after
        ``wait_limit`` polls, record a status and leave the residual untouched) without any second GPU."""
        L = N.lib()
        self = cls.__new__(cls)
        self.ctx = DistContext(rank, world, 0, torch.device(device), None, "loopback")
        self.width, self.max_rows = width, max_rows
        self.n_ctas, self.wait_limit = n_ctas, wait_limit
        self.slot_floats = max_rows * width
        self.data_bytes = 2 * world * self.slot_floats * 4
        self.flag_bytes = 2 * world * L.he_comm_max_ctas() * 4
        base = C.c_void_p()
        N.check(L.he_comm_alloc(C.c_longlong(self.data_bytes + self.flag_bytes), C.byref(base)), "he_comm_alloc")
        self._local = base.value
        self._peer_ptrs = [self._local] * world
        self._opened = []
        self.epoch = torch.zeros(L.he_comm_max_ctas(), dtype=torch.int32, device=device)
        self.partial = torch.zeros(max_rows, width, dtype=torch.float32, device=device)
        self.calls = 0
        return self

    def local_rows(self, rows: int) -> torch.Tensor:
        """Staging rows the producer kernel writes its partial products to."""
        return self.partial[:rows]

    def reduce_add(self, resid: torch.Tensor, rows: int, out: torch.Tensor = None) -> None:
        """resid[:rows] += sum over ranks of each rank's ``local_rows(rows)`` (one kernel, no host sync)."""
        a = _CommArgs()
        for r, p in enumerate(self._peer_ptrs):
            a.data[r] = p
            a.flags[r] = p + self.data_bytes
        a.epoch = self.epoch.data_ptr()
        a.partial = self.partial.data_ptr()
        a.resid = resid.data_ptr() if resid is not None else None
        a.out = out.data_ptr() if out is not None else None
        a.ld_resid = resid.stride(0) if resid is not None else 0
        a.ld_out = out.stride(0) if out is not None else 0
        a.rows, a.width, a.slot_floats = rows, self.width, self.slot_floats
        a.world, a.rank = self.ctx.world, self.ctx.rank
        a.status = K.status_tensor(self.ctx.device).data_ptr()
        a.wait_limit = self.wait_limit
        N.check(N.lib().he_comm_push_reduce(C.byref(a), C.c_int(self.n_ctas), K._stream()), "he_comm_push_reduce")
        self.calls += 1

    def close(self) -> None:
        L = N.lib()
        torch.cuda.synchronize()
        if self.ctx.backend != "loopback":
            self.ctx.barrier()
        for p in self._opened:
            L.he_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self._local:
            L.he_comm_free(C.c_void_p(self._local))
            self._local = 0
