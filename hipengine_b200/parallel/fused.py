"""Symmetric peer-mapped buffers and the fused push all-reduce + residual add (``csrc/comm.cu``).

Set-up (once per executor): every rank allocates one region with ``cudaMalloc`` through the native library,
exports a CUDA IPC handle, the handles are exchanged with ``all_gather_object`` and every rank opens its peers'
regions.  After that a reduction is one kernel launch with no host involvement, safe to capture in a CUDA
graph.  Single node only (IPC handles do not cross hosts).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

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


class _FuseArgs(C.Structure):
    _fields_ = [("stage", C.c_void_p * _MAX_WORLD), ("result", C.c_void_p * _MAX_WORLD),
                ("flags", C.c_void_p * _MAX_WORLD), ("sync", C.c_void_p), ("resid", C.c_void_p),
                ("ld_resid", C.c_longlong), ("world", C.c_int), ("rank", C.c_int), ("max_tiles", C.c_int),
                ("owned_cap", C.c_int), ("phases", C.c_int), ("wait_limit", C.c_uint), ("direct", C.c_int),
                ("reserved", C.c_int)]


class FusedGemmAllReduce:
    """Row-parallel projection for many rows: ``resid += all_reduce(x_rank @ W_rank^T)`` as ONE tcgen05 kernel per
    rank (``csrc/gemm_sm100.cu::gemm_bf16_allreduce_kernel``).

    The GEMM epilogue stores each partial tile into the stage buffer of the tile's owner rank through peer memory
    while later tiles are still in the tensor cores; owners sum in rank order and write the bf16 result into every
    rank, and each rank adds it into its fp32 residual -- all behind bounded per-warp flag waits.  Regions are plain
    device allocations shared through CUDA IPC (single node).  The reference engine is single-device: no counterpart.
    """

    def __init__(self, ctx: DistContext, width: int, max_rows: int = 4096, wait_limit: int = 1 << 24,
                 _regions: List[int] = None, direct: Optional[bool] = None):
        L = N.lib()
        assert L.he_gemm_fuse_args_size() == C.sizeof(_FuseArgs), "ABI mismatch for FuseArgs"
        assert ctx.world <= _MAX_WORLD and width % 8 == 0
        self.ctx, self.width, self.max_rows, self.wait_limit = ctx, width, max_rows, wait_limit
        self.tile_elems = L.he_gemm_fuse_tile_elems()
        self.max_tiles = L.he_gemm_fuse_tiles(C.c_int(max_rows), C.c_int(width))
        # one-hop ("direct") form up to this world size, owner (reduce-scatter + broadcast) form above it
        if direct is None:
            direct = ctx.world <= int(os.environ.get("HE_FUSED_GEMM_DIRECT_MAX_WORLD", "2"))
        self.direct = bool(direct)
        if self.direct:
            self.owned_cap = self.max_tiles
            self.stage_bytes = 2 * ctx.world * self.max_tiles * self.tile_elems * 2
            self.result_bytes = 0
        else:
            self.owned_cap = (self.max_tiles + ctx.world - 1) // ctx.world
            self.stage_bytes = ctx.world * self.owned_cap * self.tile_elems * 2
            self.result_bytes = self.max_tiles * self.tile_elems * 2
        self.flag_bytes = (self.max_tiles * ctx.world * 4 + self.max_tiles * 4) * 4
        self.total_bytes = self.stage_bytes + self.result_bytes + self.flag_bytes
        self._opened: List[int] = []
        self._local = 0
        if _regions is not None:                      # emulated ranks of one process share plain pointers
            self._peer_ptrs = list(_regions)
        else:
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(self.total_bytes), C.byref(base)), "he_comm_alloc")
            self._local = base.value
            self._peer_ptrs = [self._local] * ctx.world
            if ctx.world > 1:
                hsz = L.he_comm_ipc_handle_size()
                handle = (C.c_char * hsz)()
                N.check(L.he_comm_ipc_get(C.c_void_p(self._local), handle), "he_comm_ipc_get")
                handles: List[bytes] = [b""] * ctx.world
                dist.all_gather_object(handles, bytes(handle.raw), group=ctx.group)
                for r in range(ctx.world):
                    if r == ctx.rank:
                        continue
                    p = C.c_void_p()
                    buf = (C.c_char * hsz).from_buffer_copy(handles[r])
                    N.check(L.he_comm_ipc_open(buf, C.byref(p)), "he_comm_ipc_open")
                    self._peer_ptrs[r] = p.value
                    self._opened.append(p.value)
        self.sync = torch.zeros(2, dtype=torch.int32, device=ctx.device)
        if _regions is None and ctx.world > 1:
            ctx.barrier()       # every region is zeroed and mapped before the first kernel runs
        self.calls = 0

    @classmethod
    def emulated_group(cls, device, width: int, world: int, max_rows: int = 512,
                       direct: Optional[bool] = None) -> List["FusedGemmAllReduce"]:
        """``world`` instances in ONE process on one GPU, wired to each other's regions.  Their kernels must be run
        phase by phase (all ranks' phase 1, then all phase 2, then all phase 3) so that no launch waits for a later
        launch; see ``gemm_add(..., phases=...)``."""
        L = N.lib()
        regions: List[int] = []
        out: List[FusedGemmAllReduce] = []
        for r in range(world):
            ctx = DistContext(r, world, 0, torch.device(device), None, "loopback")
            inst = cls(ctx, width, max_rows, wait_limit=20000, _regions=[0] * world, direct=direct)
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(inst.total_bytes), C.byref(base)), "he_comm_alloc")
            regions.append(base.value)
            out.append(inst)
        for inst in out:
            inst._peer_ptrs = list(regions)
        out[0]._owned_regions = regions
        return out

    def supports(self, rows: int, resid: torch.Tensor) -> bool:
        return (rows <= self.max_rows and resid.dtype == torch.float32 and resid.stride(1) == 1
                and resid.stride(0) % 4 == 0 and resid.data_ptr() % 16 == 0)

    def gemm_add(self, x: torch.Tensor, w, resid: torch.Tensor, phases: int = 7) -> None:
        """resid[M, N] += sum over ranks of (x[M, K] @ w[N, K]^T); x bf16 (this rank's K shard), resid fp32.
        ``w`` is either a bf16 tensor or a quantised ``DeviceWeight`` (Q4_K / Q6_K / Q8_0), which the kernel reads in
        its device layout and expands inside the pipeline."""
        assert x.dtype == torch.bfloat16 and resid.dtype == torch.float32
        K._check_device(x)
        M, Kd = x.shape
        quant = isinstance(w, K.DeviceWeight)
        Nn = w.n_rows if quant else w.shape[0]
        if quant:
            assert w.n_cols == Kd and Kd % 256 == 0 and w.qtype in (8, 12, 14)
        else:
            assert w.dtype == torch.bfloat16 and w.shape[1] == Kd and w.stride(1) == 1
        assert Nn == self.width and x.stride(1) == 1
        assert self.supports(M, resid) and resid.shape[1] >= Nn
        a = _FuseArgs()
        off_res, off_flag = self.stage_bytes, self.stage_bytes + self.result_bytes
        for r, p in enumerate(self._peer_ptrs):
            a.stage[r], a.result[r], a.flags[r] = p, p + off_res, p + off_flag
        a.sync = self.sync.data_ptr()
        a.resid, a.ld_resid = resid.data_ptr(), resid.stride(0)
        a.world, a.rank = self.ctx.world, self.ctx.rank
        a.max_tiles, a.owned_cap, a.phases, a.wait_limit = self.max_tiles, self.owned_cap, phases, self.wait_limit
        a.direct = 1 if self.direct else 0
        st = K.status_tensor(x.device)
        if quant:
            N.check(N.lib().he_gemm_q_allreduce(
                C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.ptr), C.c_int(w.qtype),
                C.c_longlong(w.n_rows), C.c_int(M), C.c_int(Nn), C.c_int(Kd), C.byref(a), C.c_void_p(st.data_ptr()),
                C.c_int(N.num_sms()), K._stream()), "he_gemm_q_allreduce")
        else:
            N.check(N.lib().he_gemm_bf16_allreduce(
                C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.data_ptr()),
                C.c_longlong(w.stride(0)), C.c_int(M), C.c_int(Nn), C.c_int(Kd), C.byref(a),
                C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()), K._stream()), "he_gemm_bf16_allreduce")
        self.calls += 1

    def close(self) -> None:
        L = N.lib()
        torch.cuda.synchronize()
        if self.ctx.backend not in ("loopback", "none") and self.ctx.world > 1:
            self.ctx.barrier()
        for p in self._opened:
            L.he_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self._local:
            L.he_comm_free(C.c_void_p(self._local))
            self._local = 0
        for p in getattr(self, "_owned_regions", []):
            L.he_comm_free(C.c_void_p(p))
        self._owned_regions = []


class PeerResidual:
    """Receive regions and device state for the all-reduce that tensor-parallel decode folds into its GEMVs.

    A row-parallel projection *pushes* (its GEMV epilogue stores the partial rows into every rank's region and the last
    CTA stamps a sequence number), the next reader of the residual *reduces* (a GEMV prologue, or ``reduce_in`` for
    other readers, waits for all stamps and adds the rows in rank order).  Region per rank:
    ``[2 parities][world][max_rows * width]`` 8-byte words ``{fp32 value, sequence tag}`` then ``[2][world]`` u32
    stamps.  A ``width == 1`` region carries one (value, token id) pair per row for the vocab-parallel greedy head
    (``argmax_merge``).  Everything is driven by device-side
    counters, so captured CUDA graphs replay without host patching.  Single node (CUDA IPC)."""

    def __init__(self, ctx: DistContext, width: int, max_rows: int = 8, wait_limit: int = 1 << 22,
                 _regions: Optional[List[int]] = None):
        L = N.lib()
        assert ctx.world <= _MAX_WORLD
        self.ctx, self.width, self.max_rows, self.wait_limit = ctx, width, max_rows, wait_limit
        self.slot_floats = max_rows * width
        self.data_bytes = 2 * ctx.world * self.slot_floats * 8      # one 8-byte {value, tag} word per element
        self.total_bytes = (self.data_bytes + 2 * ctx.world * 4 + 255) // 256 * 256
        self._opened: List[int] = []
        self._local = 0
        if _regions is not None:
            self._peer_ptrs = list(_regions)
        else:
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(self.total_bytes), C.byref(base)), "he_comm_alloc")
            self._local = base.value
            self._peer_ptrs = [self._local] * ctx.world
            if ctx.world > 1:
                hsz = L.he_comm_ipc_handle_size()
                handle = (C.c_char * hsz)()
                N.check(L.he_comm_ipc_get(C.c_void_p(self._local), handle), "he_comm_ipc_get")
                handles: List[bytes] = [b""] * ctx.world
                dist.all_gather_object(handles, bytes(handle.raw), group=ctx.group)
                for r in range(ctx.world):
                    if r == ctx.rank:
                        continue
                    p = C.c_void_p()
                    buf = (C.c_char * hsz).from_buffer_copy(handles[r])
                    N.check(L.he_comm_ipc_open(buf, C.byref(p)), "he_comm_ipc_open")
                    self._peer_ptrs[r] = p.value
                    self._opened.append(p.value)
        self.state = torch.zeros(16, dtype=torch.int32, device=ctx.device)
        if _regions is None and ctx.world > 1:
            ctx.barrier()
        self.pending_rows = 0        # rows pushed and not yet reduced into the residual

    @classmethod
    def emulated_group(cls, device, width: int, world: int, max_rows: int = 8,
                       wait_limit: int = 2000) -> List["PeerResidual"]:
        """``world`` instances in one process on one GPU wired to each other's regions.  All ranks' pushes must be
        launched before any rank's reduce (no launch may wait for a later launch)."""
        L = N.lib()
        regions: List[int] = []
        out: List[PeerResidual] = []
        for r in range(world):
            ctx = DistContext(r, world, 0, torch.device(device), None, "loopback")
            inst = cls(ctx, width, max_rows, wait_limit, _regions=[0] * world)
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(inst.total_bytes), C.byref(base)), "he_comm_alloc")
            regions.append(base.value)
            out.append(inst)
        for inst in out:
            inst._peer_ptrs = list(regions)
        out[0]._owned_regions = regions
        return out

    def comm(self, mode: int = 0) -> K.GemvComm:
        c = K.GemvComm()
        for r, p in enumerate(self._peer_ptrs):
            c.recv[r] = p
            c.flags[r] = p + self.data_bytes
        c.state = self.state.data_ptr()
        c.world, c.rank = self.ctx.world, self.ctx.rank
        c.slot_floats, c.width, c.mode, c.wait_limit = self.slot_floats, self.width, mode, self.wait_limit
        return c

    def reduce_in(self, resid: torch.Tensor, rows: int) -> None:
        """resid[:rows] += sum over ranks of the rows of the last push (stand-alone consumer)."""
        st = K.status_tensor(self.ctx.device)
        c = self.comm()
        N.check(N.lib().he_comm_reduce_in(C.byref(c), C.c_void_p(resid.data_ptr()), C.c_longlong(resid.stride(0)),
                                          C.c_int(rows), C.c_void_p(st.data_ptr()), K._stream()), "he_comm_reduce_in")

    def push_rows(self, partial: torch.Tensor, rows: int) -> None:
        """Push ``rows`` contiguous fp32 rows of this rank to every rank (stand-alone producer)."""
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1] == self.width
        c = self.comm()
        N.check(N.lib().he_comm_push_rows(C.byref(c), C.c_void_p(partial.data_ptr()), C.c_int(rows), K._stream()),
                "he_comm_push_rows")

    def argmax_merge(self, loc_val: torch.Tensor, loc_idx: torch.Tensor, vocab_off: int, rows: int,
                     out_ids: torch.Tensor) -> None:
        """Greedy vocab-parallel head: merge every rank's per-row (max, local id) into global token ids."""
        assert self.width == 1 and loc_val.dtype == torch.float32 and loc_idx.dtype == torch.int64
        st = K.status_tensor(self.ctx.device)
        c = self.comm()
        N.check(N.lib().he_comm_argmax_merge(C.byref(c), C.c_void_p(loc_val.data_ptr()), C.c_void_p(loc_idx.data_ptr()),
                                             C.c_int(vocab_off), C.c_int(rows), C.c_void_p(out_ids.data_ptr()),
                                             C.c_void_p(st.data_ptr()), K._stream()), "he_comm_argmax_merge")

    def close(self) -> None:
        L = N.lib()
        torch.cuda.synchronize()
        if self.ctx.backend not in ("loopback", "none") and self.ctx.world > 1:
            self.ctx.barrier()
        for p in self._opened:
            L.he_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self._local:
            L.he_comm_free(C.c_void_p(self._local))
            self._local = 0
        for p in getattr(self, "_owned_regions", []):
            L.he_comm_free(C.c_void_p(p))
        self._owned_regions = []


class _RawCuda:
    """Zero-copy handle of raw device memory for ``torch.as_tensor`` (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    raw = torch.as_tensor(_RawCuda(ptr, nbytes), device=device)
    return raw.view(dtype).reshape(*shape)


class _WqFuse(C.Structure):
    _fields_ = [("stage", C.c_void_p * _MAX_WORLD), ("flags", C.c_void_p * _MAX_WORLD), ("sync", C.c_void_p),
                ("resid", C.c_void_p), ("ld_resid", C.c_longlong), ("world", C.c_int), ("rank", C.c_int),
                ("slots", C.c_int), ("phases", C.c_int), ("wait_limit", C.c_uint), ("reserved", C.c_int)]


class _SpPushArgs(C.Structure):
    _fields_ = [("dst", C.c_void_p * _MAX_WORLD), ("flags", C.c_void_p * _MAX_WORLD), ("state", C.c_void_p),
                ("h", C.c_void_p), ("norm_w", C.c_void_p), ("ld_h", C.c_longlong), ("ld_dst", C.c_longlong),
                ("eps", C.c_float), ("T", C.c_int), ("H", C.c_int), ("mt", C.c_int), ("world", C.c_int),
                ("rank", C.c_int), ("mode", C.c_int)]


class _SpRowsArgs(C.Structure):
    _fields_ = [("stage", C.c_void_p * _MAX_WORLD), ("flags", C.c_void_p * _MAX_WORLD), ("state", C.c_void_p),
                ("partial", C.c_void_p), ("resid", C.c_void_p), ("ld_p", C.c_longlong), ("ld_h", C.c_longlong),
                ("T", C.c_int), ("H", C.c_int), ("mt", C.c_int), ("world", C.c_int), ("rank", C.c_int),
                ("rows_cap", C.c_int), ("wait_limit", C.c_uint), ("status", C.c_void_p)]


class SeqParallel:
    """Sequence-parallel tensor-parallel prefill over peer memory.

    The fp32 residual is sharded by M-tiles (tile ``tm`` of ``mt`` rows belongs to rank ``tm % world``):

    * ``gemm_rs``   : row-parallel projection, GEMM -> reduce-scatter -> residual add in ONE tcgen05 kernel per rank
      (``csrc/gemm_wq_sm100.cu::gemm_wq_rs_kernel``): partial tiles leave the epilogue as bf16 peer stores into the
      owner's stage, owners sum in fp32 straight into their residual rows;
    * ``norm_push`` : RMSNorm of the owned rows written as bf16 into EVERY rank's activation buffer (the all-gather,
      as peer stores of whole rows) + a stamp;
    * the next column-parallel GEMM reads the gathered rows from local memory and waits, tile by tile inside its TMA
      producer, for the stamp of each tile's owner (``ops/gemm.py::gemm_quant(..., ag=...)``).

    The sharding contract follows the reference's planning notes (``docs/reference/TENSOR_PARALLEL.md:44-52,81-90``);
    the reference itself is single-device.  Region per rank (CUDA IPC, single node): stage, reduce-scatter stamps,
    activation rows, residual rows, all-gather stamps.
    """

    def __init__(self, ctx: DistContext, hidden: int, max_rows: int = 4096, wait_limit: int = 1 << 22,
                 _regions: Optional[List[int]] = None):
        L = N.lib()
        assert L.he_gemm_q_fuse_args_size() == C.sizeof(_WqFuse), "ABI mismatch for WqFuse"
        assert L.he_sp_push_args_size() == C.sizeof(_SpPushArgs), "ABI mismatch for SpPushArgs"
        assert ctx.world <= _MAX_WORLD and hidden % 8 == 0
        self.ctx, self.hidden, self.max_rows, self.wait_limit = ctx, hidden, max_rows, wait_limit
        W = ctx.world
        self.tile_elems = L.he_gemm_q_rs_tile_elems()
        self.tiles_n = (hidden + 127) // 128
        # slots for the finest tiling a call of up to max_rows rows can have (192-row tiles above 192 rows, one tile below)
        mt_big = int(L.he_gemm_q_mt(C.c_int(max(max_rows, 192))))
        self.slots = max(1, ((max_rows + mt_big - 1) // mt_big + W - 1) // W) * self.tiles_n
        al = lambda b: (b + 1023) // 1024 * 1024
        self.off_stage = 0
        self.off_rsflags = al(W * self.slots * self.tile_elems * 2)
        self.off_xn = self.off_rsflags + al(self.slots * W * 4 * 4)
        self.off_h = self.off_xn + al(max_rows * hidden * 2)
        self.off_agflags = self.off_h + al(max_rows * hidden * 4)
        self.off_rowflags = self.off_agflags + 1024
        self.total_bytes = self.off_rowflags + 1024
        assert L.he_sp_rows_args_size() == C.sizeof(_SpRowsArgs), "ABI mismatch for SpRowsArgs"
        self.rows_cap = self.slots * self.tile_elems // hidden       # stage rows available per source rank
        self._opened: List[int] = []
        self._local = 0
        if _regions is not None:
            self._peer_ptrs = list(_regions)
        else:
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(self.total_bytes), C.byref(base)), "he_comm_alloc")
            self._local = base.value
            self._peer_ptrs = [self._local] * W
            if W > 1:
                hsz = L.he_comm_ipc_handle_size()
                handle = (C.c_char * hsz)()
                N.check(L.he_comm_ipc_get(C.c_void_p(self._local), handle), "he_comm_ipc_get")
                handles: List[bytes] = [b""] * W
                dist.all_gather_object(handles, bytes(handle.raw), group=ctx.group)
                for r in range(W):
                    if r == ctx.rank:
                        continue
                    p = C.c_void_p()
                    buf = (C.c_char * hsz).from_buffer_copy(handles[r])
                    N.check(L.he_comm_ipc_open(buf, C.byref(p)), "he_comm_ipc_open")
                    self._peer_ptrs[r] = p.value
                    self._opened.append(p.value)
        self.rs_sync = torch.zeros(2, dtype=torch.int32, device=ctx.device)
        self.sp_state = torch.zeros(2, dtype=torch.int32, device=ctx.device)
        self.rows_state = torch.zeros(2, dtype=torch.int32, device=ctx.device)
        self._views_ready = False
        if _regions is None:
            self._make_views()
            if W > 1:
                ctx.barrier()
        self.rs_calls = 0
        self.ag_pending = False

    def _make_views(self) -> None:
        me = self._peer_ptrs[self.ctx.rank]
        dev = self.ctx.device
        self.xn = tensor_from_ptr(me + self.off_xn, (self.max_rows, self.hidden), torch.bfloat16, dev)
        self.h = tensor_from_ptr(me + self.off_h, (self.max_rows, self.hidden), torch.float32, dev)
        self._views_ready = True

    @classmethod
    def emulated_group(cls, device, hidden: int, world: int, max_rows: int = 512) -> List["SeqParallel"]:
        """``world`` instances in ONE process on one GPU wired to each other's regions; kernels must be run phase by
        phase (all ranks' phase 1, then all phase 2) so that no launch waits for a later one."""
        L = N.lib()
        regions: List[int] = []
        out: List[SeqParallel] = []
        for r in range(world):
            ctx = DistContext(r, world, 0, torch.device(device), None, "loopback")
            inst = cls(ctx, hidden, max_rows, wait_limit=20000, _regions=[0] * world)
            base = C.c_void_p()
            N.check(L.he_comm_alloc(C.c_longlong(inst.total_bytes), C.byref(base)), "he_comm_alloc")
            regions.append(base.value)
            out.append(inst)
        for inst in out:
            inst._peer_ptrs = list(regions)
            inst._make_views()
        out[0]._owned_regions = regions
        return out

    # ------------------------------------------------------------------ tiling
    def mt(self, rows: int) -> int:
        return int(N.lib().he_gemm_q_mt(C.c_int(rows)))

    def owned_rows(self, rows: int) -> List[int]:
        mt, W, r = self.mt(rows), self.ctx.world, self.ctx.rank
        out: List[int] = []
        for tm in range(r, (rows + mt - 1) // mt, W):
            out += list(range(tm * mt, min(rows, (tm + 1) * mt)))
        return out

    # ------------------------------------------------------------------ kernels
    def gemm_rs(self, x: torch.Tensor, w: "K.DeviceWeight", rows: int, phases: int = 3) -> None:
        """self.h[owned rows of the first ``rows``] += sum over ranks of x_rank[rows, K] @ W_rank[hidden, K]^T."""
        assert x.dtype == torch.bfloat16 and x.shape[0] == rows and rows <= self.max_rows and x.stride(1) == 1
        assert w.n_rows == self.hidden and w.n_cols == x.shape[1] and w.qtype in (8, 12, 14)
        K._check_device(x)
        a = _WqFuse()
        for r, p in enumerate(self._peer_ptrs):
            a.stage[r], a.flags[r] = p + self.off_stage, p + self.off_rsflags
        a.sync = self.rs_sync.data_ptr()
        a.resid, a.ld_resid = self.h.data_ptr(), self.h.stride(0)
        a.world, a.rank, a.slots, a.phases, a.wait_limit = (self.ctx.world, self.ctx.rank, self.slots, phases,
                                                            self.wait_limit)
        st = K.status_tensor(x.device)
        N.check(N.lib().he_gemm_q_reduce_scatter(
            C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.ptr), C.c_int(w.qtype),
            C.c_longlong(w.n_rows), C.c_int(rows), C.c_int(self.hidden), C.c_int(w.n_cols), C.byref(a),
            C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()), K._stream()), "he_gemm_q_reduce_scatter")
        self.rs_calls += 1

    def rows_rs(self, partial: torch.Tensor, rows: int, phases: int = 3) -> None:
        """self.h[owned rows] += sum over ranks of partial_rank[rows, hidden] (fp32, token order): the combine of
        expert parallelism over the row-sharded residual (bf16 rows on the wire, fp32 sums on the owner)."""
        assert partial.dtype == torch.float32 and partial.stride(1) == 1 and partial.shape[1] == self.hidden
        a = _SpRowsArgs()
        for r, p in enumerate(self._peer_ptrs):
            a.stage[r], a.flags[r] = p + self.off_stage, p + self.off_rowflags
        a.state = self.rows_state.data_ptr()
        a.partial, a.ld_p = partial.data_ptr(), partial.stride(0)
        a.resid, a.ld_h = self.h.data_ptr(), self.h.stride(0)
        a.T, a.H, a.mt = rows, self.hidden, self.mt(rows)
        a.world, a.rank, a.rows_cap, a.wait_limit = self.ctx.world, self.ctx.rank, self.rows_cap, self.wait_limit
        a.status = K.status_tensor(self.ctx.device).data_ptr()
        N.check(N.lib().he_sp_rows_reduce_scatter(C.byref(a), C.c_int(phases), C.c_int(N.num_sms()), K._stream()),
                "he_sp_rows_reduce_scatter")

    def _push(self, rows: int, norm_w: Optional[torch.Tensor], eps: float, mode: int) -> None:
        a = _SpPushArgs()
        off = self.off_xn if mode == 0 else self.off_h
        for r, p in enumerate(self._peer_ptrs):
            a.dst[r], a.flags[r] = p + off, p + self.off_agflags
        a.state = self.sp_state.data_ptr()
        a.h, a.ld_h = self.h.data_ptr(), self.h.stride(0)
        a.norm_w = norm_w.data_ptr() if norm_w is not None else None
        a.ld_dst = self.hidden
        a.eps, a.T, a.H, a.mt = eps, rows, self.hidden, self.mt(rows)
        a.world, a.rank, a.mode = self.ctx.world, self.ctx.rank, mode
        N.check(N.lib().he_sp_norm_push(C.byref(a), C.c_int(N.num_sms()), K._stream()), "he_sp_norm_push")
        self.ag_pending = True

    def norm_push(self, rows: int, norm_w: torch.Tensor, eps: float) -> torch.Tensor:
        """RMSNorm of this rank's rows of ``self.h`` into every rank's activation buffer; returns the (local) buffer,
        whose rows are complete once the consumers' all-gather wait (``ag_args``) or ``wait`` has passed."""
        self._push(rows, norm_w, eps, 0)
        return self.xn[:rows]

    def gather_residual(self, rows: int) -> torch.Tensor:
        """Copy this rank's residual rows to every rank and wait for the others': ``self.h[:rows]`` complete."""
        self._push(rows, None, 0.0, 1)
        self.wait()
        return self.h[:rows]

    def ag_args(self):
        """(flags pointer, epoch pointer, world, wait limit) for the all-gather wait of a consumer GEMM."""
        me = self._peer_ptrs[self.ctx.rank]
        return (me + self.off_agflags, self.sp_state.data_ptr(), self.ctx.world, self.wait_limit)

    def wait(self) -> None:
        """Stream-ordered wait for every rank's last push (consumers other than the all-gather GEMM)."""
        fl, ep, W, lim = self.ag_args()
        st = K.status_tensor(self.ctx.device)
        N.check(N.lib().he_sp_wait(C.c_void_p(fl), C.c_void_p(ep), C.c_int(W), C.c_uint(lim),
                                   C.c_void_p(st.data_ptr()), K._stream()), "he_sp_wait")
        self.ag_pending = False

    def close(self) -> None:
        L = N.lib()
        torch.cuda.synchronize()
        self.xn = self.h = None
        if self.ctx.backend not in ("loopback", "none") and self.ctx.world > 1:
            self.ctx.barrier()
        for p in self._opened:
            L.he_comm_ipc_close(C.c_void_p(p))
        self._opened = []
        if self._local:
            L.he_comm_free(C.c_void_p(self._local))
            self._local = 0
        for p in getattr(self, "_owned_regions", []):
            L.he_comm_free(C.c_void_p(p))
        self._owned_regions = []
