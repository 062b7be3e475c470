"""ctypes face of the native host runtime (``csrc/runtime.cpp``): validated cycle launches, graph-exec cache,
launch sequences.  The Python structs mirror ``csrc/he_cycle_abi.h`` and are size-checked against the library."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

from . import native as N

HE_CYCLE_MAGIC = 0x48454359
HE_CYCLE_VERSION = 1
MAX_REQUESTS = 64
STAGE_PROPOSE, STAGE_VERIFY, STAGE_ACCEPT, STAGE_COMMIT, STAGE_UPDATE_CURSORS, STAGE_DECODE_STEP = (1, 2, 4, 8, 16, 32)
STAGES_FULL_CYCLE = STAGE_PROPOSE | STAGE_VERIFY | STAGE_ACCEPT | STAGE_COMMIT | STAGE_UPDATE_CURSORS


class CycleControl(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("version", C.c_uint32), ("struct_bytes", C.c_uint32),
                ("stage_mask", C.c_uint32), ("mode", C.c_uint32), ("n_requests", C.c_uint32), ("depth", C.c_uint32),
                ("wait", C.c_uint32), ("status_word", C.c_uint64), ("n_accept", C.c_uint64),
                ("reserved", C.c_uint64 * 4)]


class CycleResult(C.Structure):
    _fields_ = [("rc", C.c_int32), ("device_status", C.c_int32), ("n_accept", C.c_int32 * MAX_REQUESTS),
                ("launches", C.c_uint64)]


def _lib():
    L = N.lib()
    if not getattr(L, "_he_runtime_ready", False):
        assert L.he_cycle_control_size() == C.sizeof(CycleControl), "ABI mismatch: HeCycleControlV1"
        assert L.he_cycle_result_size() == C.sizeof(CycleResult), "ABI mismatch: HeCycleResultV1"
        L.he_graph_cache_get.restype = C.c_void_p
        L.he_native_graph_launches.restype = C.c_uint64
        L._he_runtime_ready = True
    return L


def make_control(stage_mask: int, n_requests: int, depth: int, wait: bool = False, status_word: int = 0,
                 n_accept: int = 0) -> CycleControl:
    c = CycleControl()
    c.magic, c.version, c.struct_bytes = HE_CYCLE_MAGIC, HE_CYCLE_VERSION, C.sizeof(CycleControl)
    c.stage_mask, c.mode, c.n_requests, c.depth, c.wait = stage_mask, 0, n_requests, depth, int(wait)
    c.status_word, c.n_accept = status_word, n_accept
    return c


def validate(c: CycleControl) -> int:
    return int(_lib().he_cycle_validate(C.byref(c)))


def cycle_launch(c: CycleControl, graph_exec: int, stream: int) -> CycleResult:
    out = CycleResult()
    _lib().he_cycle_launch(C.byref(c), C.c_void_p(graph_exec), C.c_void_p(stream), C.byref(out))
    return out


def graph_exec_handle(graph) -> Optional[int]:
    """Raw ``cudaGraphExec_t`` of a captured ``torch.cuda.CUDAGraph`` (None when torch does not expose it)."""
    fn = getattr(graph, "raw_cuda_graph_exec", None)
    if fn is None:
        return None
    try:
        return int(fn())
    except Exception:
        return None


class GraphExecCache:
    """Key -> graph exec map living in the native library."""

    def put(self, key: int, graph_exec: int) -> None:
        N.check(_lib().he_graph_cache_put(C.c_uint64(key), C.c_void_p(graph_exec)), "he_graph_cache_put")

    def get(self, key: int) -> Optional[int]:
        return _lib().he_graph_cache_get(C.c_uint64(key))

    def launch(self, key: int, stream: int) -> int:
        return int(_lib().he_graph_cache_launch(C.c_uint64(key), C.c_void_p(stream)))

    def erase(self, key: int) -> bool:
        return _lib().he_graph_cache_erase(C.c_uint64(key)) == 0

    def clear(self) -> None:
        _lib().he_graph_cache_clear()

    def stats(self) -> Tuple[int, int, int]:
        e, h, m = C.c_uint64(), C.c_uint64(), C.c_uint64()
        _lib().he_graph_cache_stats(C.byref(e), C.byref(h), C.byref(m))
        return e.value, h.value, m.value


def launch_sequence(graph_execs: Sequence[int], stream: int) -> Tuple[int, int]:
    arr = (C.c_void_p * len(graph_execs))(*graph_execs)
    failed = C.c_int(-1)
    rc = _lib().he_launch_sequence(arr, C.c_int(len(graph_execs)), C.c_void_p(stream), C.byref(failed))
    return int(rc), failed.value
