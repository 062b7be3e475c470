"""ctypes binding of the in-tree sm_100a kernel library.

The library exports plain ``extern "C"`` launchers that take raw device pointers
and a stream (the same call style as the reference's JIT-built ``.so`` files,
``hipengine/core/build.py:353-420`` + per-kernel wrappers), so binding it costs
no compile time and no torch ABI coupling.  ``lib()`` raises if the library is
absent: on a GPU machine a missing extension must be a loud failure, never a
silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import build as _build

_LOCK = threading.Lock()
_LIB: Optional[ctypes.CDLL] = None


class NativeLibraryMissing(RuntimeError):
    pass


def lib_available() -> bool:
    return _build.lib_path().exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            p = _build.lib_path()
            if not p.exists():
                if os.environ.get("HE_BUILD_ON_IMPORT", "0") == "1":
                    _build.build()
                else:
                    raise NativeLibraryMissing(
                        f"{p} not found: run `python -m hipengine_b200.core.build` (or __graft_entry__.build()) first")
            _LIB = ctypes.CDLL(str(p))
    return _LIB


def bounds_status(reset: bool = True):
    """(code, site, index, limit) recorded by the range checks of the ``checked`` library variant, (0, 0, 0, 0) when
    clean, or None when the loaded library is the product build (which has no checks)."""
    out = (ctypes.c_int * 4)()
    rc = lib().he_bounds_status(out, ctypes.c_int(1 if reset else 0))
    if rc == -1:
        return None
    if rc < 0:
        raise RuntimeError("he_bounds_status: reading the device words failed")
    return tuple(int(v) for v in out)


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# kernels launched per successful launcher call (used for launch accounting)
KERNELS_PER_CALL = {"he_attn_decode": 2, "he_gemm_bf16_splitk_det": 2, "he_gdn_decode": 2, "he_argmax_rows": 2, "he_conv1d+state": 2, "he_gemm_quant": 2}
_LAUNCHES = [0]


def launch_count() -> int:
    return _LAUNCHES[0]


def add_launches(n: int) -> None:
    _LAUNCHES[0] += n


def check(code: int, what: str) -> None:
    if code == 0:
        _LAUNCHES[0] += KERNELS_PER_CALL.get(what, 1)
    if code != 0:
        if code < 0:
            raise RuntimeError(f"{what}: bad argument / status {-code}")
        raise RuntimeError(f"{what}: CUDA error {code}")


_NUM_SMS = {}


def num_sms(device: Optional[int] = None) -> int:
    d = torch.cuda.current_device() if device is None else device
    if d not in _NUM_SMS:
        _NUM_SMS[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _NUM_SMS[d]
