"""Prefill (flash) attention launcher.  The decode/split-K launcher lives in ``ops.kernels``."""
from __future__ import annotations

import ctypes as C

import torch

from ..core import native as N


def flash_prefill_available(head_dim: int) -> bool:
    try:
        return head_dim in (64, 128, 256) and hasattr(N.lib(), "he_flash_prefill")
    except Exception:
        return False


def flash_prefill(q, gate, kv_cache, block_table, slot: int, pos0: int, out, H, Hkv, D, page, scale,
                  window: int = 0) -> None:
    """Causal paged GQA attention over one segment's rows (append-then-attend) with the sigmoid gate fused.

    ``q`` / ``gate`` / ``out`` hold the T rows of the segment, which sit at positions pos0 .. pos0+T-1 of the
    request that owns block-table row ``slot``.
    """
    L = N.lib()
    T = q.shape[0]
    bt_row = block_table[slot]
    N.check(L.he_flash_prefill(C.c_void_p(q.data_ptr()), C.c_void_p(None if gate is None else gate.data_ptr()),
                               C.c_void_p(kv_cache.data_ptr()), C.c_void_p(bt_row.data_ptr()),
                               C.c_void_p(out.data_ptr()), C.c_int(T), C.c_int(H), C.c_int(Hkv), C.c_int(D),
                               C.c_int(page), C.c_int(pos0), C.c_float(scale), C.c_int(window),
                               C.c_void_p(torch.cuda.current_stream().cuda_stream)), "he_flash_prefill")
