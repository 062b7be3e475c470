"""tcgen05 / TMEM GEMM launchers (``csrc/gemm_sm100.cu``).

``gemm_bf16`` multiplies bf16 activations by a bf16 weight; ``gemm_quant`` multiplies by a weight kept in
its GGUF-derived device layout (Q4_K / Q6_K / Q8_0 / float).  Kernels report a failed bounded wait through
a device status word; ``check_status`` reads it (a sync) and raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..core import native as N
from .kernels import DeviceWeight, _check_device, _stream, dequant_bf16

from .kernels import check_status, status_tensor as status_word  # noqa: E402,F401


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: Optional[int] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T.  x, w bf16 (row strides allowed); out bf16 or fp32."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    _check_device(x)
    M, K = x.shape
    Nn = w.shape[0]
    assert w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if epi is None:
        epi = 0 if out.dtype == torch.bfloat16 else 1
    st = status_word(x.device)
    N.check(N.lib().he_gemm_bf16(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.data_ptr()),
                                 C.c_longlong(w.stride(0)), C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)),
                                 C.c_int(M), C.c_int(Nn), C.c_int(K), C.c_int(epi), C.c_void_p(st.data_ptr()),
                                 C.c_int(N.num_sms()), _stream()), "he_gemm_bf16")
    return out


QUANT_GEMM_TYPES = (8, 12, 14)     # Q8_0, Q4_K, Q6_K: read in their device layout by the tensor-core pipeline


def quant_gemm_ok(w: DeviceWeight) -> bool:
    return w.qtype in QUANT_GEMM_TYPES and w.n_cols % 256 == 0


def _row_bytes(w: DeviceWeight) -> int:
    return w.data.numel() * w.data.element_size() // w.n_rows


def _float_weight_bf16(w: DeviceWeight, scratch) -> torch.Tensor:
    """bf16 view of a weight that is stored as floats (bf16 as is; f32 / f16 widened once and kept: these are the
    few small unquantised matrices of a checkpoint)."""
    if w.qtype == 30:
        return w.data.view(torch.bfloat16).reshape(w.n_rows, w.n_cols)
    cache = scratch.__dict__.setdefault("_float_bf16", {})
    wb = cache.get(w.ptr)
    if wb is None:
        wb = dequant_bf16(w)
        cache[w.ptr] = wb
    return wb


def gemm_quant(x: torch.Tensor, w: DeviceWeight, out: torch.Tensor, scratch, row0: int = 0,
               rows: Optional[int] = None, epi: Optional[int] = None, ag=None) -> torch.Tensor:
    """out[M, rows] = x[M, K] @ W[row0:row0+rows]^T for a device-layout weight.

    Q4_K / Q6_K / Q8_0 weights are read as stored (raw blocks by TMA, expanded to bf16 operand tiles inside the
    kernel's shared-memory pipeline): the only copy of the weight in HBM is the quantised one.  Counterpart of the
    reference's quantised prefill GEMMs (``hipengine/kernels/hip_gfx1100/quant/gguf_q4_k_prefill.hip:170-296``,
    ``gguf_q8_0_prefill.hip``).
    """
    rows = w.n_rows - row0 if rows is None else rows
    if not quant_gemm_ok(w):
        wb = _float_weight_bf16(w, scratch)
        return gemm_bf16(x, wb[row0:row0 + rows], out, epi)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and out.stride(1) == 1 and x.shape[1] <= w.n_cols
    _check_device(x)
    if epi is None:
        epi = 0 if out.dtype == torch.bfloat16 else 1
    M, a_cols = x.shape        # fewer columns than the weight's (zero-padded) K read as zeros
    st = status_word(x.device)
    if ag is not None:
        # sequence-parallel activations: rows of M-tile tm were written by rank tm % world; the kernel's TMA
        # producer waits for that rank's stamp before the first load of the tile (all-gather -> GEMM)
        fl, ep, world, lim = ag
        N.check(N.lib().he_gemm_q_ag(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_int(a_cols),
                                     C.c_void_p(w.ptr + row0 * _row_bytes(w)), C.c_int(w.qtype), C.c_longlong(rows),
                                     C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)), C.c_int(M),
                                     C.c_int(rows), C.c_int(w.n_cols), C.c_int(epi), C.c_void_p(fl), C.c_void_p(ep),
                                     C.c_int(world), C.c_uint(lim), C.c_void_p(st.data_ptr()),
                                     C.c_int(N.num_sms()), _stream()), "he_gemm_q_ag")
        return out
    N.check(N.lib().he_gemm_q(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_int(a_cols),
                              C.c_void_p(w.ptr + row0 * _row_bytes(w)), C.c_int(w.qtype), C.c_longlong(rows),
                              C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)), C.c_int(M), C.c_int(rows),
                              C.c_int(w.n_cols), C.c_int(epi), C.c_void_p(None), C.c_void_p(st.data_ptr()),
                              C.c_int(N.num_sms()), _stream()), "he_gemm_q")
    return out


def gemm_quant_grouped(a_sorted: torch.Tensor, w: DeviceWeight, out: torch.Tensor, n_groups: int,
                       tile_group: torch.Tensor, epi: Optional[int] = None) -> torch.Tensor:
    """Grouped form of ``gemm_quant`` for MoE experts: ``w`` stacks ``n_groups`` expert matrices of
    ``w.n_rows // n_groups`` rows; 128-row tile ``tm`` of ``a_sorted`` uses expert ``tile_group[tm]`` (-1: skip)."""
    assert quant_gemm_ok(w) and a_sorted.dtype == torch.bfloat16
    M, a_cols = a_sorted.shape
    Nn = w.n_rows // n_groups
    assert tile_group.numel() >= (M + 127) // 128 and a_cols <= w.n_cols
    if epi is None:
        epi = 0 if out.dtype == torch.bfloat16 else 1
    st = status_word(a_sorted.device)
    N.check(N.lib().he_gemm_q(C.c_void_p(a_sorted.data_ptr()), C.c_longlong(a_sorted.stride(0)), C.c_int(a_cols),
                              C.c_void_p(w.ptr), C.c_int(w.qtype), C.c_longlong(w.n_rows), C.c_void_p(out.data_ptr()),
                              C.c_longlong(out.stride(0)), C.c_int(M), C.c_int(Nn), C.c_int(w.n_cols), C.c_int(epi),
                              C.c_void_p(tile_group.data_ptr()), C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()),
                              _stream()), "he_gemm_q(grouped)")
    return out


def gemm_quant_splitk(x: torch.Tensor, w: DeviceWeight, out: torch.Tensor, scratch, add: bool = False
                      ) -> torch.Tensor:
    """out[M, N] (fp32) = (or +=) x @ W^T for few rows (<= 128): the K range is split over the SMs so that all of
    them stream a share of the quantised weight; partial tiles are summed in split order (bit-reproducible)."""
    assert x.dtype == torch.bfloat16 and out.dtype == torch.float32
    if not quant_gemm_ok(w):
        return gemm_bf16_splitk_det(x, _float_weight_bf16(w, scratch), out, scratch, add=add)
    _check_device(x)
    M, K = x.shape
    L = N.lib()
    L.he_gemm_q_splitk_plan.restype = C.c_longlong
    ks = int(L.he_gemm_q_splitk_plan(C.c_int(M), C.c_int(w.n_rows), C.c_int(K), C.c_int(N.num_sms()))) & 0xffffffff
    part = scratch.get("splitk_part", (ks * M * w.n_rows,), torch.float32)
    st = status_word(x.device)
    N.check(L.he_gemm_q_splitk_det(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.ptr),
                                   C.c_int(w.qtype), C.c_longlong(w.n_rows), C.c_void_p(part.data_ptr()),
                                   C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)), C.c_int(M),
                                   C.c_int(w.n_rows), C.c_int(K), C.c_int(1 if add else 0),
                                   C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()), _stream()),
            "he_gemm_q_splitk_det")
    return out


def gemm_bf16_grouped(a_sorted: torch.Tensor, w_stacked: torch.Tensor, out: torch.Tensor, n_groups: int,
                      tile_group: torch.Tensor, epi: Optional[int] = None) -> torch.Tensor:
    """Grouped GEMM for MoE experts: 128-row tile ``tm`` of ``a_sorted`` multiplies expert ``tile_group[tm]``'s
    block of ``w_stacked`` ([n_groups * N, K]); tiles marked -1 are skipped."""
    M, K = a_sorted.shape
    Nn = w_stacked.shape[0] // n_groups
    assert w_stacked.shape[1] == K and tile_group.numel() >= (M + 127) // 128
    if epi is None:
        epi = 0 if out.dtype == torch.bfloat16 else 1
    st = status_word(a_sorted.device)
    N.check(N.lib().he_gemm_bf16_grouped(
        C.c_void_p(a_sorted.data_ptr()), C.c_longlong(a_sorted.stride(0)), C.c_void_p(w_stacked.data_ptr()),
        C.c_longlong(w_stacked.stride(0)), C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)), C.c_int(M),
        C.c_int(Nn), C.c_int(K), C.c_int(n_groups), C.c_void_p(tile_group.data_ptr()), C.c_int(epi),
        C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()), _stream()), "he_gemm_bf16_grouped")
    return out


def gemm_bf16_splitk_add(x: torch.Tensor, w: torch.Tensor, acc: torch.Tensor, k_splits: int = 0) -> torch.Tensor:
    """acc[M, N] (fp32, in place) += x[M, K] @ w[N, K]^T with the K range split over CTAs (atomic accumulation).
    For small M against a narrow output (decode batches on the tensor-core path)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and acc.dtype == torch.float32
    _check_device(x)
    M, K = x.shape
    st = status_word(x.device)
    N.check(N.lib().he_gemm_bf16_splitk(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.data_ptr()),
                                        C.c_longlong(w.stride(0)), C.c_void_p(acc.data_ptr()),
                                        C.c_longlong(acc.stride(0)), C.c_int(M), C.c_int(w.shape[0]), C.c_int(K),
                                        C.c_int(k_splits), C.c_void_p(st.data_ptr()), C.c_int(N.num_sms()), _stream()),
            "he_gemm_bf16_splitk")
    return acc


def gemm_bf16_splitk_det(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch, add: bool = False
                         ) -> torch.Tensor:
    """out[M, N] (fp32) = (or +=) x[M, K] @ w[N, K]^T with K split over CTAs and the partial tiles summed in a
    fixed order: the bit-reproducible form of ``gemm_bf16_splitk_add`` (``out`` may be a strided row view)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.float32
    _check_device(x)
    M, K = x.shape
    Nn = w.shape[0]
    L = N.lib()
    L.he_gemm_splitk_plan.restype = C.c_longlong
    ks = int(L.he_gemm_splitk_plan(C.c_int(M), C.c_int(Nn), C.c_int(K), C.c_int(N.num_sms())))
    part = scratch.get("splitk_part", (ks * M * Nn,), torch.float32)
    st = status_word(x.device)
    N.check(L.he_gemm_bf16_splitk_det(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(w.data_ptr()),
                                      C.c_longlong(w.stride(0)), C.c_void_p(part.data_ptr()),
                                      C.c_void_p(out.data_ptr()), C.c_longlong(out.stride(0)), C.c_int(M), C.c_int(Nn),
                                      C.c_int(K), C.c_int(1 if add else 0), C.c_void_p(st.data_ptr()),
                                      C.c_int(N.num_sms()), _stream()), "he_gemm_bf16_splitk_det")
    return out
