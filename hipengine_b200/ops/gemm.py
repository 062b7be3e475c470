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


def gemm_quant(x: torch.Tensor, w: DeviceWeight, out: torch.Tensor, scratch, row0: int = 0,
               rows: Optional[int] = None, epi: Optional[int] = None, shadow: Optional[dict] = None) -> torch.Tensor:
    """out[M, rows] = x[M, K] @ W[row0:row0+rows]^T for a quantized device-layout weight.

    The weight is expanded to bf16 for the tensor cores.  With ``shadow`` (a dict owned by the executor, holding a
    byte budget under the key ``"_left"``) the expansion is kept resident in HBM after its first use, so later
    prefill chunks read bf16 tiles straight through TMA; without it the expansion goes to scratch every call.
    """
    rows = w.n_rows - row0 if rows is None else rows
    if w.qtype == 30 and row0 == 0 and rows == w.n_rows:   # already bf16
        return gemm_bf16(x, w.data.view(torch.bfloat16).reshape(w.n_rows, w.n_cols), out, epi)
    if shadow is not None:
        key = (w.ptr, row0, rows)
        wb = shadow.get(key)
        if wb is None:
            need = rows * w.n_cols * 2
            if shadow.get("_left", 0) >= need:
                wb = torch.empty(rows, w.n_cols, dtype=torch.bfloat16, device=x.device)
                dequant_bf16(w, wb, row0=row0, rows=rows)
                shadow[key] = wb
                shadow["_left"] -= need
        if wb is not None:
            return gemm_bf16(x, wb, out, epi)
    wb = scratch.get("gemm_deq", (rows, w.n_cols), torch.bfloat16)
    dequant_bf16(w, wb, row0=row0, rows=rows)
    return gemm_bf16(x, wb, out, epi)


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


def bf16_weight(w: DeviceWeight, scratch, shadow: Optional[dict] = None) -> torch.Tensor:
    """The bf16 expansion of a quantised weight: the resident shadow copy when there is one, else scratch."""
    if w.qtype == 30:
        return w.data.view(torch.bfloat16).reshape(w.n_rows, w.n_cols)
    if shadow is not None:
        key = (w.ptr, 0, w.n_rows)
        wb = shadow.get(key)
        if wb is None and shadow.get("_left", 0) >= w.n_rows * w.n_cols * 2:
            wb = torch.empty(w.n_rows, w.n_cols, dtype=torch.bfloat16, device=w.data.device)
            dequant_bf16(w, wb)
            shadow[key] = wb
            shadow["_left"] -= w.n_rows * w.n_cols * 2
        if wb is not None:
            return wb
    wb = scratch.get("gemm_deq", (w.n_rows, w.n_cols), torch.bfloat16)
    dequant_bf16(w, wb)
    return wb
