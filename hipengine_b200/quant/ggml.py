"""GGML block-quant formats: layout table, bit-exact dequantizers and quantizers.

The on-disk formats are the public GGML ones (the same the reference records in
``hipengine/quant/gguf.py:23-57`` and dequantizes at ``:604-665``):

* ``Q4_K``: 144 B per 256 weights = fp16 ``d``, fp16 ``dmin``, 12 B of packed
  6-bit (scale, min) pairs for 8 sub-blocks of 32, 128 B of nibbles.
  ``w = (d*sc)*q - (dmin*m)`` evaluated in fp32 in exactly that order.
* ``Q5_K``: 176 B per 256 (Q4_K plus one high bit per weight).
* ``Q6_K``: 210 B per 256 = 128 B low nibbles, 64 B high 2-bit, 16 int8 scales,
  fp16 ``d``.  ``w = (d*sc)*(q-32)``.
* ``Q8_0``: 34 B per 32 = fp16 ``d`` + 32 int8.
* ``Q4_0/Q4_1/Q5_0/Q5_1``: legacy 32-wide blocks.

Two implementations of every dequantizer live here: NumPy (the oracle, used
for "read bit-exact" tests) and torch (runs on CPU or CUDA, used by loaders,
the synthetic-weight builder and GPU test oracles).  They produce identical
fp32 bits; ``tests/test_unit_ggml_quant.py`` checks that.

The quantizers are deliberately simple closed-form ones (min/max affine per
sub-block, then 6-bit re-quantization of scales) rather than llama.cpp's
iterative search: the files they produce are valid GGUF that any reader
decodes, which is all random-init benchmark weights need.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Tuple

import numpy as np

try:  # torch is the framework layer, but keep this module importable without it
    import torch
except Exception:  # pragma: no cover
    torch = None  # type: ignore

QK_K = 256


class GGMLType(IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    BF16 = 30


@dataclass(frozen=True)
class BlockLayout:
    block_elems: int
    block_bytes: int


_LAYOUTS = {
    GGMLType.F32: BlockLayout(1, 4),
    GGMLType.F16: BlockLayout(1, 2),
    GGMLType.BF16: BlockLayout(1, 2),
    GGMLType.F64: BlockLayout(1, 8),
    GGMLType.I8: BlockLayout(1, 1),
    GGMLType.I16: BlockLayout(1, 2),
    GGMLType.I32: BlockLayout(1, 4),
    GGMLType.I64: BlockLayout(1, 8),
    GGMLType.Q4_0: BlockLayout(32, 18),
    GGMLType.Q4_1: BlockLayout(32, 20),
    GGMLType.Q5_0: BlockLayout(32, 22),
    GGMLType.Q5_1: BlockLayout(32, 24),
    GGMLType.Q8_0: BlockLayout(32, 34),
    GGMLType.Q8_1: BlockLayout(32, 36),
    GGMLType.Q2_K: BlockLayout(256, 84),
    GGMLType.Q3_K: BlockLayout(256, 110),
    GGMLType.Q4_K: BlockLayout(256, 144),
    GGMLType.Q5_K: BlockLayout(256, 176),
    GGMLType.Q6_K: BlockLayout(256, 210),
    GGMLType.Q8_K: BlockLayout(256, 292),
}


def layout_of(t: int) -> BlockLayout:
    return _LAYOUTS[GGMLType(t)]


def row_bytes(t: int, n_cols: int) -> int:
    lay = layout_of(t)
    if n_cols % lay.block_elems:
        raise ValueError(f"{GGMLType(t).name}: row length {n_cols} is not a multiple of {lay.block_elems}")
    return n_cols // lay.block_elems * lay.block_bytes


def tensor_nbytes(t: int, shape: Tuple[int, ...]) -> int:
    """Bytes of a GGUF tensor whose *GGUF-order* shape (fastest dim first) is ``shape``."""
    n_cols = shape[0]
    rows = 1
    for s in shape[1:]:
        rows *= s
    return rows * row_bytes(t, n_cols)


# --------------------------------------------------------------------------- numpy oracles

def _f16(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


def _k4_scales_np(sc12: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Unpack 12 bytes -> 8 six-bit scales and 8 six-bit mins (uint8 [..., 8] each)."""
    q = sc12.astype(np.uint8)
    sc = np.empty(q.shape[:-1] + (8,), np.uint8)
    mn = np.empty_like(sc)
    sc[..., 0:4] = q[..., 0:4] & 63
    mn[..., 0:4] = q[..., 4:8] & 63
    sc[..., 4:8] = (q[..., 8:12] & 0x0F) | ((q[..., 0:4] >> 6) << 4)
    mn[..., 4:8] = (q[..., 8:12] >> 4) | ((q[..., 4:8] >> 6) << 4)
    return sc, mn


def dequant_q4_k_np(blocks: np.ndarray) -> np.ndarray:
    """``blocks``: uint8 [..., 144] -> float32 [..., 256]."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    dmin = _f16(b[..., 2:4].copy())[..., 0]
    sc, mn = _k4_scales_np(b[..., 4:16])
    qs = b[..., 16:144].reshape(b.shape[:-1] + (4, 32))
    lo = (qs & 0x0F).astype(np.float32)
    hi = (qs >> 4).astype(np.float32)
    q = np.stack([lo, hi], axis=-2).reshape(b.shape[:-1] + (8, 32))
    d1 = (d[..., None] * sc.astype(np.float32)).astype(np.float32)
    m1 = (dmin[..., None] * mn.astype(np.float32)).astype(np.float32)
    y = (d1[..., None] * q).astype(np.float32) - m1[..., None]
    return y.astype(np.float32).reshape(b.shape[:-1] + (256,))


def dequant_q5_k_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    dmin = _f16(b[..., 2:4].copy())[..., 0]
    sc, mn = _k4_scales_np(b[..., 4:16])
    qh = b[..., 16:48]  # [..., 32]
    qs = b[..., 48:176].reshape(b.shape[:-1] + (4, 32))
    lo = (qs & 0x0F).astype(np.int32)
    hi = (qs >> 4).astype(np.int32)
    q = np.stack([lo, hi], axis=-2).reshape(b.shape[:-1] + (8, 32))
    bits = np.arange(8, dtype=np.uint8)
    hb = ((qh[..., None, :] >> bits[:, None]) & 1).astype(np.int32)  # [..., 8, 32]
    q = (q + 16 * hb).astype(np.float32)
    d1 = (d[..., None] * sc.astype(np.float32)).astype(np.float32)
    m1 = (dmin[..., None] * mn.astype(np.float32)).astype(np.float32)
    y = (d1[..., None] * q).astype(np.float32) - m1[..., None]
    return y.astype(np.float32).reshape(b.shape[:-1] + (256,))


def dequant_q6_k_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    lead = b.shape[:-1]
    ql = b[..., 0:128].reshape(lead + (2, 64))
    qh = b[..., 128:192].reshape(lead + (2, 32))
    sc = b[..., 192:208].view(np.int8).reshape(lead + (2, 8)).astype(np.float32)
    d = _f16(b[..., 208:210].copy())[..., 0]
    l0 = ql[..., 0:32]
    l1 = ql[..., 32:64]
    q1 = ((l0 & 0x0F) | (((qh >> 0) & 3) << 4)).astype(np.int32) - 32
    q2 = ((l1 & 0x0F) | (((qh >> 2) & 3) << 4)).astype(np.int32) - 32
    q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int32) - 32
    q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int32) - 32
    q = np.stack([q1, q2, q3, q4], axis=-2).astype(np.float32)  # [..., 2, 4, 32]
    # scale index for element l of quarter j in half n: n*8 + 2*j + l//16
    scq = sc.reshape(lead + (2, 4, 2))
    scale = np.repeat(scq, 16, axis=-1)  # [..., 2, 4, 32]
    ds = (d[..., None, None, None] * scale).astype(np.float32)
    y = (ds * q).astype(np.float32)
    return y.reshape(lead + (256,))


def dequant_q8_0_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    q = b[..., 2:34].view(np.int8).astype(np.float32)
    return (d[..., None] * q).astype(np.float32)


def dequant_q4_0_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    qs = b[..., 2:18]
    q = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=-1).astype(np.float32) - 8.0
    return (d[..., None] * q).astype(np.float32)


def dequant_q4_1_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    m = _f16(b[..., 2:4].copy())[..., 0]
    qs = b[..., 4:20]
    q = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=-1).astype(np.float32)
    return ((d[..., None] * q).astype(np.float32) + m[..., None]).astype(np.float32)


def _q5_high_bits_np(qh4: np.ndarray) -> np.ndarray:
    qh = qh4.copy().view(np.uint32)[..., 0]
    j = np.arange(32, dtype=np.uint32)
    return ((qh[..., None] >> j) & 1).astype(np.int32)


def dequant_q5_0_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    hb = _q5_high_bits_np(b[..., 2:6])
    qs = b[..., 6:22]
    q = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=-1).astype(np.int32)
    q = (q | (hb << 4)).astype(np.float32) - 16.0
    return (d[..., None] * q).astype(np.float32)


def dequant_q5_1_np(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = _f16(b[..., 0:2].copy())[..., 0]
    m = _f16(b[..., 2:4].copy())[..., 0]
    hb = _q5_high_bits_np(b[..., 4:8])
    qs = b[..., 8:24]
    q = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=-1).astype(np.int32)
    q = (q | (hb << 4)).astype(np.float32)
    return ((d[..., None] * q).astype(np.float32) + m[..., None]).astype(np.float32)


_NP_DEQUANT = {
    GGMLType.Q4_K: dequant_q4_k_np,
    GGMLType.Q5_K: dequant_q5_k_np,
    GGMLType.Q6_K: dequant_q6_k_np,
    GGMLType.Q8_0: dequant_q8_0_np,
    GGMLType.Q4_0: dequant_q4_0_np,
    GGMLType.Q4_1: dequant_q4_1_np,
    GGMLType.Q5_0: dequant_q5_0_np,
    GGMLType.Q5_1: dequant_q5_1_np,
}


def dequantize_np(raw: np.ndarray, t: int, n_rows: int, n_cols: int) -> np.ndarray:
    """Dequantize a row-major GGML tensor (``raw``: uint8 bytes) to float32 [n_rows, n_cols]."""
    t = GGMLType(t)
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    if t == GGMLType.F32:
        return raw.view(np.float32).reshape(n_rows, n_cols).copy()
    if t == GGMLType.F16:
        return raw.view(np.float16).astype(np.float32).reshape(n_rows, n_cols)
    if t == GGMLType.BF16:
        u = raw.view(np.uint16).astype(np.uint32) << 16
        return u.view(np.float32).reshape(n_rows, n_cols)
    lay = layout_of(t)
    nb = n_cols // lay.block_elems
    blocks = raw.reshape(n_rows, nb, lay.block_bytes)
    return _NP_DEQUANT[t](blocks).reshape(n_rows, n_cols)


# --------------------------------------------------------------------------- torch twins

def _tf16(b: "torch.Tensor") -> "torch.Tensor":
    return b.contiguous().view(torch.float16).to(torch.float32)


def _k4_scales_t(sc12: "torch.Tensor"):
    q = sc12.to(torch.int32)
    sc_lo = q[..., 0:4] & 63
    mn_lo = q[..., 4:8] & 63
    sc_hi = (q[..., 8:12] & 0x0F) | ((q[..., 0:4] >> 6) << 4)
    mn_hi = (q[..., 8:12] >> 4) | ((q[..., 4:8] >> 6) << 4)
    return torch.cat([sc_lo, sc_hi], -1), torch.cat([mn_lo, mn_hi], -1)


def dequant_q4_k_t(b: "torch.Tensor") -> "torch.Tensor":
    lead = b.shape[:-1]
    d = _tf16(b[..., 0:2])[..., 0]
    dmin = _tf16(b[..., 2:4])[..., 0]
    sc, mn = _k4_scales_t(b[..., 4:16])
    qs = b[..., 16:144].reshape(lead + (4, 32)).to(torch.int32)
    q = torch.stack([qs & 0x0F, qs >> 4], dim=-2).reshape(lead + (8, 32)).to(torch.float32)
    d1 = d[..., None] * sc.to(torch.float32)
    m1 = dmin[..., None] * mn.to(torch.float32)
    y = d1[..., None] * q - m1[..., None]
    return y.reshape(lead + (256,))


def dequant_q5_k_t(b: "torch.Tensor") -> "torch.Tensor":
    lead = b.shape[:-1]
    d = _tf16(b[..., 0:2])[..., 0]
    dmin = _tf16(b[..., 2:4])[..., 0]
    sc, mn = _k4_scales_t(b[..., 4:16])
    qh = b[..., 16:48].to(torch.int32)
    qs = b[..., 48:176].reshape(lead + (4, 32)).to(torch.int32)
    q = torch.stack([qs & 0x0F, qs >> 4], dim=-2).reshape(lead + (8, 32))
    bits = torch.arange(8, device=b.device, dtype=torch.int32)
    hb = (qh[..., None, :] >> bits[:, None]) & 1
    q = (q + 16 * hb).to(torch.float32)
    d1 = d[..., None] * sc.to(torch.float32)
    m1 = dmin[..., None] * mn.to(torch.float32)
    y = d1[..., None] * q - m1[..., None]
    return y.reshape(lead + (256,))


def dequant_q6_k_t(b: "torch.Tensor") -> "torch.Tensor":
    lead = b.shape[:-1]
    ql = b[..., 0:128].reshape(lead + (2, 64)).to(torch.int32)
    qh = b[..., 128:192].reshape(lead + (2, 32)).to(torch.int32)
    sc = b[..., 192:208].contiguous().view(torch.int8).reshape(lead + (2, 4, 2)).to(torch.float32)
    d = _tf16(b[..., 208:210])[..., 0]
    l0 = ql[..., 0:32]
    l1 = ql[..., 32:64]
    q1 = ((l0 & 0x0F) | (((qh >> 0) & 3) << 4)) - 32
    q2 = ((l1 & 0x0F) | (((qh >> 2) & 3) << 4)) - 32
    q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)) - 32
    q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)) - 32
    q = torch.stack([q1, q2, q3, q4], dim=-2).to(torch.float32)
    scale = sc.repeat_interleave(16, dim=-1)
    ds = d[..., None, None, None] * scale
    return (ds * q).reshape(lead + (256,))


def dequant_q8_0_t(b: "torch.Tensor") -> "torch.Tensor":
    d = _tf16(b[..., 0:2])[..., 0]
    q = b[..., 2:34].contiguous().view(torch.int8).to(torch.float32)
    return d[..., None] * q


_T_DEQUANT = {
    GGMLType.Q4_K: dequant_q4_k_t,
    GGMLType.Q5_K: dequant_q5_k_t,
    GGMLType.Q6_K: dequant_q6_k_t,
    GGMLType.Q8_0: dequant_q8_0_t,
}


def dequantize_torch(raw: "torch.Tensor", t: int, n_rows: int, n_cols: int,
                     row_chunk: int = 8192) -> "torch.Tensor":
    """Torch dequantizer (CPU or CUDA): ``raw`` uint8 -> float32 [n_rows, n_cols]."""
    t = GGMLType(t)
    raw = raw.contiguous().view(torch.uint8).reshape(-1)
    if t == GGMLType.F32:
        return raw.view(torch.float32).reshape(n_rows, n_cols).clone()
    if t == GGMLType.F16:
        return raw.view(torch.float16).to(torch.float32).reshape(n_rows, n_cols)
    if t == GGMLType.BF16:
        return raw.view(torch.bfloat16).to(torch.float32).reshape(n_rows, n_cols)
    if t not in _T_DEQUANT:
        arr = dequantize_np(raw.cpu().numpy(), t, n_rows, n_cols)
        return torch.from_numpy(arr).to(raw.device)
    lay = layout_of(t)
    nb = n_cols // lay.block_elems
    blocks = raw.reshape(n_rows, nb, lay.block_bytes)
    out = torch.empty(n_rows, n_cols, dtype=torch.float32, device=raw.device)
    for r0 in range(0, n_rows, row_chunk):
        r1 = min(n_rows, r0 + row_chunk)
        out[r0:r1] = _T_DEQUANT[t](blocks[r0:r1]).reshape(r1 - r0, n_cols)
    return out


# --------------------------------------------------------------------------- quantizers (torch)

def _to_f16_bytes(x: "torch.Tensor") -> "torch.Tensor":
    return x.to(torch.float16).contiguous().view(torch.uint8)


def _pack_k4_scales(sc: "torch.Tensor", mn: "torch.Tensor") -> "torch.Tensor":
    """sc, mn: int32 [..., 8] in 0..63 -> uint8 [..., 12]."""
    out = torch.empty(sc.shape[:-1] + (12,), dtype=torch.int32, device=sc.device)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    return out.to(torch.uint8)


def quantize_q4_k(w: "torch.Tensor") -> "torch.Tensor":
    """float [rows, cols] -> uint8 [rows, cols/256*144] of Q4_K blocks."""
    rows, cols = w.shape
    assert cols % 256 == 0, "Q4_K needs a multiple of 256 columns"
    x = w.to(torch.float32).reshape(rows, cols // 256, 8, 32)
    mx = x.amax(-1)
    mnv = x.amin(-1).clamp(max=0.0)
    scale = ((mx - mnv) / 15.0).clamp(min=0.0)
    minv = -mnv
    d = (scale.amax(-1) / 63.0).to(torch.float16).to(torch.float32)
    dmin = (minv.amax(-1) / 63.0).to(torch.float16).to(torch.float32)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    inv_dm = torch.where(dmin > 0, 1.0 / dmin, torch.zeros_like(dmin))
    sc = torch.round(scale * inv_d[..., None]).clamp(0, 63).to(torch.int32)
    mn = torch.round(minv * inv_dm[..., None]).clamp(0, 63).to(torch.int32)
    d1 = d[..., None] * sc.to(torch.float32)
    m1 = dmin[..., None] * mn.to(torch.float32)
    inv_d1 = torch.where(d1 > 0, 1.0 / d1, torch.zeros_like(d1))
    q = torch.round((x + m1[..., None]) * inv_d1[..., None]).clamp(0, 15).to(torch.int32)
    q = q.reshape(rows, cols // 256, 4, 2, 32)
    qs = (q[..., 0, :] | (q[..., 1, :] << 4)).to(torch.uint8).reshape(rows, cols // 256, 128)
    out = torch.empty(rows, cols // 256, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _to_f16_bytes(d).reshape(rows, cols // 256, 2)
    out[..., 2:4] = _to_f16_bytes(dmin).reshape(rows, cols // 256, 2)
    out[..., 4:16] = _pack_k4_scales(sc, mn)
    out[..., 16:144] = qs
    return out.reshape(rows, cols // 256 * 144)


def quantize_q6_k(w: "torch.Tensor") -> "torch.Tensor":
    rows, cols = w.shape
    assert cols % 256 == 0, "Q6_K needs a multiple of 256 columns"
    nb = cols // 256
    x = w.to(torch.float32).reshape(rows, nb, 16, 16)
    amax = x.abs().amax(-1)
    s = amax / 31.0
    d = (s.amax(-1) / 127.0).to(torch.float16).to(torch.float32)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    sc = torch.round(s * inv_d[..., None]).clamp(0, 127).to(torch.int32)
    ds = d[..., None] * sc.to(torch.float32)
    inv_ds = torch.where(ds > 0, 1.0 / ds, torch.zeros_like(ds))
    q = (torch.round(x * inv_ds[..., None]).clamp(-32, 31) + 32).to(torch.int32)
    # element e of the block lives in half n=e//128, quarter j=(e%128)//32, lane l=e%32
    q = q.reshape(rows, nb, 2, 4, 32)
    q1, q2, q3, q4 = q[..., 0, :], q[..., 1, :], q[..., 2, :], q[..., 3, :]
    ql0 = (q1 & 0x0F) | ((q3 & 0x0F) << 4)
    ql1 = (q2 & 0x0F) | ((q4 & 0x0F) << 4)
    ql = torch.cat([ql0, ql1], dim=-1).reshape(rows, nb, 128)
    qh = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).reshape(rows, nb, 64)
    out = torch.empty(rows, nb, 210, dtype=torch.uint8, device=w.device)
    out[..., 0:128] = ql.to(torch.uint8)
    out[..., 128:192] = qh.to(torch.uint8)
    out[..., 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = _to_f16_bytes(d).reshape(rows, nb, 2)
    return out.reshape(rows, nb * 210)


def quantize_q8_0(w: "torch.Tensor") -> "torch.Tensor":
    rows, cols = w.shape
    assert cols % 32 == 0, "Q8_0 needs a multiple of 32 columns"
    nb = cols // 32
    x = w.to(torch.float32).reshape(rows, nb, 32)
    d = (x.abs().amax(-1) / 127.0).to(torch.float16).to(torch.float32)
    inv_d = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(x * inv_d[..., None]).clamp(-127, 127).to(torch.int8)
    out = torch.empty(rows, nb, 34, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _to_f16_bytes(d).reshape(rows, nb, 2)
    out[..., 2:34] = q.view(torch.uint8)
    return out.reshape(rows, nb * 34)


def quantize(w: "torch.Tensor", t: int) -> "torch.Tensor":
    """Quantize float [rows, cols] to a uint8 byte tensor [rows, row_bytes] of GGML type ``t``."""
    t = GGMLType(t)
    if t == GGMLType.Q4_K:
        return quantize_q4_k(w)
    if t == GGMLType.Q6_K:
        return quantize_q6_k(w)
    if t == GGMLType.Q8_0:
        return quantize_q8_0(w)
    if t == GGMLType.F32:
        return w.to(torch.float32).contiguous().view(torch.uint8).reshape(w.shape[0], -1)
    if t == GGMLType.F16:
        return w.to(torch.float16).contiguous().view(torch.uint8).reshape(w.shape[0], -1)
    if t == GGMLType.BF16:
        return w.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(w.shape[0], -1)
    raise ValueError(f"no quantizer for {t.name}")
