"""Python launchers for the sm_100a kernel library (thin ctypes wrappers over ``csrc/*.cu``).

Every function here launches hand-written CUDA on the current torch stream and
raises if the native library is missing -- there is no PyTorch fallback on the
hot path.  Argument structs mirror the C structs field for field.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from ..core import native as N
from ..quant.ggml import GGMLType

c_vp = C.c_void_p
c_ll = C.c_longlong

EPI_F32, EPI_BF16, EPI_ADD_F32, EPI_SILU_MUL, EPI_GELU_MUL = 0, 1, 2, 3, 4


class _GemvSeg(C.Structure):
    _fields_ = [("w", c_vp), ("w2", c_vp), ("out", c_vp), ("out_stride", c_ll), ("n_rows", C.c_int),
                ("qtype", C.c_int), ("qtype2", C.c_int), ("epi", C.c_int)]


class GemvComm(C.Structure):
    """Peer-memory description of a tensor-parallel group for the decode kernels (``csrc/peer_comm.cuh``)."""
    _fields_ = [("recv", c_vp * 8), ("flags", c_vp * 8), ("state", c_vp), ("world", C.c_int), ("rank", C.c_int),
                ("slot_floats", C.c_int), ("width", C.c_int), ("mode", C.c_int), ("wait_limit", C.c_uint)]


COMM_PUSH, COMM_REDUCE = 1, 2


class _GemvArgs(C.Structure):
    _fields_ = [("seg", _GemvSeg * 4), ("n_seg", C.c_int), ("K", C.c_int), ("R", C.c_int), ("x_dtype", C.c_int),
                ("x", c_vp), ("x_stride", c_ll), ("norm_w", c_vp), ("eps", C.c_float), ("n_slots", C.c_int),
                ("rg", C.c_int), ("slot_bytes", C.c_int), ("status", c_vp), ("comm", GemvComm), ("x_image", c_vp)]


class _QkvArgs(C.Structure):
    _fields_ = [("q", c_vp), ("k", c_vp), ("v", c_vp), ("in_dtype", C.c_int),
                ("q_stride", c_ll), ("k_stride", c_ll), ("v_stride", c_ll),
                ("q_norm", c_vp), ("k_norm", c_vp), ("v_norm", C.c_int),
                ("q_out", c_vp), ("gate_out", c_vp), ("kv_cache", c_vp), ("block_table", c_vp),
                ("slot", c_vp), ("pos", c_vp), ("max_pages", C.c_int),
                ("H", C.c_int), ("Hkv", C.c_int), ("D", C.c_int), ("page", C.c_int), ("gated", C.c_int),
                ("rope_dim", C.c_int), ("theta", C.c_float), ("eps", C.c_float), ("q_scale", C.c_float),
                ("rope_denom", C.c_int)]


class _ConvArgs(C.Structure):
    _fields_ = [("x", c_vp), ("in_dtype", C.c_int), ("x_stride", c_ll), ("w", c_vp), ("state", c_vp),
                ("seg_start", c_vp), ("seg_slot", c_vp), ("tok_seg", c_vp), ("out", c_vp), ("journal", c_vp),
                ("C", C.c_int), ("KW", C.c_int), ("T", C.c_int), ("n_seg", C.c_int)]


class _GdnPrepArgs(C.Structure):
    _fields_ = [("qkv", c_vp), ("a", c_vp), ("b", c_vp), ("a_stride", c_ll), ("b_stride", c_ll),
                ("ssm_a", c_vp), ("dt_bias", c_vp), ("decay", c_vp), ("beta", c_vp),
                ("C", C.c_int), ("G", C.c_int), ("Hv", C.c_int), ("S", C.c_int), ("T", C.c_int)]


class _GdnScanArgs(C.Structure):
    _fields_ = [("qkv", c_vp), ("decay", c_vp), ("beta", c_vp), ("state", c_vp), ("seg_start", c_vp),
                ("seg_slot", c_vp), ("out", c_vp), ("journal", c_vp),
                ("C", C.c_int), ("G", C.c_int), ("Hv", C.c_int), ("T", C.c_int), ("n_seg", C.c_int),
                ("write_state", C.c_int)]


class _AttnDecArgs(C.Structure):
    _fields_ = [("q", c_vp), ("gate", c_vp), ("kv_cache", c_vp), ("block_table", c_vp), ("slot", c_vp),
                ("ctx_len", c_vp), ("partial", c_vp), ("out", c_vp),
                ("R", C.c_int), ("H", C.c_int), ("Hkv", C.c_int), ("D", C.c_int), ("page", C.c_int),
                ("max_pages", C.c_int), ("split_len", C.c_int), ("max_splits", C.c_int), ("window", C.c_int),
                ("scale", C.c_float), ("status", c_vp)]


class _GdnDecodeArgs(C.Structure):
    _fields_ = [("x", c_vp), ("x_stride", c_ll), ("conv_w", c_vp), ("conv_state", c_vp), ("a", c_vp), ("b", c_vp),
                ("a_stride", c_ll), ("b_stride", c_ll), ("ssm_a", c_vp), ("dt_bias", c_vp), ("slot", c_vp),
                ("qkv", c_vp), ("decay", c_vp), ("beta", c_vp), ("state", c_vp), ("z", c_vp), ("z_dtype", C.c_int),
                ("z_stride", c_ll), ("norm_w", c_vp), ("out", c_vp), ("out_stride", c_ll), ("eps", C.c_float),
                ("C", C.c_int), ("G", C.c_int), ("Hv", C.c_int), ("R", C.c_int)]


class _GdnChunkArgs(C.Structure):
    _fields_ = [("qkv", c_vp), ("decay", c_vp), ("beta", c_vp), ("state", c_vp), ("seg_start", c_vp),
                ("seg_slot", c_vp), ("out", c_vp), ("C", C.c_int), ("G", C.c_int), ("Hv", C.c_int), ("T", C.c_int),
                ("n_seg", C.c_int), ("write_state", C.c_int)]


class _MoeSelArgs(C.Structure):
    _fields_ = [("x", c_vp), ("ldx", c_ll), ("norm_w", c_vp), ("eps", C.c_float), ("ids", c_vp), ("wts", c_vp),
                ("w1", c_vp), ("w2", c_vp), ("qtype1", C.c_int), ("qtype2", C.c_int),
                ("T", C.c_int), ("k", C.c_int), ("K", C.c_int), ("N", C.c_int), ("act", C.c_int),
                ("out", c_vp), ("ldo", c_ll), ("rows_per_cta", C.c_int), ("expert_rows", C.c_int),
                ("expert_lo", C.c_int), ("expert_n", C.c_int)]


_CHECKED = False


def _check_abi() -> None:
    """Struct sizes must agree with the compiled library (catches drift between Python and C)."""
    global _CHECKED
    if _CHECKED:
        return
    L = N.lib()
    pairs = [("he_gemv_args_size", _GemvArgs), ("he_qkv_args_size", _QkvArgs), ("he_conv_args_size", _ConvArgs),
             ("he_gdn_prep_args_size", _GdnPrepArgs), ("he_gdn_scan_args_size", _GdnScanArgs),
             ("he_attn_dec_args_size", _AttnDecArgs), ("he_moe_sel_args_size", _MoeSelArgs),
             ("he_gdn_decode_args_size", _GdnDecodeArgs), ("he_gdn_chunk_args_size", _GdnChunkArgs),
             ("he_gemv_comm_size", GemvComm)]
    for fn, st in pairs:
        got = getattr(L, fn)()
        if got != C.sizeof(st):
            raise RuntimeError(f"ABI mismatch for {st.__name__}: C={got} Python={C.sizeof(st)}")
    _CHECKED = True


def launch_count() -> int:
    """Number of kernels of this library launched so far in this process (graph replays included)."""
    return N.launch_count()


def add_launches(n: int) -> None:
    N.add_launches(n)


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"unsupported activation dtype {t.dtype}")


def _stream() -> c_vp:
    return c_vp(torch.cuda.current_stream().cuda_stream)


# ----------------------------------------------------------------------------- device weights

@dataclass
class DeviceWeight:
    """A weight matrix in its device layout (Q4_K as stored; Q6_K / Q8_0 planar; float types as stored)."""
    qtype: int
    n_rows: int
    n_cols: int
    data: torch.Tensor  # uint8 / float storage on the device

    @property
    def ptr(self) -> int:
        return self.data.data_ptr()


_KERNEL_QTYPES = (GGMLType.Q4_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.F32, GGMLType.F16, GGMLType.BF16)


def device_row_bytes(qtype: int, n_cols: int) -> int:
    L = N.lib()
    L.he_device_row_bytes.restype = C.c_longlong
    return int(L.he_device_row_bytes(C.c_int(int(qtype)), C.c_int(n_cols)))


def to_device_weight(raw: torch.Tensor, qtype: int, n_rows: int, n_cols: int) -> DeviceWeight:
    """Repack GGUF bytes (uint8 [rows, row_bytes], already on the device) into the kernel layout."""
    qtype = GGMLType(qtype)
    if qtype not in _KERNEL_QTYPES:
        # formats without a native kernel are widened to bf16 once at load time
        from ..quant.ggml import dequantize_torch
        w = dequantize_torch(raw, qtype, n_rows, n_cols).to(torch.bfloat16).contiguous()
        return DeviceWeight(int(GGMLType.BF16), n_rows, n_cols, w)
    raw = raw.contiguous()
    if qtype in (GGMLType.Q6_K, GGMLType.Q8_0):
        _check_abi()
        out = torch.empty(n_rows * device_row_bytes(qtype, n_cols), dtype=torch.uint8, device=raw.device)
        N.check(N.lib().he_repack(c_vp(raw.data_ptr()), c_vp(out.data_ptr()), C.c_int(int(qtype)),
                                  c_ll(n_rows), c_ll(n_cols), C.c_int(0), _stream()), "he_repack")
        return DeviceWeight(int(qtype), n_rows, n_cols, out)
    return DeviceWeight(int(qtype), n_rows, n_cols, raw)


def unpack_device_weight(dw: DeviceWeight) -> torch.Tensor:
    """Inverse of ``to_device_weight``: the exact GGUF bytes (lossless; used by round-trip tests)."""
    t = GGMLType(dw.qtype)
    if t in (GGMLType.Q6_K, GGMLType.Q8_0):
        from ..quant.ggml import row_bytes
        out = torch.empty(dw.n_rows * row_bytes(t, dw.n_cols), dtype=torch.uint8, device=dw.data.device)
        N.check(N.lib().he_repack(c_vp(dw.ptr), c_vp(out.data_ptr()), C.c_int(int(t)), c_ll(dw.n_rows),
                                  c_ll(dw.n_cols), C.c_int(1), _stream()), "he_repack")
        return out.reshape(dw.n_rows, -1)
    return dw.data.reshape(dw.n_rows, -1)


# ----------------------------------------------------------------------------- GEMV

@dataclass
class GemvSegment:
    w: DeviceWeight
    out: torch.Tensor          # [R, >= n_rows] fp32 or bf16 (row stride = out.stride(0))
    epi: int = EPI_F32
    w2: Optional[DeviceWeight] = None


_GEMV_IMAGES: Dict[Tuple[str, int], torch.Tensor] = {}
# rows from which the activation rows are normalised + quantised once per launch by a small kernel instead of by every
# CTA of the GEMV (HE_GEMV_PREQUANT_ROWS; 0 = never): measured on the 27B, the per-CTA prologue is ~2.6 ms per extra
# row of a decode step
PREQUANT_MIN_ROWS = int(os.environ.get("HE_GEMV_PREQUANT_ROWS", "2"))


def _gemv_image(device: torch.device, nbytes: int) -> torch.Tensor:
    """Persistent buffer for the activation image (kept for the life of the process: captured graphs bake it in).
    One buffer per device and size serves every launch because the launches of a device are issued on one stream
    (the engine's driver thread owns it): the pre-pass of the next launch waits for the GEMV before it.  A caller that
    drives one device from several streams at once must not share it (``HE_GEMV_PREQUANT_ROWS=0`` avoids the buffer)."""
    key = (str(device), nbytes)
    t = _GEMV_IMAGES.get(key)
    if t is None:
        t = _GEMV_IMAGES[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return t


def gemv(x: torch.Tensor, segs: Sequence[GemvSegment], norm_w: Optional[torch.Tensor] = None,
         eps: float = 1e-6, comm: Optional[GemvComm] = None) -> None:
    """Fused [RMSNorm] + int8 activation quantize + quantized GEMV + epilogue for 1..8 rows.

    ``comm`` (tensor-parallel decode) with mode ``COMM_PUSH`` makes the epilogue store the outputs of the single
    fp32 segment into every rank's receive region instead of ``out``; with ``COMM_REDUCE`` the prologue first adds
    the partial rows every rank pushed to the fp32 rows ``x`` (and writes the sums back)."""
    _check_abi()
    _check_device(x)
    R, K = x.shape
    a = _GemvArgs()
    for i, s in enumerate(segs):
        sg = a.seg[i]
        sg.w = s.w.ptr
        sg.w2 = s.w2.ptr if s.w2 is not None else None
        sg.out = s.out.data_ptr()
        sg.out_stride = s.out.stride(0) if s.out.dim() > 1 else s.out.numel()
        sg.n_rows = s.w.n_rows
        sg.qtype = s.w.qtype
        sg.qtype2 = s.w2.qtype if s.w2 is not None else 0
        sg.epi = s.epi
        assert s.w.n_cols == K, (s.w.n_cols, K)
    a.n_seg = len(segs)
    a.K = K
    a.R = R
    a.x_dtype = _dt(x)
    a.x = x.data_ptr()
    a.x_stride = x.stride(0)
    a.norm_w = _p(norm_w)
    a.eps = eps
    a.status = _status_ptr(x.device)
    if comm is not None:
        a.comm = comm
    elif PREQUANT_MIN_ROWS and R >= max(2, PREQUANT_MIN_ROWS):
        L = N.lib()
        L.he_gemv_image_bytes.restype = C.c_longlong
        img = _gemv_image(x.device, int(L.he_gemv_image_bytes(C.c_int(R), C.c_int(K))))
        N.check(L.he_gemv_prequant(c_vp(x.data_ptr()), C.c_int(_dt(x)), c_ll(x.stride(0)), c_vp(_p(norm_w)),
                                   C.c_float(eps), C.c_int(K), C.c_int(R), c_vp(img.data_ptr()), _stream()),
                "he_gemv_prequant")
        a.x_image = img.data_ptr()
    rc = N.lib().he_gemv(C.byref(a), C.c_int(N.num_sms()), _stream())
    if rc == -3 and R > 1 and comm is None:
        # activation rows + staging rings do not fit shared memory: run the rows in two halves
        h = R // 2
        gemv(x[:h], [GemvSegment(s.w, s.out[:h], s.epi, s.w2) for s in segs], norm_w, eps)
        gemv(x[h:], [GemvSegment(s.w, s.out[h:], s.epi, s.w2) for s in segs], norm_w, eps)
        return
    N.check(rc, "he_gemv")


_STATUS_WORDS = {}


def status_tensor(device) -> torch.Tensor:
    """Per-device int32[4] status word that kernels with bounded waits write on failure."""
    dev = torch.device(device)
    # "cuda" without an index means this thread's current device (rank r of a multi-GPU job runs on cuda:r)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _STATUS_WORDS:
        _STATUS_WORDS[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS_WORDS[key]


def _status_ptr(device) -> int:
    return status_tensor(device).data_ptr()


class DeviceStatusError(RuntimeError):
    """A kernel's bounded wait gave up (mbarrier, peer flag): what it was computing is incomplete."""


def check_status(device="cuda") -> None:
    """Read the status word (synchronises) and raise if any bounded wait gave up."""
    st = status_tensor(device)
    v = int(st[0].item())
    if v != 0:
        st.zero_()
        raise DeviceStatusError(f"sm_100a kernel reported status {v} (a bounded wait gave up)")


def dequant_bf16(w: DeviceWeight, out: Optional[torch.Tensor] = None, row0: int = 0,
                 rows: Optional[int] = None) -> torch.Tensor:
    rows = w.n_rows - row0 if rows is None else rows
    if out is None:
        out = torch.empty(rows, w.n_cols, dtype=torch.bfloat16, device=w.data.device)
    N.check(N.lib().he_dequant_bf16(c_vp(w.ptr), c_vp(out.data_ptr()), C.c_int(w.qtype), c_ll(row0), c_ll(rows),
                                    c_ll(w.n_rows), C.c_int(w.n_cols), _stream()), "he_dequant_bf16")
    return out


def _check_device(t: torch.Tensor) -> None:
    """Launches go to the calling thread's current device: refuse tensors that live on another GPU."""
    if t.device.index != torch.cuda.current_device():
        raise RuntimeError(f"tensor on cuda:{t.device.index} but this thread's current device is "
                           f"cuda:{torch.cuda.current_device()} (call torch.cuda.set_device in the launching thread)")


def embed(w: DeviceWeight, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    _check_device(out)
    assert ids.dtype == torch.int64 and out.dtype == torch.float32
    N.check(N.lib().he_embed(c_vp(w.ptr), C.c_int(w.qtype), c_ll(w.n_rows), C.c_int(w.n_cols), c_vp(ids.data_ptr()),
                             c_vp(out.data_ptr()), C.c_float(scale), C.c_int(ids.numel()), _stream()), "he_embed")
    return out


# ----------------------------------------------------------------------------- row-wise layers

def rmsnorm_rows(x: torch.Tensor, w: Optional[torch.Tensor], out: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    T, H = x.shape
    assert x.dtype == torch.float32
    N.check(N.lib().he_rmsnorm_rows(c_vp(x.data_ptr()), c_vp(_p(w)), c_vp(out.data_ptr()),
                                    C.c_int(1 if out.dtype == torch.bfloat16 else 0), C.c_int(T), C.c_int(H),
                                    C.c_float(eps), c_ll(x.stride(0)), c_ll(out.stride(0)), _stream()),
            "he_rmsnorm_rows")
    return out


def act_mul(gu: torch.Tensor, out: torch.Tensor, act: str = "silu") -> torch.Tensor:
    T, F2 = gu.shape
    if gu.dtype == torch.float32:
        N.check(N.lib().he_act_mul_f32(c_vp(gu.data_ptr()), c_vp(out.data_ptr()), c_ll(T), C.c_int(F2 // 2),
                                       C.c_int(0 if act == "silu" else 1), _stream()), "he_act_mul")
        return out
    N.check(N.lib().he_act_mul(c_vp(gu.data_ptr()), c_vp(out.data_ptr()), c_ll(T), C.c_int(F2 // 2),
                               C.c_int(0 if act == "silu" else 1), _stream()), "he_act_mul")
    return out


def resid_add_bf16(h: torch.Tensor, y: torch.Tensor) -> None:
    assert h.dtype == torch.float32 and y.dtype == torch.bfloat16 and h.numel() == y.numel()
    N.check(N.lib().he_resid_add_bf16(c_vp(h.data_ptr()), c_vp(y.data_ptr()), c_ll(h.numel()), _stream()),
            "he_resid_add_bf16")


def qkv_post(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_norm, k_norm, q_out: torch.Tensor,
             gate_out: Optional[torch.Tensor], kv_cache: torch.Tensor, block_table: torch.Tensor,
             slot: torch.Tensor, pos: torch.Tensor, H: int, Hkv: int, D: int, page: int, gated: bool,
             rope_dim: int, theta: float, eps: float, q_scale: float = 1.0, v_norm: bool = False,
             rope_denom: int = 0) -> None:
    _check_abi()
    T = q.shape[0]
    a = _QkvArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.in_dtype = _dt(q)
    a.q_stride, a.k_stride, a.v_stride = q.stride(0), k.stride(0), v.stride(0)
    a.q_norm, a.k_norm, a.v_norm = _p(q_norm), _p(k_norm), int(v_norm)
    a.q_out, a.gate_out = q_out.data_ptr(), _p(gate_out)
    a.kv_cache, a.block_table = kv_cache.data_ptr(), block_table.data_ptr()
    a.slot, a.pos = slot.data_ptr(), pos.data_ptr()
    a.max_pages = block_table.shape[1]
    a.H, a.Hkv, a.D, a.page, a.gated = H, Hkv, D, page, int(gated)
    a.rope_dim, a.theta, a.eps, a.q_scale = rope_dim, theta, eps, q_scale
    a.rope_denom = rope_denom
    N.check(N.lib().he_qkv_post(C.byref(a), C.c_int(T), _stream()), "he_qkv_post")


def conv1d(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor,
           tok_seg: torch.Tensor, out: torch.Tensor, channels: int, update_state: bool = True,
           journal: Optional[torch.Tensor] = None) -> None:
    _check_abi()
    a = _ConvArgs()
    a.x, a.in_dtype, a.x_stride = x.data_ptr(), _dt(x), x.stride(0)
    a.w, a.state = w.data_ptr(), state.data_ptr()
    a.seg_start, a.seg_slot, a.tok_seg = seg_start.data_ptr(), seg_slot.data_ptr(), tok_seg.data_ptr()
    a.out, a.journal = out.data_ptr(), _p(journal)
    a.C, a.KW, a.T, a.n_seg = channels, w.shape[1], x.shape[0], seg_slot.numel()
    N.check(N.lib().he_conv1d(C.byref(a), C.c_int(int(update_state)), _stream()),
            "he_conv1d+state" if update_state else "he_conv1d")


def gdn_prepare(qkv: torch.Tensor, a_proj: torch.Tensor, b_proj: torch.Tensor, ssm_a: torch.Tensor,
                dt_bias: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, G: int, Hv: int, S: int) -> None:
    _check_abi()
    p = _GdnPrepArgs()
    p.qkv, p.a, p.b = qkv.data_ptr(), a_proj.data_ptr(), b_proj.data_ptr()
    p.a_stride, p.b_stride = a_proj.stride(0), b_proj.stride(0)
    p.ssm_a, p.dt_bias, p.decay, p.beta = ssm_a.data_ptr(), dt_bias.data_ptr(), decay.data_ptr(), beta.data_ptr()
    p.C, p.G, p.Hv, p.S, p.T = qkv.shape[1], G, Hv, S, qkv.shape[0]
    N.check(N.lib().he_gdn_prepare(C.byref(p), _stream()), "he_gdn_prepare")


def gdn_scan(qkv: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
             seg_start: torch.Tensor, seg_slot: torch.Tensor, out: torch.Tensor, G: int, Hv: int,
             write_state: bool = True, journal: Optional[torch.Tensor] = None) -> None:
    _check_abi()
    p = _GdnScanArgs()
    p.qkv, p.decay, p.beta, p.state = qkv.data_ptr(), decay.data_ptr(), beta.data_ptr(), state.data_ptr()
    p.seg_start, p.seg_slot, p.out, p.journal = seg_start.data_ptr(), seg_slot.data_ptr(), out.data_ptr(), _p(journal)
    p.C, p.G, p.Hv, p.T, p.n_seg, p.write_state = qkv.shape[1], G, Hv, qkv.shape[0], seg_slot.numel(), int(write_state)
    N.check(N.lib().he_gdn_scan(C.byref(p), _stream()), "he_gdn_scan")


def gdn_scan_chunked(qkv: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
                     seg_start: torch.Tensor, seg_slot: torch.Tensor, out: torch.Tensor, G: int, Hv: int,
                     write_state: bool = True) -> None:
    """Chunked (16-token, WY form) tensor-core scan for prefill segments; same contract as ``gdn_scan`` without the
    journal.  Products run in TF32 with fp32 accumulation."""
    _check_abi()
    p = _GdnChunkArgs()
    p.qkv, p.decay, p.beta, p.state = qkv.data_ptr(), decay.data_ptr(), beta.data_ptr(), state.data_ptr()
    p.seg_start, p.seg_slot, p.out = seg_start.data_ptr(), seg_slot.data_ptr(), out.data_ptr()
    p.C, p.G, p.Hv, p.T, p.n_seg, p.write_state = qkv.shape[1], G, Hv, qkv.shape[0], seg_slot.numel(), int(write_state)
    assert qkv.dtype == torch.float32 and qkv.is_contiguous()
    N.check(N.lib().he_gdn_scan_chunked(C.byref(p), _stream()), "he_gdn_scan_chunked")


def gdn_gated_norm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, out: torch.Tensor, Hv: int, Dv: int,
                   eps: float) -> None:
    T = o.shape[0]
    N.check(N.lib().he_gdn_gated_norm(c_vp(o.data_ptr()), c_vp(z.data_ptr()), C.c_int(_dt(z)), c_ll(z.stride(0)),
                                      c_vp(w.data_ptr()), c_vp(out.data_ptr()), c_ll(out.stride(0)), C.c_int(T),
                                      C.c_int(Hv), C.c_int(Dv), C.c_float(eps), _stream()), "he_gdn_gated_norm")


def gdn_decode(x: torch.Tensor, conv_w: torch.Tensor, conv_state: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
               ssm_a: torch.Tensor, dt_bias: torch.Tensor, slot: torch.Tensor, qkv: torch.Tensor,
               decay: torch.Tensor, beta: torch.Tensor, state: torch.Tensor, z: torch.Tensor, norm_w: torch.Tensor,
               out: torch.Tensor, G: int, Hv: int, eps: float) -> None:
    """Decode fast path of a gated delta-net layer (single-token segments): conv + gates, then one recurrent
    step with the gated RMSNorm, in two launches."""
    _check_abi()
    p = _GdnDecodeArgs()
    p.x, p.x_stride, p.conv_w, p.conv_state = x.data_ptr(), x.stride(0), conv_w.data_ptr(), conv_state.data_ptr()
    p.a, p.b, p.a_stride, p.b_stride = a.data_ptr(), b.data_ptr(), a.stride(0), b.stride(0)
    p.ssm_a, p.dt_bias, p.slot = ssm_a.data_ptr(), dt_bias.data_ptr(), slot.data_ptr()
    p.qkv, p.decay, p.beta, p.state = qkv.data_ptr(), decay.data_ptr(), beta.data_ptr(), state.data_ptr()
    p.z, p.z_dtype, p.z_stride, p.norm_w = z.data_ptr(), _dt(z), z.stride(0), norm_w.data_ptr()
    p.out, p.out_stride, p.eps = out.data_ptr(), out.stride(0), eps
    p.C, p.G, p.Hv, p.R = qkv.shape[1], G, Hv, x.shape[0]
    assert x.dtype == torch.float32
    N.check(N.lib().he_gdn_decode(C.byref(p), _stream()), "he_gdn_decode")


def state_commit(state: torch.Tensor, journal: torch.Tensor, seg_slot: torch.Tensor, commit_row: torch.Tensor,
                 per_slot: int) -> None:
    N.check(N.lib().he_state_commit(c_vp(state.data_ptr()), c_vp(journal.data_ptr()), c_vp(seg_slot.data_ptr()),
                                    c_vp(commit_row.data_ptr()), C.c_int(seg_slot.numel()), c_ll(per_slot), _stream()),
            "he_state_commit")


# ----------------------------------------------------------------------------- attention

def attn_decode_split(span: int, rows: int, Hkv: int) -> Tuple[int, int]:
    """(split_len, max_splits) of the split-K decode attention for `rows` rows of up to `span` visible keys: spans
    of whole 64-key tiles sized so that rows * Hkv * splits is about four CTAs per SM (one tile per CTA for a single
    short row, up to 1024 keys per CTA for wide batches, where a CTA then streams its span through a deep ring)."""
    want = 4 * 148
    split_len = -(-(span * max(rows, 1) * Hkv) // want)
    split_len = min(1024, max(64, ((split_len + 63) // 64) * 64))
    return split_len, max(1, -(-span // split_len))


def attn_decode_scratch_floats(R: int, H: int, max_splits: int, D: int) -> int:
    return R * H * max_splits * (D + 2)


def attn_decode(q: torch.Tensor, gate: Optional[torch.Tensor], kv_cache: torch.Tensor, block_table: torch.Tensor,
                slot: torch.Tensor, ctx_len: torch.Tensor, partial: torch.Tensor, out: torch.Tensor, H: int, Hkv: int,
                D: int, page: int, split_len: int, max_splits: int, scale: float, window: int = 0) -> None:
    _check_abi()
    a = _AttnDecArgs()
    a.q, a.gate, a.kv_cache = q.data_ptr(), _p(gate), kv_cache.data_ptr()
    a.block_table, a.slot, a.ctx_len = block_table.data_ptr(), slot.data_ptr(), ctx_len.data_ptr()
    a.partial, a.out = partial.data_ptr(), out.data_ptr()
    a.R, a.H, a.Hkv, a.D, a.page = q.shape[0], H, Hkv, D, page
    a.max_pages = block_table.shape[1]
    a.split_len, a.max_splits, a.window, a.scale = split_len, max_splits, window, scale
    a.status = status_tensor(q.device).data_ptr()
    assert partial.numel() >= attn_decode_scratch_floats(a.R, H, max_splits, D)
    N.check(N.lib().he_attn_decode(C.byref(a), _stream()), "he_attn_decode")


def resid_add_f32(h: torch.Tensor, y: torch.Tensor) -> None:
    assert h.dtype == torch.float32 and y.dtype == torch.float32 and h.numel() == y.numel()
    assert h.is_contiguous() and y.is_contiguous()
    N.check(N.lib().he_resid_add_f32(c_vp(h.data_ptr()), c_vp(y.data_ptr()), c_ll(h.numel()), _stream()),
            "he_resid_add_f32")


def norm_add(h: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float) -> None:
    """h += RMSNorm(y) * w, row-wise (sandwich norm on a branch output)."""
    T, H = h.shape
    N.check(N.lib().he_norm_add(c_vp(h.data_ptr()), c_ll(h.stride(0)), c_vp(y.data_ptr()), C.c_int(_dt(y)),
                                c_ll(y.stride(0)), c_vp(w.data_ptr()), C.c_int(T), C.c_int(H), C.c_float(eps),
                                _stream()), "he_norm_add")


def ffn_combine(h: torch.Tensor, dense: torch.Tensor, expert: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                w3: torch.Tensor, scalar: Optional[torch.Tensor], eps: float) -> None:
    """h = (h + RMSNorm(RMSNorm(dense)*w1 + RMSNorm(expert)*w2) * w3) * scalar."""
    T, H = h.shape
    N.check(N.lib().he_ffn_combine(c_vp(h.data_ptr()), c_ll(h.stride(0)), c_vp(dense.data_ptr()),
                                   C.c_int(_dt(dense)), c_ll(dense.stride(0)), c_vp(expert.data_ptr()),
                                   C.c_int(_dt(expert)), c_ll(expert.stride(0)), c_vp(w1.data_ptr()),
                                   c_vp(w2.data_ptr()), c_vp(w3.data_ptr()), c_vp(_p(scalar)), C.c_int(T),
                                   C.c_int(H), C.c_float(eps), _stream()), "he_ffn_combine")


# ----------------------------------------------------------------------------- mixture of experts

def moe_route(logits: torch.Tensor, k: int, ids: torch.Tensor, wts: torch.Tensor, n_experts: Optional[int] = None,
              mode: int = 0, expert_scale: Optional[torch.Tensor] = None) -> None:
    """logits fp32 [T, >=E] (row stride allowed) -> ids int32 [T, k], wts fp32 [T, k]."""
    T = logits.shape[0]
    E = logits.shape[1] if n_experts is None else n_experts
    N.check(N.lib().he_moe_route(c_vp(logits.data_ptr()), c_ll(logits.stride(0)), C.c_int(T), C.c_int(E), C.c_int(k),
                                 C.c_int(mode), c_vp(_p(expert_scale)), c_vp(ids.data_ptr()), c_vp(wts.data_ptr()),
                                 _stream()), "he_moe_route")


def moe_sorted_rows_bound(P: int, E: int) -> int:
    return ((P + 127) // 128 + E) * 128


def moe_group(ids: torch.Tensor, E: int, pos: torch.Tensor, tile_group: torch.Tensor, meta: torch.Tensor,
              expert_lo: int = 0) -> None:
    """Bucket the (token, expert) pairs by expert.  ``E`` local experts starting at ``expert_lo``; pairs routed to
    other experts get pos = -1."""
    N.check(N.lib().he_moe_group(c_vp(ids.data_ptr()), C.c_int(ids.numel()), C.c_int(E), C.c_int(expert_lo),
                                 c_vp(pos.data_ptr()),
                                 c_vp(tile_group.data_ptr()), C.c_int(tile_group.numel()), c_vp(meta.data_ptr()),
                                 _stream()), "he_moe_group")


def moe_gather(x: torch.Tensor, pos: torch.Tensor, k: int, sorted_rows: torch.Tensor) -> None:
    N.check(N.lib().he_moe_gather(c_vp(x.data_ptr()), c_ll(x.stride(0)), c_vp(pos.data_ptr()), C.c_int(pos.numel()),
                                  C.c_int(k), C.c_int(x.shape[1]), c_vp(sorted_rows.data_ptr()),
                                  c_ll(sorted_rows.stride(0)), _stream()), "he_moe_gather")


def moe_combine(h: torch.Tensor, y: torch.Tensor, pos: torch.Tensor, wts: torch.Tensor, k: int,
                ysh: Optional[torch.Tensor] = None, sg: Optional[torch.Tensor] = None) -> None:
    T, Nn = h.shape
    N.check(N.lib().he_moe_combine(c_vp(h.data_ptr()), c_ll(h.stride(0)), c_vp(y.data_ptr()), c_ll(y.stride(0)),
                                   c_vp(pos.data_ptr()), c_vp(wts.data_ptr()), C.c_int(T), C.c_int(k),
                                   c_vp(_p(ysh)), c_ll(ysh.stride(0) if ysh is not None else 0), c_vp(_p(sg)),
                                   c_ll(sg.stride(0) if sg is not None else 0), C.c_int(Nn), _stream()),
            "he_moe_combine")


def moe_scale_rows(act: torch.Tensor, sg: torch.Tensor) -> None:
    T, Nn = act.shape
    N.check(N.lib().he_moe_scale_rows(c_vp(act.data_ptr()), c_ll(act.stride(0)), C.c_int(T), C.c_int(Nn),
                                      c_vp(sg.data_ptr()), c_ll(sg.stride(0)), _stream()), "he_moe_scale_rows")


def _moe_sel(fn: str, x, norm_w, eps, ids, wts, w1: "DeviceWeight", w2, n_rows: int, out, act: str,
             expert_rows: int = 0, w2_row0: int = 0, expert_range: Tuple[int, int] = (0, 0)) -> None:
    _check_abi()
    a = _MoeSelArgs()
    a.x, a.ldx, a.norm_w, a.eps = x.data_ptr(), x.stride(0), _p(norm_w), eps
    a.ids, a.wts = ids.data_ptr(), wts.data_ptr()
    a.w1, a.qtype1 = w1.ptr, w1.qtype
    a.w2, a.qtype2 = (w2.ptr + w2_row0 * device_row_bytes(w2.qtype, w2.n_cols), w2.qtype) if w2 is not None \
        else (None, w1.qtype)
    a.expert_rows = expert_rows
    a.expert_lo, a.expert_n = expert_range[0], max(0, expert_range[1] - expert_range[0])
    a.T, a.k, a.K, a.N = ids.shape[0], ids.shape[1], w1.n_cols, n_rows
    a.act = 0 if act == "silu" else 1
    a.out, a.ldo = out.data_ptr(), out.stride(0)
    N.check(getattr(N.lib(), fn)(C.byref(a), _stream()), fn)


def moe_gateup_sel(h: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float, ids: torch.Tensor,
                   wts: torch.Tensor, w_gate: "DeviceWeight", w_up: "DeviceWeight", n_ff: int, out: torch.Tensor,
                   act: str = "silu", fused_gate_up: bool = False, expert_range: Tuple[int, int] = (0, 0)) -> None:
    """out[t*k+j, :] = act(Wg[e] xn_t) * (Wu[e] xn_t) (bf16) for the selected experts e = ids[t, j].
    ``fused_gate_up``: ``w_gate`` holds, per expert, n_ff gate rows followed by n_ff up rows (``w_up`` ignored)."""
    if fused_gate_up:
        _moe_sel("he_moe_gateup_sel", h, norm_w, eps, ids, wts, w_gate, w_gate, n_ff, out, act,
                 expert_rows=2 * n_ff, w2_row0=n_ff, expert_range=expert_range)
    else:
        _moe_sel("he_moe_gateup_sel", h, norm_w, eps, ids, wts, w_gate, w_up, n_ff, out, act,
                 expert_range=expert_range)


def moe_down_sel(act_rows: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_down: "DeviceWeight", n_out: int,
                 h: torch.Tensor, expert_range: Tuple[int, int] = (0, 0)) -> None:
    """h[t, :] += sum_j wts[t, j] * Wd[ids[t, j]] act_rows[t*k+j, :]  (fp32 residual, in place).
    ``expert_range`` = (lo, hi) restricts the sum to the local experts of an expert-parallel rank."""
    _moe_sel("he_moe_down_sel", act_rows, None, 0.0, ids, wts, w_down, None, n_out, h, "silu",
             expert_range=expert_range)


# ----------------------------------------------------------------------------- speculative decoding

class _SpecSampledArgs(C.Structure):
    _fields_ = [("p_logits", c_vp), ("q_logits", c_vp), ("draft", c_vp), ("temperature", c_vp), ("seed", c_vp),
                ("counter", c_vp), ("n_accept", c_vp), ("out", c_vp), ("R", C.c_int), ("K", C.c_int), ("V", C.c_int)]


def spec_accept_greedy(draft: torch.Tensor, target: torch.Tensor, n_accept: torch.Tensor, out: torch.Tensor,
                       max_emit: Optional[torch.Tensor] = None) -> None:
    """draft int64 [R, K], target int64 [R, K+1] -> n_accept int32 [R], out int64 [R, K+1] (-1 padded)."""
    R, Kd = draft.shape
    N.check(N.lib().he_spec_accept_greedy(c_vp(draft.data_ptr()), c_vp(target.data_ptr()), C.c_int(R), C.c_int(Kd),
                                          c_vp(n_accept.data_ptr()), c_vp(out.data_ptr()), c_vp(_p(max_emit)),
                                          _stream()), "he_spec_accept_greedy")


def spec_accept_sampled(p_logits: torch.Tensor, q_logits: Optional[torch.Tensor], draft: torch.Tensor,
                        temperature: torch.Tensor, seed: torch.Tensor, counter: torch.Tensor,
                        n_accept: torch.Tensor, out: torch.Tensor) -> None:
    """Exact speculative sampling on the device.  p_logits fp32 [R, K+1, V]; q_logits fp32 [R, K, V] or None when
    the drafts were chosen greedily; seed / counter uint64 (as int64 tensors) per request."""
    L = N.lib()
    assert L.he_spec_sampled_args_size() == C.sizeof(_SpecSampledArgs)
    R, Kd = draft.shape
    a = _SpecSampledArgs()
    a.p_logits, a.q_logits, a.draft = p_logits.data_ptr(), _p(q_logits), draft.data_ptr()
    a.temperature, a.seed, a.counter = temperature.data_ptr(), seed.data_ptr(), counter.data_ptr()
    a.n_accept, a.out = n_accept.data_ptr(), out.data_ptr()
    a.R, a.K, a.V = R, Kd, p_logits.shape[-1]
    assert p_logits.is_contiguous() and (q_logits is None or q_logits.is_contiguous())
    N.check(L.he_spec_accept_sampled(C.byref(a), _stream()), "he_spec_accept_sampled")


def spec_commit(n_accept: torch.Tensor, out: torch.Tensor, tokens: torch.Tensor, pos: torch.Tensor,
                ctx_len: Optional[torch.Tensor], commit_row: Optional[torch.Tensor],
                hidden_row: Optional[torch.Tensor]) -> None:
    R, K1 = out.shape
    N.check(N.lib().he_spec_commit(c_vp(n_accept.data_ptr()), c_vp(out.data_ptr()), C.c_int(R), C.c_int(K1 - 1),
                                   c_vp(tokens.data_ptr()), c_vp(pos.data_ptr()), c_vp(_p(ctx_len)),
                                   c_vp(_p(commit_row)), c_vp(_p(hidden_row)), _stream()), "he_spec_commit")


def gather_rows_f32(src: torch.Tensor, rows: torch.Tensor, dst: torch.Tensor) -> None:
    R, H = dst.shape
    N.check(N.lib().he_gather_rows_f32(c_vp(src.data_ptr()), c_ll(src.stride(0)), c_vp(rows.data_ptr()),
                                       c_vp(dst.data_ptr()), c_ll(dst.stride(0)), C.c_int(R), C.c_int(H), _stream()),
            "he_gather_rows_f32")


# ----------------------------------------------------------------------------- sampling

class SampleParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float),
                ("seed", C.c_ulonglong), ("counter", C.c_ulonglong)]


def argmax_rows(logits: torch.Tensor, scratch_v: torch.Tensor, scratch_i: torch.Tensor, out_ids: torch.Tensor,
                out_val: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    N.check(N.lib().he_argmax_rows(c_vp(logits.data_ptr()), c_ll(logits.stride(0)), C.c_int(R), C.c_int(V),
                                   c_vp(scratch_v.data_ptr()), c_vp(scratch_i.data_ptr()), c_vp(out_ids.data_ptr()),
                                   c_vp(_p(out_val)), _stream()), "he_argmax_rows")
    return out_ids


def sample_rows(logits: torch.Tensor, params_dev: torch.Tensor, out_ids: torch.Tensor,
                out_logprob: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    N.check(N.lib().he_sample_rows(c_vp(logits.data_ptr()), c_ll(logits.stride(0)), C.c_int(R), C.c_int(V),
                                   c_vp(params_dev.data_ptr()), c_vp(out_ids.data_ptr()), c_vp(_p(out_logprob)),
                                   _stream()), "he_sample_rows")
    return out_ids


def pack_sample_params(rows: Sequence[Tuple[float, int, float, float, int, int]], device) -> torch.Tensor:
    arr = (SampleParams * len(rows))()
    for i, (t, k, p, mp, seed, ctr) in enumerate(rows):
        arr[i].temperature, arr[i].top_k, arr[i].top_p, arr[i].min_p = t, k, p, mp
        arr[i].seed, arr[i].counter = seed & (2 ** 64 - 1), ctr & (2 ** 64 - 1)
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    return host.to(device)


def topn_logprobs(logits: torch.Tensor, n: int, temperature: float, chosen: Optional[torch.Tensor]):
    R, V = logits.shape
    ids = torch.empty(R, max(n, 1), dtype=torch.int32, device=logits.device)
    lps = torch.empty(R, max(n, 1), dtype=torch.float32, device=logits.device)
    clp = torch.empty(R, dtype=torch.float32, device=logits.device)
    N.check(N.lib().he_topn_logprobs(c_vp(logits.data_ptr()), c_ll(logits.stride(0)), C.c_int(R), C.c_int(V),
                                     C.c_int(n), C.c_float(temperature), c_vp(_p(chosen)), c_vp(ids.data_ptr()),
                                     c_vp(lps.data_ptr()), c_vp(clp.data_ptr()), _stream()), "he_topn_logprobs")
    return ids[:, :n], lps[:, :n], clp


def softcap_(x: torch.Tensor, cap: float) -> None:
    N.check(N.lib().he_softcap(c_vp(x.data_ptr()), c_ll(x.numel()), C.c_float(cap), _stream()), "he_softcap")


def small_gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] (fp32) = x[T, K] @ w[N, K]^T with fp32 weights (router / ssm_alpha / ssm_beta at prefill)."""
    T, K = x.shape
    Nn = w.shape[0]
    assert w.dtype == torch.float32 and out.dtype == torch.float32
    N.check(N.lib().he_small_gemm_f32(c_vp(x.data_ptr()), C.c_int(_dt(x)), c_ll(x.stride(0)), c_vp(w.data_ptr()),
                                      c_vp(out.data_ptr()), c_ll(out.stride(0)), C.c_int(T), C.c_int(Nn), C.c_int(K),
                                      _stream()), "he_small_gemm_f32")
    return out
