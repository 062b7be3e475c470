"""GGUF v2/v3 container: header scan, memory-mapped tensor access, and a writer.

Behavioural parity with the reference scanner (``hipengine/loading/gguf.py:134-267``):
the scan parses header + metadata + tensor table without touching weight
bytes; tensors are exposed as memory-mapped ``uint8 [rows, bytes_per_row]``
views; alignment defaults to 32; ``execution_fingerprint`` hashes the tensor
table plus routing metadata and ignores ``tokenizer.*`` / ``general.*`` keys
(``hipengine/loading/gguf.py:289-321``).

The writer has no counterpart in the reference (it only reads GGUF); it is
needed here because benchmark and test checkpoints are random-init weights
quantized on the fly into real GGUF files.
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, BinaryIO, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from ..quant.ggml import GGMLType, dequantize_np, layout_of, row_bytes

GGUF_MAGIC = 0x46554747
GGUF_DEFAULT_ALIGNMENT = 32

# value type codes
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STR, _ARR, _U64, _I64, _F64 = range(13)
_SCALAR_FMT = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i",
               _F32: "<f", _BOOL: "<?", _U64: "<Q", _I64: "<q", _F64: "<d"}
_NP_FMT = {_U8: np.uint8, _I8: np.int8, _U16: np.uint16, _I16: np.int16, _U32: np.uint32,
           _I32: np.int32, _F32: np.float32, _BOOL: np.bool_, _U64: np.uint64, _I64: np.int64,
           _F64: np.float64}


@dataclass(frozen=True)
class GGUFTensorInfo:
    name: str
    shape: Tuple[int, ...]        # GGUF order: fastest-varying dimension first
    ggml_type: GGMLType
    offset: int                   # relative to the data section
    nbytes: int

    @property
    def n_cols(self) -> int:
        return self.shape[0]

    @property
    def n_rows(self) -> int:
        r = 1
        for s in self.shape[1:]:
            r *= s
        return r

    @property
    def torch_shape(self) -> Tuple[int, ...]:
        """Row-major shape (slowest first), i.e. the shape a framework tensor would have."""
        return tuple(reversed(self.shape))


@dataclass
class GGUFModelInfo:
    path: Path
    version: int
    metadata: Dict[str, Any]
    tensors: Dict[str, GGUFTensorInfo]
    data_offset: int
    alignment: int

    @property
    def architecture(self) -> Optional[str]:
        return self.metadata.get("general.architecture")

    @property
    def tensor_count(self) -> int:
        return len(self.tensors)

    @property
    def total_tensor_nbytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())

    def tensor(self, name: str) -> GGUFTensorInfo:
        try:
            return self.tensors[name]
        except KeyError:
            raise KeyError(f"GGUF tensor {name!r} not found in {self.path}") from None

    def require(self, names: Iterable[str]) -> Tuple[GGUFTensorInfo, ...]:
        missing = [n for n in names if n not in self.tensors]
        if missing:
            raise KeyError(f"GGUF file {self.path} is missing tensors: {missing[:8]}")
        return tuple(self.tensors[n] for n in names)

    def names_with_prefix(self, prefix: str) -> Tuple[str, ...]:
        return tuple(n for n in self.tensors if n.startswith(prefix))

    def get(self, key: str, default: Any = None) -> Any:
        return self.metadata.get(key, default)

    def arch_key(self, suffix: str, default: Any = None) -> Any:
        return self.metadata.get(f"{self.architecture}.{suffix}", default)


def _align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def _read(fh: BinaryIO, n: int) -> bytes:
    b = fh.read(n)
    if len(b) != n:
        raise EOFError("truncated GGUF file")
    return b


def _read_str(fh: BinaryIO) -> str:
    (n,) = struct.unpack("<Q", _read(fh, 8))
    return _read(fh, n).decode("utf-8", errors="replace")


def _read_value(fh: BinaryIO, vt: int) -> Any:
    if vt == _STR:
        return _read_str(fh)
    if vt == _ARR:
        (it,) = struct.unpack("<I", _read(fh, 4))
        (n,) = struct.unpack("<Q", _read(fh, 8))
        if it == _STR:
            return [_read_str(fh) for _ in range(n)]
        if it == _ARR:
            return [_read_value(fh, _ARR) for _ in range(n)]
        dt = np.dtype(_NP_FMT[it])
        return np.frombuffer(_read(fh, dt.itemsize * n), dtype=dt).tolist()
    fmt = _SCALAR_FMT[vt]
    return struct.unpack(fmt, _read(fh, struct.calcsize(fmt)))[0]


def scan_gguf(path: str | os.PathLike) -> GGUFModelInfo:
    """Parse header, metadata and tensor table.  No weight bytes are read."""
    path = Path(path)
    with open(path, "rb") as fh:
        magic, version = struct.unpack("<II", _read(fh, 8))
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file (magic {magic:#x})")
        if version not in (2, 3):
            raise ValueError(f"{path}: unsupported GGUF version {version}")
        n_tensors, n_kv = struct.unpack("<QQ", _read(fh, 16))
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = _read_str(fh)
            (vt,) = struct.unpack("<I", _read(fh, 4))
            meta[key] = _read_value(fh, vt)
        tensors: Dict[str, GGUFTensorInfo] = {}
        for _ in range(n_tensors):
            name = _read_str(fh)
            (nd,) = struct.unpack("<I", _read(fh, 4))
            dims = struct.unpack(f"<{nd}Q", _read(fh, 8 * nd))
            t, off = struct.unpack("<IQ", _read(fh, 12))
            gt = GGMLType(t)
            rows = 1
            for s in dims[1:]:
                rows *= s
            tensors[name] = GGUFTensorInfo(name, tuple(int(x) for x in dims), gt, int(off),
                                           rows * row_bytes(gt, int(dims[0])))
        alignment = int(meta.get("general.alignment", GGUF_DEFAULT_ALIGNMENT))
        data_offset = _align_up(fh.tell(), alignment)
    return GGUFModelInfo(path, version, meta, tensors, data_offset, alignment)


class GGUFReader:
    """Memory-mapped tensor access over a scanned GGUF file."""

    def __init__(self, path: str | os.PathLike):
        self.info = scan_gguf(path)
        self._fh = open(self.info.path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = np.frombuffer(self._mm, dtype=np.uint8)

    @property
    def path(self) -> Path:
        return self.info.path

    @property
    def metadata(self) -> Dict[str, Any]:
        return self.info.metadata

    def tensor_info(self, name: str) -> GGUFTensorInfo:
        return self.info.tensor(name)

    def has(self, name: str) -> bool:
        return name in self.info.tensors

    def tensor_data(self, name: str) -> np.ndarray:
        """Raw bytes as ``uint8 [rows, bytes_per_row]`` (a view on the mapping; read-only)."""
        ti = self.info.tensor(name)
        start = self.info.data_offset + ti.offset
        raw = self._buf[start:start + ti.nbytes]
        return raw.reshape(ti.n_rows, ti.nbytes // max(ti.n_rows, 1))

    def dequantize_tensor(self, name: str) -> np.ndarray:
        ti = self.info.tensor(name)
        arr = dequantize_np(self.tensor_data(name), ti.ggml_type, ti.n_rows, ti.n_cols)
        return arr.reshape(ti.torch_shape)

    def close(self) -> None:
        try:
            self._buf = None  # type: ignore
            self._mm.close()
        except Exception:
            pass
        self._fh.close()

    def __enter__(self) -> "GGUFReader":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def discover_gguf_files(model_path: str | os.PathLike) -> Tuple[Path, ...]:
    """A GGUF path, or a directory holding ``*.gguf`` files (sorted).  Never downloads."""
    p = Path(model_path)
    if p.is_file():
        return (p,)
    if p.is_dir():
        return tuple(sorted(p.glob("*.gguf")))
    return ()


def execution_fingerprint(info: GGUFModelInfo) -> str:
    """sha256 over the tensor table + routing metadata; tokenizer/general keys excluded."""
    meta = {k: v for k, v in sorted(info.metadata.items())
            if not (k.startswith("tokenizer.") or k.startswith("general."))}
    table = [(t.name, list(t.shape), int(t.ggml_type), t.offset, t.nbytes)
             for t in sorted(info.tensors.values(), key=lambda x: x.name)]
    payload = json.dumps({"arch": info.architecture, "meta": meta, "tensors": table},
                         sort_keys=True, default=str).encode()
    return hashlib.sha256(payload).hexdigest()


# --------------------------------------------------------------------------- writer

def _w_str(fh: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    fh.write(struct.pack("<Q", len(b)))
    fh.write(b)


def _vt_of(v: Any) -> int:
    if isinstance(v, bool):
        return _BOOL
    if isinstance(v, int):
        return _U32 if 0 <= v < 2 ** 32 else (_I64 if v < 0 else _U64)
    if isinstance(v, float):
        return _F32
    if isinstance(v, str):
        return _STR
    if isinstance(v, (list, tuple)):
        return _ARR
    raise TypeError(f"unsupported GGUF metadata value {type(v)}")


def _w_value(fh: BinaryIO, v: Any, vt: Optional[int] = None) -> None:
    vt = _vt_of(v) if vt is None else vt
    if vt == _STR:
        _w_str(fh, v)
    elif vt == _ARR:
        items = list(v)
        it = _vt_of(items[0]) if items else _U32
        if it == _U32 and any(isinstance(x, int) and x < 0 for x in items):
            it = _I32
        fh.write(struct.pack("<IQ", it, len(items)))
        if it == _STR:
            for x in items:
                _w_str(fh, x)
        else:
            fh.write(np.asarray(items, dtype=_NP_FMT[it]).tobytes())
    else:
        fh.write(struct.pack(_SCALAR_FMT[vt], v))


@dataclass
class _PendingTensor:
    name: str
    shape: Tuple[int, ...]
    ggml_type: GGMLType
    data: Any  # numpy uint8 array or bytes-like


class GGUFWriter:
    """Minimal GGUF v3 writer (metadata + tensors with aligned data section)."""

    def __init__(self, path: str | os.PathLike, architecture: str, alignment: int = GGUF_DEFAULT_ALIGNMENT):
        self.path = Path(path)
        self.alignment = alignment
        self.meta: Dict[str, Any] = {"general.architecture": architecture, "general.alignment": alignment}
        self._typed: Dict[str, int] = {}
        self._tensors: List[_PendingTensor] = []

    def add_meta(self, key: str, value: Any, vt: Optional[int] = None) -> None:
        self.meta[key] = value
        if vt is not None:
            self._typed[key] = vt

    def add_f32(self, key: str, value: float) -> None:
        self.add_meta(key, float(value), _F32)

    def add_u32(self, key: str, value: int) -> None:
        self.add_meta(key, int(value), _U32)

    def add_tensor_raw(self, name: str, shape_row_major: Sequence[int], ggml_type: int, raw) -> None:
        """``shape_row_major``: framework shape (slowest first); ``raw``: uint8 bytes of the GGML encoding."""
        gt = GGMLType(ggml_type)
        shape = tuple(int(s) for s in reversed(tuple(shape_row_major)))
        arr = np.ascontiguousarray(np.asarray(raw)).view(np.uint8).reshape(-1)
        rows = 1
        for s in shape[1:]:
            rows *= s
        expect = rows * row_bytes(gt, shape[0])
        if arr.size != expect:
            raise ValueError(f"{name}: {arr.size} bytes given, {expect} expected for {gt.name} {shape}")
        self._tensors.append(_PendingTensor(name, shape, gt, arr))

    def add_tensor(self, name: str, tensor, ggml_type: int) -> None:
        """Quantize a torch float tensor (any rank; quantized along the last dim) and add it."""
        import torch
        from ..quant.ggml import quantize
        t2 = tensor.reshape(-1, tensor.shape[-1])
        raw = quantize(t2, ggml_type).cpu().numpy()
        self.add_tensor_raw(name, tuple(tensor.shape), ggml_type, raw)

    def write(self) -> Path:
        with open(self.path, "wb") as fh:
            fh.write(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(self._tensors), len(self.meta)))
            for k, v in self.meta.items():
                _w_str(fh, k)
                vt = self._typed.get(k, _vt_of(v))
                fh.write(struct.pack("<I", vt))
                _w_value(fh, v, vt)
            off = 0
            offsets = []
            for t in self._tensors:
                _w_str(fh, t.name)
                fh.write(struct.pack("<I", len(t.shape)))
                fh.write(struct.pack(f"<{len(t.shape)}Q", *t.shape))
                fh.write(struct.pack("<IQ", int(t.ggml_type), off))
                offsets.append(off)
                off = _align_up(off + t.data.size, self.alignment)
            pos = fh.tell()
            fh.write(b"\x00" * (_align_up(pos, self.alignment) - pos))
            base = fh.tell()
            for t, o in zip(self._tensors, offsets):
                cur = fh.tell() - base
                if cur < o:
                    fh.write(b"\x00" * (o - cur))
                fh.write(t.data.tobytes())
            cur = fh.tell() - base
            fh.write(b"\x00" * (_align_up(cur, self.alignment) - cur))
        return self.path
