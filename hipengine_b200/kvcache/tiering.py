"""Cold tier for evicted prefix-cache content: compressed, checksummed objects in host memory or on a local disk.

When the radix cache has to evict a block whose KV (and, for hybrid models, whose recurrent-state snapshot) took real
prefill work to produce, the owner can hand the bytes to a ``ColdTier`` instead of dropping them, and bring them
back later if restoring is cheaper than recomputing (``restore_is_worthwhile``).  One object = a header (magic,
version, codec, tensor table, CRC-32 of the raw payload, caller metadata) plus the payload, zlib-compressed or raw.
Objects live in a byte-bounded LRU; with ``directory`` set they are files, so they also survive the process.

Reference counterpart: ``hipengine/kvcache/tiering.py`` (host / NVMe tier with a zlib codec, checksummed objects
under a magic tag, restore economics).  The object format here is this project's own.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import zlib
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Dict, Iterable, Optional, Sequence, Tuple

import numpy as np

_COLD_MAGIC = b"HEB2COLD"
_COLD_VERSION = 1
_HEADER = struct.Struct("<8sIIQ")          # magic, version, header-json bytes, payload bytes


class ColdTierCorruption(RuntimeError):
    """The stored object failed its magic, length or checksum test."""


@dataclass(frozen=True)
class ColdObjectInfo:
    key: str
    raw_bytes: int
    stored_bytes: int
    codec: str


def prefix_key(compat: Any, tokens: Sequence[int]) -> str:
    """Content key of a token prefix under a compatibility identity (model / quant / layout / RoPE ...)."""
    h = hashlib.sha256()
    h.update(repr(compat).encode())
    h.update(np.asarray(list(tokens), dtype=np.int64).tobytes())
    return h.hexdigest()


def _to_numpy(t) -> np.ndarray:
    if isinstance(t, np.ndarray):
        return t
    import torch
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:          # numpy has no bf16: carry the bit pattern
            return t.view(torch.int16).numpy()
        return t.numpy()
    raise TypeError(f"unsupported array type {type(t)}")


def encode_object(arrays: Dict[str, Any], meta: Optional[Dict[str, Any]] = None, codec: str = "zlib",
                  level: int = 1) -> Tuple[bytes, int]:
    """Serialise named arrays.  Returns (object bytes, raw payload bytes)."""
    table, chunks, off = [], [], 0
    for name, arr in arrays.items():
        is_bf16 = False
        try:
            import torch
            is_bf16 = isinstance(arr, torch.Tensor) and arr.dtype == torch.bfloat16
        except ImportError:
            pass
        a = np.ascontiguousarray(_to_numpy(arr))
        raw = a.tobytes()
        table.append({"name": name, "dtype": "bfloat16" if is_bf16 else str(a.dtype), "shape": list(a.shape),
                      "offset": off, "bytes": len(raw)})
        chunks.append(raw)
        off += len(raw)
    payload = b"".join(chunks)
    crc = zlib.crc32(payload) & 0xFFFFFFFF
    if codec == "zlib":
        stored = zlib.compress(payload, level)
    elif codec == "raw":
        stored = payload
    else:
        raise ValueError(f"unknown codec {codec!r}")
    header = json.dumps({"codec": codec, "raw_bytes": len(payload), "crc32": crc, "tensors": table,
                         "meta": meta or {}}).encode()
    return _HEADER.pack(_COLD_MAGIC, _COLD_VERSION, len(header), len(stored)) + header + stored, len(payload)


def decode_object(blob: bytes, as_torch: bool = False) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """Inverse of ``encode_object``; raises ``ColdTierCorruption`` on any mismatch."""
    if len(blob) < _HEADER.size:
        raise ColdTierCorruption("object shorter than its fixed header")
    magic, version, hlen, plen = _HEADER.unpack_from(blob, 0)
    if magic != _COLD_MAGIC or version != _COLD_VERSION:
        raise ColdTierCorruption("bad magic or version")
    if len(blob) != _HEADER.size + hlen + plen:
        raise ColdTierCorruption("length does not match the header")
    try:
        header = json.loads(blob[_HEADER.size:_HEADER.size + hlen])
        stored = blob[_HEADER.size + hlen:]
        payload = zlib.decompress(stored) if header["codec"] == "zlib" else stored
    except (ValueError, zlib.error, KeyError) as exc:
        raise ColdTierCorruption(f"undecodable object: {exc}") from exc
    if len(payload) != header["raw_bytes"] or (zlib.crc32(payload) & 0xFFFFFFFF) != header["crc32"]:
        raise ColdTierCorruption("payload checksum mismatch")
    out: Dict[str, Any] = {}
    for t in header["tensors"]:
        is_bf16 = t["dtype"] == "bfloat16"
        a = np.frombuffer(payload, dtype=np.int16 if is_bf16 else np.dtype(t["dtype"]), count=int(np.prod(t["shape"])),
                          offset=t["offset"]).reshape(t["shape"])
        if as_torch or is_bf16:
            import torch
            x = torch.from_numpy(a.copy())
            out[t["name"]] = x.view(torch.bfloat16) if is_bf16 else x
        else:
            out[t["name"]] = a.copy()
    return out, header["meta"]


class ColdTier:
    def __init__(self, capacity_bytes: int, directory: Optional[str] = None, codec: str = "zlib", level: int = 1):
        self.capacity = int(capacity_bytes)
        self.directory = directory
        self.codec, self.level = codec, level
        self.index: "OrderedDict[str, ColdObjectInfo]" = OrderedDict()
        self.mem: Dict[str, bytes] = {}
        self.bytes_stored = 0
        self.stats = {"puts": 0, "hits": 0, "misses": 0, "evicted": 0, "corrupt": 0, "raw_bytes_in": 0,
                      "stored_bytes_in": 0, "raw_bytes_out": 0}
        if directory:
            os.makedirs(directory, exist_ok=True)
            for fn in sorted(os.listdir(directory)):               # adopt objects left by an earlier process
                if fn.endswith(".cold"):
                    sz = os.path.getsize(os.path.join(directory, fn))
                    self.index[fn[:-5]] = ColdObjectInfo(fn[:-5], 0, sz, "?")
                    self.bytes_stored += sz

    def _path(self, key: str) -> str:
        return os.path.join(self.directory, key + ".cold")

    def __contains__(self, key: str) -> bool:
        return key in self.index

    def __len__(self) -> int:
        return len(self.index)

    def put(self, key: str, arrays: Dict[str, Any], meta: Optional[Dict[str, Any]] = None) -> Optional[ColdObjectInfo]:
        """Store (or replace) an object; evicts least-recently-used objects to make room.  Returns None when the
        object alone exceeds the tier's capacity."""
        blob, raw = encode_object(arrays, meta, self.codec, self.level)
        if len(blob) > self.capacity:
            return None
        self.drop(key)
        while self.bytes_stored + len(blob) > self.capacity and self.index:
            old, _ = next(iter(self.index.items()))
            self.drop(old)
            self.stats["evicted"] += 1
        if self.directory:
            tmp = self._path(key) + ".tmp"
            with open(tmp, "wb") as f:
                f.write(blob)
            os.replace(tmp, self._path(key))
        else:
            self.mem[key] = blob
        info = ColdObjectInfo(key, raw, len(blob), self.codec)
        self.index[key] = info
        self.bytes_stored += len(blob)
        self.stats["puts"] += 1
        self.stats["raw_bytes_in"] += raw
        self.stats["stored_bytes_in"] += len(blob)
        return info

    def get(self, key: str, as_torch: bool = True) -> Optional[Tuple[Dict[str, Any], Dict[str, Any]]]:
        """The arrays and metadata stored under ``key``, or None (missing, or corrupt -- a corrupt object is dropped
        and counted, never returned)."""
        if key not in self.index:
            self.stats["misses"] += 1
            return None
        try:
            if self.directory:
                with open(self._path(key), "rb") as f:
                    blob = f.read()
            else:
                blob = self.mem[key]
            arrays, meta = decode_object(blob, as_torch=as_torch)
        except (OSError, KeyError, ColdTierCorruption):
            self.stats["corrupt"] += 1
            self.drop(key)
            return None
        self.index.move_to_end(key)
        self.stats["hits"] += 1
        self.stats["raw_bytes_out"] += sum(int(np.prod(a.shape)) * a.element_size() if hasattr(a, "element_size")
                                          else a.nbytes for a in arrays.values())
        return arrays, meta

    def drop(self, key: str) -> bool:
        info = self.index.pop(key, None)
        if info is None:
            return False
        self.bytes_stored -= info.stored_bytes
        if self.directory:
            try:
                os.remove(self._path(key))
            except OSError:
                pass
        else:
            self.mem.pop(key, None)
        return True

    def keys(self) -> Iterable[str]:
        return list(self.index)

    def compression_ratio(self) -> float:
        return self.stats["raw_bytes_in"] / max(1, self.stats["stored_bytes_in"])


def restore_is_worthwhile(n_tokens: int, stored_bytes: int, raw_bytes: int, prefill_tok_s: float,
                          read_gbs: float = 5.0, inflate_gbs: float = 0.4, h2d_gbs: float = 40.0,
                          margin: float = 1.25) -> bool:
    """Restore economics: bring a cold prefix back only if reading + inflating + uploading it is clearly cheaper than
    recomputing its ``n_tokens`` at the engine's measured prefill rate."""
    if n_tokens <= 0 or prefill_tok_s <= 0:
        return False
    t_restore = stored_bytes / (read_gbs * 1e9) + raw_bytes / (inflate_gbs * 1e9) + raw_bytes / (h2d_gbs * 1e9)
    t_recompute = n_tokens / prefill_tok_s
    return t_restore * margin < t_recompute
