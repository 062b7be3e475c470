"""Bounded extraction of image / video parts from chat messages.

OpenAI-style content parts (``{"type": "image_url", "image_url": {"url": "data:image/png;base64,..."}}``, also
``input_image`` / ``image`` / ``video_url``) are parsed with hard limits before anything else looks at them: part
count, encoded and decoded bytes, media type, and pixel count read from the container header without decoding the
picture.  Remote URLs are refused -- this server never downloads anything (the same rule as for model files).
The text-only models this build serves cannot use the media, so ``request_build.build_chat`` answers a request that
carries valid media with ``unsupported_feature`` (501) and one that carries malformed or oversized media with
``invalid_request`` (400); silently dropping the parts would answer a different question than the one asked.

Counterpart of the reference's ``hipengine/server/multimodal.py`` (bounded image / video data-URL extraction with
pixel and byte limits).
"""
from __future__ import annotations

import base64
import binascii
import struct
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

IMAGE_TYPES = ("image_url", "input_image", "image")
VIDEO_TYPES = ("video_url", "input_video", "video")
IMAGE_MIMES = ("image/png", "image/jpeg", "image/gif", "image/webp")
VIDEO_MIMES = ("video/mp4", "video/webm")


@dataclass(frozen=True)
class MediaLimits:
    max_parts: int = 16
    max_image_bytes: int = 20 << 20
    max_video_bytes: int = 64 << 20
    max_total_bytes: int = 96 << 20
    max_pixels: int = 4096 * 4096
    max_side: int = 16384


@dataclass(frozen=True)
class MediaPart:
    kind: str                 # "image" | "video"
    mime: str
    n_bytes: int
    width: Optional[int]
    height: Optional[int]
    message_index: int
    part_index: int

    def as_dict(self) -> Dict[str, Any]:
        return {"kind": self.kind, "mime": self.mime, "bytes": self.n_bytes, "width": self.width,
                "height": self.height, "message": self.message_index, "part": self.part_index}


class MediaError(ValueError):
    def __init__(self, message: str, param: str):
        super().__init__(message)
        self.param = param


def _url_of(part: Mapping[str, Any], key: str) -> Optional[str]:
    v = part.get(key)
    if isinstance(v, Mapping):
        v = v.get("url")
    return v if isinstance(v, str) else None


def split_data_url(url: str, param: str, max_bytes: int) -> Tuple[str, bytes]:
    """``data:<mime>;base64,<payload>`` -> (mime, decoded bytes).  The encoded length is checked before decoding, so
    an oversized payload is never materialised."""
    if not url.startswith("data:"):
        scheme = url.split(":", 1)[0].lower() if ":" in url[:16] else "relative"
        raise MediaError(f"media must be inline data URLs; {scheme} URLs are not fetched", param)
    head, sep, payload = url[5:].partition(",")
    if not sep:
        raise MediaError("malformed data URL (no comma)", param)
    fields = head.split(";")
    mime = fields[0].strip().lower()
    if "base64" not in [f.strip().lower() for f in fields[1:]]:
        raise MediaError("data URL payload must be base64", param)
    if (len(payload) // 4) * 3 > max_bytes + 3:
        raise MediaError(f"media part exceeds {max_bytes} bytes", param)
    try:
        raw = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError):
        raise MediaError("data URL payload is not valid base64", param) from None
    if len(raw) > max_bytes:
        raise MediaError(f"media part exceeds {max_bytes} bytes", param)
    if not raw:
        raise MediaError("empty media part", param)
    return mime, raw


def sniff_image(raw: bytes) -> Tuple[Optional[str], Optional[int], Optional[int]]:
    """(mime, width, height) from the container header; (None, None, None) for an unknown container.  Nothing is
    decoded: PNG IHDR, GIF logical screen, JPEG start-of-frame marker, WebP VP8 / VP8L / VP8X chunk."""
    if raw[:8] == b"\x89PNG\r\n\x1a\n" and raw[12:16] == b"IHDR" and len(raw) >= 24:
        w, h = struct.unpack(">II", raw[16:24])
        return "image/png", w, h
    if raw[:6] in (b"GIF87a", b"GIF89a") and len(raw) >= 10:
        w, h = struct.unpack("<HH", raw[6:10])
        return "image/gif", w, h
    if raw[:2] == b"\xff\xd8":
        i, n = 2, len(raw)
        while i + 9 < n:
            if raw[i] != 0xFF:
                i += 1
                continue
            marker = raw[i + 1]
            if marker in (0xD8, 0x01) or 0xD0 <= marker <= 0xD7 or marker == 0xFF:
                i += 2 if marker != 0xFF else 1
                continue
            seg = struct.unpack(">H", raw[i + 2:i + 4])[0]
            if 0xC0 <= marker <= 0xCF and marker not in (0xC4, 0xC8, 0xCC):
                h, w = struct.unpack(">HH", raw[i + 5:i + 9])
                return "image/jpeg", w, h
            i += 2 + seg
        return "image/jpeg", None, None
    if raw[:4] == b"RIFF" and raw[8:12] == b"WEBP" and len(raw) >= 30:
        tag = raw[12:16]
        if tag == b"VP8X":
            w = 1 + int.from_bytes(raw[24:27], "little")
            h = 1 + int.from_bytes(raw[27:30], "little")
            return "image/webp", w, h
        if tag == b"VP8L" and raw[20] == 0x2F:
            bits = int.from_bytes(raw[21:25], "little")
            return "image/webp", 1 + (bits & 0x3FFF), 1 + ((bits >> 14) & 0x3FFF)
        if tag == b"VP8 " and raw[23:26] == b"\x9d\x01\x2a":
            w, h = struct.unpack("<HH", raw[26:30])
            return "image/webp", w & 0x3FFF, h & 0x3FFF
        return "image/webp", None, None
    return None, None, None


def sniff_video(raw: bytes) -> Optional[str]:
    if raw[4:8] == b"ftyp":
        return "video/mp4"
    if raw[:4] == b"\x1a\x45\xdf\xa3":
        return "video/webm"
    return None


def extract_media(messages: Sequence[Any], limits: MediaLimits = MediaLimits()) -> List[MediaPart]:
    """Every image / video part of ``messages`` (objects with ``.content`` or mappings), validated against
    ``limits``.  Raises ``MediaError`` naming the offending part."""
    out: List[MediaPart] = []
    total = 0
    for mi, m in enumerate(messages):
        content = m.get("content") if isinstance(m, Mapping) else getattr(m, "content", None)
        if not isinstance(content, (list, tuple)):
            continue
        for pi, part in enumerate(content):
            if not isinstance(part, Mapping):
                continue
            typ = part.get("type")
            if typ not in IMAGE_TYPES and typ not in VIDEO_TYPES:
                continue
            param = f"messages[{mi}].content[{pi}]"
            kind = "image" if typ in IMAGE_TYPES else "video"
            if len(out) >= limits.max_parts:
                raise MediaError(f"more than {limits.max_parts} media parts in one request", param)
            url = _url_of(part, typ) or _url_of(part, "image_url" if kind == "image" else "video_url") or _url_of(part, "url")
            if url is None:
                raise MediaError(f"{typ} part carries no URL", param)
            cap = limits.max_image_bytes if kind == "image" else limits.max_video_bytes
            mime, raw = split_data_url(url, param, cap)
            total += len(raw)
            if total > limits.max_total_bytes:
                raise MediaError(f"media parts exceed {limits.max_total_bytes} bytes in total", param)
            w = h = None
            if kind == "image":
                found, w, h = sniff_image(raw)
                if found is None or found not in IMAGE_MIMES:
                    raise MediaError("unrecognised image container (png, jpeg, gif and webp are accepted)", param)
                if mime not in IMAGE_MIMES or (mime != found and not (mime == "image/jpg" and found == "image/jpeg")):
                    raise MediaError(f"declared type {mime!r} does not match the {found} payload", param)
                if w is None or h is None or w <= 0 or h <= 0:
                    raise MediaError("image header carries no usable dimensions", param)
                if w > limits.max_side or h > limits.max_side or w * h > limits.max_pixels:
                    raise MediaError(f"image of {w}x{h} pixels exceeds the limit of {limits.max_pixels} pixels "
                                     f"({limits.max_side} per side)", param)
                mime = found
            else:
                found = sniff_video(raw)
                if found is None or mime not in VIDEO_MIMES or found != mime:
                    raise MediaError("unrecognised or mismatched video container (mp4 and webm are accepted)", param)
            out.append(MediaPart(kind, mime, len(raw), w, h, mi, pi))
    return out
