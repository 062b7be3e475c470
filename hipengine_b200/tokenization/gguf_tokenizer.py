"""Tokenizers rebuilt from GGUF metadata.

The reference rebuilds a HF ``tokenizers`` BPE from ``tokenizer.ggml.*`` keys with
the Qwen split regex and an incremental byte decoder
(``hipengine/tokenization/gguf.py:11-40``).  The same construction is used here
when the file carries a vocabulary; random-init benchmark checkpoints carry
none, so they get ``ByteTokenizer`` (UTF-8 bytes <-> ids, every other id
rendered as ``<|id|>``), which keeps text APIs, stop strings and SSE framing
exercisable without a real vocabulary.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence

QWEN_SPLIT_REGEX = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                    r"\s*[\r\n]+|\s+(?!\S)|\s+")


class StreamDecoder:
    """Incremental detokenizer that never emits a partial UTF-8 sequence."""

    def __init__(self, tok: "BaseTokenizer"):
        self.tok = tok
        self.ids: List[int] = []
        self.emitted = 0

    def feed(self, ids: Sequence[int]) -> str:
        self.ids.extend(int(i) for i in ids)
        text = self.tok.decode(self.ids)
        # hold back a trailing replacement character: it may be an incomplete multi-byte sequence
        safe = len(text)
        while safe > self.emitted and text[safe - 1] == "�":
            safe -= 1
        out = text[self.emitted:safe]
        self.emitted = safe
        return out

    def flush(self) -> str:
        text = self.tok.decode(self.ids)
        out = text[self.emitted:]
        self.emitted = len(text)
        return out


class BaseTokenizer:
    vocab_size: int = 0
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    special: Dict[str, int] = {}

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int]) -> str:
        raise NotImplementedError

    def stream_decoder(self) -> StreamDecoder:
        return StreamDecoder(self)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self.special.get(tok)


class ByteTokenizer(BaseTokenizer):
    """UTF-8 bytes map to ids [3, 259); specials: 0 <|endoftext|>, 1 <|im_start|>, 2 <|im_end|>."""

    SPECIALS = ("<|endoftext|>", "<|im_start|>", "<|im_end|>")
    _ID_RE = re.compile(r"<\|(\d+)\|>")

    def __init__(self, vocab_size: int):
        self.vocab_size = int(vocab_size)
        self.eos_token_id = 0
        self.bos_token_id = None
        self.special = {s: i for i, s in enumerate(self.SPECIALS)}
        extra = {"<think>": 259, "</think>": 260, "<tool_call>": 261, "</tool_call>": 262}
        for k, v in extra.items():
            if v < self.vocab_size:
                self.special[k] = v
        self._special_re = re.compile("|".join(re.escape(s) for s in sorted(self.special, key=len, reverse=True))
                                      + r"|<\|\d+\|>")
        self._inv = {v: k for k, v in self.special.items()}

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        pos = 0
        for m in self._special_re.finditer(text):
            out.extend(3 + b for b in text[pos:m.start()].encode("utf-8"))
            s = m.group(0)
            if s in self.special:
                out.append(self.special[s])
            else:
                out.append(int(self._ID_RE.match(s).group(1)) % self.vocab_size)
            pos = m.end()
        out.extend(3 + b for b in text[pos:].encode("utf-8"))
        return [i % self.vocab_size for i in out]

    def decode(self, ids: Sequence[int]) -> str:
        parts: List[str] = []
        buf = bytearray()
        for i in ids:
            i = int(i)
            if 3 <= i < 259:
                buf.append(i - 3)
                continue
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            parts.append(self._inv.get(i, f"<|{i}|>"))
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)


class GGUFBPETokenizer(BaseTokenizer):
    """Byte-level BPE built with the ``tokenizers`` library from GGUF vocabulary + merges."""

    def __init__(self, tokens: Sequence[str], merges: Sequence[str], token_types: Optional[Sequence[int]] = None,
                 eos_id: Optional[int] = None, bos_id: Optional[int] = None, pre: str = "qwen2"):
        from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers
        vocab = {t: i for i, t in enumerate(tokens)}
        mg = []
        for m in merges:
            a, _, b = m.partition(" ")
            mg.append((a, b))
        tk = Tokenizer(models.BPE(vocab=vocab, merges=mg, fuse_unk=False, byte_fallback=False))
        tk.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(QWEN_SPLIT_REGEX), behavior="isolated", invert=False),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        tk.decoder = decoders.ByteLevel()
        specials = []
        if token_types is not None:
            specials = [tokens[i] for i, tt in enumerate(token_types) if tt in (3, 4)]  # CONTROL, USER_DEFINED
        if specials:
            from tokenizers import AddedToken
            tk.add_special_tokens([AddedToken(s, special=True, normalized=False) for s in specials])
        self._tk = tk
        self.vocab_size = len(tokens)
        self.eos_token_id = eos_id
        self.bos_token_id = bos_id
        self.special = {s: vocab[s] for s in specials}

    def encode(self, text: str) -> List[int]:
        return self._tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self._tk.decode(list(ids), skip_special_tokens=False)

    def token_to_id(self, tok: str) -> Optional[int]:
        return self._tk.token_to_id(tok)


def tokenizer_from_metadata(meta: Mapping[str, Any], vocab_size: int) -> BaseTokenizer:
    tokens = meta.get("tokenizer.ggml.tokens")
    merges = meta.get("tokenizer.ggml.merges")
    if tokens and merges and meta.get("tokenizer.ggml.model", "gpt2") == "gpt2":
        try:
            return GGUFBPETokenizer(tokens, merges, meta.get("tokenizer.ggml.token_type"),
                                    meta.get("tokenizer.ggml.eos_token_id"), meta.get("tokenizer.ggml.bos_token_id"),
                                    meta.get("tokenizer.ggml.pre", "qwen2"))
        except Exception:
            pass
    return ByteTokenizer(vocab_size)
