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

import re
from typing import Any, Dict, List, Mapping, Optional, Sequence

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


class GGUFSPMTokenizer(BaseTokenizer):
    """SentencePiece-style tokenizer rebuilt from GGUF metadata (``tokenizer.ggml.model = llama``; Gemma files).

    Text is split on special tokens, spaces become U+2581, then adjacent symbols are merged greedily by the score
    of the merged piece (highest first, leftmost on ties) -- the bigram-queue procedure llama.cpp uses for SPM
    vocabularies; characters without a piece fall back to ``<0xNN>`` byte tokens.  Counterpart of the reference's
    Gemma tokenizer (``hipengine/tokenization/``, "Gemma 4 SPM-style").
    """

    def __init__(self, tokens: Sequence[str], scores: Sequence[float], token_types: Optional[Sequence[int]] = None,
                 eos_id: Optional[int] = None, bos_id: Optional[int] = None, add_space_prefix: bool = False):
        self.tokens = list(tokens)
        self.scores = list(scores) if scores else [0.0] * len(tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        self.vocab_size = len(self.tokens)
        self.eos_token_id, self.bos_token_id = eos_id, bos_id
        self.add_space_prefix = add_space_prefix
        tt = list(token_types) if token_types is not None else [1] * len(tokens)
        self.special = {t: i for i, t in enumerate(self.tokens) if tt[i] in (3, 4)}
        self.byte_ids = {}
        for i, t in enumerate(self.tokens):
            if tt[i] == 6 or (len(t) == 6 and t.startswith("<0x") and t.endswith(">")):
                try:
                    self.byte_ids[int(t[3:5], 16)] = i
                except ValueError:
                    pass
        self._special_re = (re.compile("|".join(re.escape(x) for x in sorted(self.special, key=len, reverse=True)))
                            if self.special else None)
        self.unk_id = self.vocab.get("<unk>", 0)

    def _encode_piece(self, text: str) -> List[int]:
        import heapq
        if not text:
            return []
        syms = list(text)
        n = len(syms)
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap = []

        def push(i):
            j = nxt[i]
            if i < 0 or j < 0:
                return
            merged = syms[i] + syms[j]
            tid = self.vocab.get(merged)
            if tid is not None:
                heapq.heappush(heap, (-self.scores[tid], i, merged))

        for i in range(n - 1):
            push(i)
        while heap:
            _, i, merged = heapq.heappop(heap)
            j = nxt[i] if alive[i] else -1
            if j < 0 or not alive[j] or syms[i] + syms[j] != merged:
                continue
            syms[i] = merged
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] >= 0:
                prev[nxt[j]] = i
            if prev[i] >= 0:
                push(prev[i])
            push(i)
        out: List[int] = []
        i = 0
        while i >= 0:
            if alive[i]:
                tid = self.vocab.get(syms[i])
                if tid is not None:
                    out.append(tid)
                else:
                    for b in syms[i].encode("utf-8"):
                        out.append(self.byte_ids.get(b, self.unk_id))
            i = nxt[i]
        return out

    def encode(self, text: str) -> List[int]:
        out: List[int] = []
        pos = 0
        first = True

        def plain(chunk: str) -> None:
            nonlocal first
            if not chunk:
                return
            t = chunk.replace(" ", "\u2581")
            if first and self.add_space_prefix and not t.startswith("\u2581"):
                t = "\u2581" + t
            first = False
            out.extend(self._encode_piece(t))

        if self._special_re is not None:
            for m in self._special_re.finditer(text):
                plain(text[pos:m.start()])
                out.append(self.special[m.group(0)])
                first = False
                pos = m.end()
        plain(text[pos:])
        return out

    def decode(self, ids: Sequence[int]) -> str:
        parts: List[str] = []
        buf = bytearray()
        inv_bytes = {v: k for k, v in self.byte_ids.items()}
        for i in ids:
            i = int(i)
            if i in inv_bytes:
                buf.append(inv_bytes[i])
                continue
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if 0 <= i < self.vocab_size:
                parts.append(self.tokens[i])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts).replace("\u2581", " ")

    def token_to_id(self, tok: str) -> Optional[int]:
        return self.vocab.get(tok)


def tokenizer_from_metadata(meta: Mapping[str, Any], vocab_size: int) -> BaseTokenizer:
    if meta.get("tokenizer.ggml.model") == "llama" and meta.get("tokenizer.ggml.tokens"):
        try:
            return GGUFSPMTokenizer(meta["tokenizer.ggml.tokens"], meta.get("tokenizer.ggml.scores") or [],
                                    meta.get("tokenizer.ggml.token_type"), meta.get("tokenizer.ggml.eos_token_id"),
                                    meta.get("tokenizer.ggml.bos_token_id"),
                                    bool(meta.get("tokenizer.ggml.add_space_prefix", False)))
        except Exception:
            pass
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
