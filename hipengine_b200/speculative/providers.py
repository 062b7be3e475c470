"""Draft providers that need no draft network, and the provider registry.

``PromptLookupDrafter`` proposes the tokens that followed the most recent earlier occurrence of the request's
current suffix n-gram in its own history (prompt + generated tokens): summaries, code edits and tool transcripts
repeat long spans of their input, and a hit costs nothing but the verify rows.  ``NGramCacheDrafter`` keeps a
bounded table of n-gram continuations across requests (most recent continuation wins).  Both are deterministic,
i.e. one-hot proposal distributions; the verifier's exact sampling rule handles them without draft probabilities.

``LookupCycle`` joins a drafter to the chain verify / accept / commit path of ``speculative/mtp.py``; it works on
any checkpoint (no NextN block needed).  Reference counterparts: ``hipengine/speculative/prompt_lookup.py``,
``hipengine/speculative/ngram_mod.py`` and ``hipengine/speculative/registry.py``
(``register_builtin_speculative_providers``, ``SpeculativeProviderConfig``).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class SpeculativeProviderConfig:
    name: str = "mtp"                 # mtp | prompt_lookup | ngram
    max_depth: int = 3
    min_ngram: int = 2
    max_ngram: int = 4
    table_entries: int = 1 << 16      # ngram provider: bound of the shared table
    hot_vocab: object = "off"         # mtp provider: off | auto | rows of the draft head slice (draft_vocab.py)
    draft_model: object = None        # gemma4_mtp provider: path of the assistant head GGUF, loaded weights, or "random"


class PromptLookupDrafter:
    """Longest-suffix match in the request's own token history."""

    def __init__(self, min_ngram: int = 2, max_ngram: int = 4):
        assert 1 <= min_ngram <= max_ngram
        self.min_ngram, self.max_ngram = min_ngram, max_ngram

    def propose(self, history: Sequence[int], depth: int) -> List[int]:
        """Up to ``depth`` tokens that followed the latest earlier occurrence of the longest matching suffix;
        an empty list when no n-gram of at least ``min_ngram`` tokens repeats."""
        n_hist = len(history)
        for n in range(min(self.max_ngram, n_hist - 1), self.min_ngram - 1, -1):
            suffix = list(history[n_hist - n:])
            # scan right to left so that the most recent occurrence wins; the match must leave a continuation
            for start in range(n_hist - n - 1, -1, -1):
                if list(history[start:start + n]) == suffix:
                    cont = list(history[start + n:start + n + depth])
                    if cont:
                        return cont
        return []

    def observe(self, history: Sequence[int]) -> None:       # per-request drafter: nothing to learn
        pass


class NGramCacheDrafter:
    """Bounded LRU table n-gram -> continuation, shared by all requests of an engine."""

    def __init__(self, min_ngram: int = 2, max_ngram: int = 4, table_entries: int = 1 << 16, span: int = 8):
        self.min_ngram, self.max_ngram, self.cap, self.span = min_ngram, max_ngram, table_entries, span
        self.table: "OrderedDict[Tuple[int, ...], Tuple[int, ...]]" = OrderedDict()

    def observe(self, history: Sequence[int]) -> None:
        """Record the continuations of the n-grams that end inside the last ``span`` tokens of ``history``."""
        h = list(history)
        lo = max(0, len(h) - 2 * self.span)
        for n in range(self.min_ngram, self.max_ngram + 1):
            for start in range(lo, len(h) - n):
                key = tuple(h[start:start + n])
                cont = tuple(h[start + n:start + n + self.span])
                if cont:
                    self.table[key] = cont
                    self.table.move_to_end(key)
        while len(self.table) > self.cap:
            self.table.popitem(last=False)

    def propose(self, history: Sequence[int], depth: int) -> List[int]:
        h = list(history)
        for n in range(min(self.max_ngram, len(h)), self.min_ngram - 1, -1):
            cont = self.table.get(tuple(h[len(h) - n:]))
            if cont:
                return list(cont[:depth])
        return PromptLookupDrafter(self.min_ngram, self.max_ngram).propose(h, depth)


class LookupCycle:
    """Chain speculation with a host drafter: propose from token histories, pad short proposals, verify on the
    device.  ``cycle`` returns ``None`` when no row has a proposal (the caller then takes the plain decode step,
    which is cheaper than a verify forward that cannot accept anything)."""

    def __init__(self, ex, drafter, max_depth: int = 3, max_requests: int = 8):
        from .mtp import ChainVerifyCycle
        self.verify = ChainVerifyCycle(ex, max_depth, max_requests)
        self.drafter = drafter
        self.max_depth, self.max_requests = max_depth, max_requests
        self.stats = self.verify.stats
        self.stats.update({"proposed_rows": 0, "empty_rows": 0, "skipped_cycles": 0})

    def capability(self):
        from dataclasses import replace
        return replace(self.verify.capability(), provider=type(self.drafter).__name__)

    def reset_slot(self, slot: int) -> None:
        pass

    def after_prefill(self, batch, h) -> None:
        pass

    def cycle(self, slots, last_tokens, positions, depth, temperature=None, seeds=None, counters=None,
              histories: Optional[Sequence[Sequence[int]]] = None):
        assert histories is not None and len(histories) == len(slots)
        props = [self.drafter.propose(h, depth) for h in histories]
        k = max((len(p) for p in props), default=0)
        if k == 0:
            self.stats["skipped_cycles"] += 1
            return None
        drafts = []
        for p, last in zip(props, last_tokens):
            self.stats["proposed_rows" if p else "empty_rows"] += 1
            drafts.append(list(p) + [int(last)] * (k - len(p)))     # padding is almost surely rejected; harmless
        return self.verify.cycle_with_drafts(slots, last_tokens, positions, drafts, temperature, seeds, counters)


# ---------------------------------------------------------------------------------------------- registry
_PROVIDERS: Dict[str, Callable] = {}


def register_speculative_provider(name: str, factory: Callable) -> None:
    """``factory(executor, cfg: SpeculativeProviderConfig, max_requests) -> cycle object or None``."""
    _PROVIDERS[name] = factory


def _gemma4_mtp_factory(ex, cfg: SpeculativeProviderConfig, max_requests: int):
    """Gemma 4 backbone + its assistant head (a separate artifact named by ``draft_model``)."""
    if getattr(getattr(ex, "cfg", None), "arch", "") != "gemma4" or cfg.draft_model in (None, "", "off"):
        return None
    if getattr(getattr(ex, "ctx", None), "world", 1) != 1:
        return None                      # the head reads the backbone's KV heads of one rank's shard only
    from ..loading.weights import ModelWeights
    from ..models.gemma4_assistant import Gemma4AssistantHead
    from .gemma4_mtp import AssistantMTPCycle
    dm = cfg.draft_model
    if isinstance(dm, ModelWeights):
        weights = dm
    elif dm == "random":
        from ..loading.gemma4 import build_random_assistant
        from ..models.config import AssistantConfig, NAMED_ASSISTANTS
        acfg = next((a for a in NAMED_ASSISTANTS.values()
                     if a.backbone_hidden == ex.cfg.hidden and a.vocab == ex.cfg.vocab and a.n_heads == ex.cfg.n_heads),
                    None) or AssistantConfig(hidden=max(256, ex.cfg.hidden // 4 // 256 * 256),
                                             backbone_hidden=ex.cfg.hidden, ffn=2 * ex.cfg.hidden // 256 * 256,
                                             n_heads=ex.cfg.n_heads, vocab=ex.cfg.vocab)
        weights = build_random_assistant(acfg, ex.cfg, seed=0, device=ex.device)
    else:
        from ..loading.gemma4 import load_assistant_gguf
        weights = load_assistant_gguf(dm, ex.cfg, device=ex.device)
    head = Gemma4AssistantHead(ex, weights, max_rows=max_requests)
    return AssistantMTPCycle(ex, head, max_depth=max(1, cfg.max_depth), max_requests=max_requests)


def _mtp_factory(ex, cfg: SpeculativeProviderConfig, max_requests: int):
    if getattr(getattr(ex, "cfg", None), "arch", "") == "gemma4":
        return _gemma4_mtp_factory(ex, cfg, max_requests)     # this family's MTP head is the assistant artifact
    if not getattr(ex, "has_nextn", False):
        return None
    import os
    from .mtp import GraphedMTPCycle, MTPCycle
    # one captured graph per cycle on a single-GPU executor; the eager cycle elsewhere (HE_SPEC_GRAPH=0 forces it)
    single = getattr(getattr(ex, "ctx", None), "world", 1) == 1
    graphed = single and str(ex.device).startswith("cuda") and os.environ.get("HE_SPEC_GRAPH", "1") != "0"
    cls = GraphedMTPCycle if graphed else MTPCycle
    from .draft_vocab import resolve_hot_vocab_rows
    # the head slice is a row prefix of the full head: a vocabulary-sharded head (tensor parallel) has none
    rows = resolve_hot_vocab_rows(cfg.hot_vocab, ex.cfg.vocab) if single else 0
    return cls(ex, max_depth=max(1, cfg.max_depth), max_requests=max_requests, draft_head_rows=rows)


def _prompt_lookup_factory(ex, cfg: SpeculativeProviderConfig, max_requests: int):
    return LookupCycle(ex, PromptLookupDrafter(cfg.min_ngram, cfg.max_ngram), max(1, cfg.max_depth), max_requests)


def _ngram_factory(ex, cfg: SpeculativeProviderConfig, max_requests: int):
    return LookupCycle(ex, NGramCacheDrafter(cfg.min_ngram, cfg.max_ngram, cfg.table_entries),
                       max(1, cfg.max_depth), max_requests)


def register_builtin_speculative_providers() -> List[str]:
    register_speculative_provider("mtp", _mtp_factory)
    register_speculative_provider("gemma4_mtp", _gemma4_mtp_factory)
    register_speculative_provider("prompt_lookup", _prompt_lookup_factory)
    register_speculative_provider("ngram", _ngram_factory)
    return sorted(_PROVIDERS)


def speculative_provider_names() -> List[str]:
    if not _PROVIDERS:
        register_builtin_speculative_providers()
    return sorted(_PROVIDERS)


def build_speculative_provider(ex, cfg: SpeculativeProviderConfig, max_requests: int = 8):
    if not _PROVIDERS:
        register_builtin_speculative_providers()
    if cfg.name not in _PROVIDERS:
        raise ValueError(f"unknown speculative provider {cfg.name!r}; known: {sorted(_PROVIDERS)}")
    return _PROVIDERS[cfg.name](ex, cfg, max_requests)
