"""Hot-vocabulary draft head: the NextN draft scores only a leading slice of the vocabulary.

The draft head is the largest single read of a draft pass (248 320 x 5120 Q6_K rows = 1.04 GB on the 27B, against
~0.4 GB for the rest of the NextN block), and a draft that the target rejects costs nothing but the rejected slot.
BPE vocabularies are ordered by merge rank, so the low ids carry most of the probability mass of running text: with
the head cut to its first ``rows`` rows the draft's argmax is unchanged whenever the full-head argmax lies in the
slice.  The rows are a prefix of the weight as stored, so the small head is the same device buffer with a smaller row
count: nothing is gathered or copied.

Verification always uses the full head; the slice only decides what is proposed.  A per-request rule decides, from
the request's own committed tokens alone (never from proposals, never from another request), whether the next cycle
may use the slice: the token the cycle is anchored on must lie inside it and at most one of the request's last
``window`` committed tokens may lie outside it.  Text that keeps leaving the slice (code with rare identifiers, other
scripts) drafts with the full head instead of wasting draft slots.

Behavioural counterpart: hipengine/speculative/draft_vocab.py:1-251 (fixed prefix + recent-miss rule; the reference's
per-request table of extra rows is not kept here: an out-of-slice token is simply a miss).
"""
from __future__ import annotations

from typing import Dict, Hashable, Optional, Sequence

DEFAULT_ROWS = 98_304          # rows of the slice before clipping to the vocabulary
DEFAULT_WINDOW = 32            # committed tokens the recent-miss rule looks back over
ROW_QUANTUM = 64               # the slice is a whole number of GEMV work items for every rows-per-item setting


def resolve_hot_vocab_rows(setting, vocab: int) -> int:
    """``off`` / ``0`` / None -> 0 (full head only); ``auto`` -> the default slice; an integer -> that many rows.
    The result is clipped below the vocabulary (a slice that covers it all is no slice) and rounded down to
    ``ROW_QUANTUM``."""
    if setting in (None, "", "off", "0", 0, False):
        return 0
    rows = DEFAULT_ROWS if setting in ("auto", "on", True) else int(setting)
    if rows <= 0:
        return 0
    if rows >= vocab:
        rows = vocab // 2
    rows = (rows // ROW_QUANTUM) * ROW_QUANTUM
    return rows if 0 < rows < vocab else 0


class DraftVocabRule:
    """One request's recent-miss bookkeeping (append-only over its committed tokens)."""

    __slots__ = ("rows", "window", "scanned", "_miss_a", "_miss_b")

    def __init__(self, rows: int, window: int = DEFAULT_WINDOW):
        if rows <= 0 or window < 1:
            raise ValueError("rows and window must be positive")
        self.rows, self.window = int(rows), int(window)
        self.scanned = 0
        self._miss_a = -1          # index of the most recent committed token outside the slice
        self._miss_b = -1          # and of the one before it

    def catch_up(self, prompt: Sequence[int], generated: Sequence[int]) -> int:
        """Consume the committed history ``prompt + generated`` beyond what was already seen; returns how many
        tokens were read.  A history shorter than what was seen belongs to another request: start over."""
        n_p, total = len(prompt), len(prompt) + len(generated)
        if total < self.scanned:
            self.scanned, self._miss_a, self._miss_b = 0, -1, -1
        first = self.scanned
        for i in range(first, total):
            t = prompt[i] if i < n_p else generated[i - n_p]
            if t >= self.rows or t < 0:
                self._miss_b, self._miss_a = self._miss_a, i
        self.scanned = total
        return total - first

    def fits(self, anchor: int) -> bool:
        """May the cycle anchored on ``anchor`` (the last committed token) draft with the slice?"""
        if not 0 <= anchor < self.rows:
            return False
        # only the second most recent miss matters: outside the window means at most one miss inside it
        return self._miss_b < 0 or self._miss_b + self.window < self.scanned


class DraftVocabBook:
    """The rules of all live requests of one runner, and the counters the capability record shows."""

    def __init__(self, rows: int, window: int = DEFAULT_WINDOW):
        self.rows, self.window = int(rows), int(window)
        self._rules: Dict[Hashable, DraftVocabRule] = {}
        self.stats = {"small_head_cycles": 0, "full_head_cycles": 0}

    def fits(self, rid: Hashable, prompt: Sequence[int], generated: Sequence[int], anchor: int) -> bool:
        rule = self._rules.get(rid)
        if rule is None:
            rule = self._rules[rid] = DraftVocabRule(self.rows, self.window)
        rule.catch_up(prompt, generated)
        return rule.fits(anchor)

    def decide(self, rows_fit: Sequence[bool]) -> bool:
        """One head per cycle: the slice only when every row of the cycle may use it."""
        small = bool(rows_fit) and all(rows_fit)
        self.stats["small_head_cycles" if small else "full_head_cycles"] += 1
        return small

    def drop(self, rid: Hashable) -> None:
        self._rules.pop(rid, None)

    def clear(self) -> None:
        self._rules.clear()

    def __len__(self) -> int:
        return len(self._rules)

    def as_dict(self) -> Optional[dict]:
        return {"rows": self.rows, "window": self.window, "requests": len(self._rules), **self.stats}
