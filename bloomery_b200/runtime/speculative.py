"""Speculative decoding on the host side: draft sources, verification bookkeeping and the
width chooser.

The contract is the reference's (``crates/runtime/src/lib.rs:13-17``, ``speculative.rs:250``):
a draft changes which passes run and never a token.  Verification feeds the last accepted
token and the k drafted ids as k+1 rows of one pass; rows of a pass are bit-equal to their
own 1-row steps, so the greedy picks are the ones plain decoding would have made; the
longest agreeing prefix is kept and the KV rows of the rest are cut.

* :class:`NgramDraft` -- prompt-lookup draft: the longest recent n-gram that occurred before
  proposes what followed it (the reference's n-gram lookup draft).
* :class:`WidthChooser` -- picks the draft width k that maximises expected accepted tokens
  per unit of measured pass time (``crates/runtime/src/width.rs:1-50``): per-depth acceptance
  rates are running means, pass walls are measured per row count.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple


class NgramDraft:
    def __init__(self, max_n: int = 4, min_n: int = 1):
        self.max_n, self.min_n = max_n, min_n

    def propose(self, ids: Sequence[int], k: int) -> List[int]:
        n_ids = len(ids)
        if k <= 0 or n_ids < self.min_n + 1:
            return []
        for n in range(min(self.max_n, n_ids - 1), self.min_n - 1, -1):
            tail = list(ids[n_ids - n:])
            # most recent earlier occurrence
            for start in range(n_ids - n - 1, -1, -1):
                if list(ids[start:start + n]) == tail:
                    nxt = list(ids[start + n:start + n + k])
                    if nxt:
                        return nxt
                    break
        return []


class MtpDraft:
    """Draft source backed by the model's own multi-token-prediction layer: the engine runs that layer beside
    every pass and keeps, per slot, the id it predicts after the next token (``crates/runtime/src/mtp``:
    the MTP window; one draft per step here)."""

    wants_slot = True

    def __init__(self, engine):
        self.engine = engine

    def propose(self, ids: Sequence[int], k: int, slot: int = 0) -> List[int]:
        return self.engine.draft(slot, len(ids))[:k] if k > 0 else []


class WidthChooser:
    def __init__(self, max_width: int = 7, prior_accept: float = 0.5):
        self.max_width = max_width
        self.acc_n = [1.0] * (max_width + 1)           # trials at depth d (1-based)
        self.acc_k = [prior_accept] * (max_width + 1)  # acceptances at depth d
        self.wall: Dict[int, float] = {}                # rows in the pass -> seconds (running mean)
        self.wall_n: Dict[int, int] = {}

    def observe_pass(self, rows: int, seconds: float) -> None:
        n = self.wall_n.get(rows, 0)
        self.wall[rows] = (self.wall.get(rows, seconds) * n + seconds) / (n + 1)
        self.wall_n[rows] = min(n + 1, 64)

    def observe_accept(self, drafted: int, accepted: int) -> None:
        for d in range(1, drafted + 1):
            if d - 1 > accepted:
                break                                   # depth d was only tried if all before it were accepted
            self.acc_n[d] += 1.0
            if d <= accepted:
                self.acc_k[d] += 1.0

    def rate(self, d: int) -> float:
        return self.acc_k[d] / self.acc_n[d]

    def _wall(self, rows: int) -> float:
        if rows in self.wall:
            return self.wall[rows]
        if not self.wall:
            return 1.0 + 0.05 * (rows - 1)              # no measurement yet: rows are cheap on a latency-bound step
        known = sorted(self.wall)
        lo = max([r for r in known if r <= rows], default=known[0])
        hi = min([r for r in known if r >= rows], default=known[-1])
        if lo == hi:
            return self.wall[lo] * (1.0 + 0.03 * (rows - lo))
        t = (rows - lo) / (hi - lo)
        return self.wall[lo] * (1 - t) + self.wall[hi] * t

    def choose(self, available: int) -> int:
        """Draft ids to verify next (0 = plain step)."""
        best_k, best_v = 0, 1.0 / self._wall(1)
        exp_tokens, p_all = 1.0, 1.0
        for k in range(1, min(available, self.max_width) + 1):
            p_all *= self.rate(k)
            exp_tokens += p_all
            v = exp_tokens / self._wall(k + 1)
            if v > best_v * 1.02:
                best_k, best_v = k, v
        return best_k


def accept_prefix(drafted: Sequence[int], picks: Sequence[int]) -> int:
    """picks[i] is the greedy token after row i (row 0 = last accepted token, row i = drafted[i-1]).
    Returns how many drafted ids are kept."""
    n = 0
    while n < len(drafted) and n < len(picks) and picks[n] == drafted[n]:
        n += 1
    return n
