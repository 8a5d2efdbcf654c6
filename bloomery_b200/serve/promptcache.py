"""Host-RAM prompt cache: saved sequence states keyed by their token ids, LRU by bytes.

Rules taken from the reference (``crates/serve/src/promptcache.rs:1-21``): a lookup ranks
states by how many leading positions they share with the new prompt (what is *keepable*); a
newer state evicts older ones it wholly covers; states whose copy is still in flight are
pinned and never evicted; eviction is least recently used until the byte budget holds.
"""
from __future__ import annotations

import collections
import threading
from typing import Dict, List, Optional, Sequence, Tuple

from .engine import Saved


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = min(len(a), len(b))
    i = 0
    while i < n and a[i] == b[i]:
        i += 1
    return i


class PromptCache:
    def __init__(self, budget_bytes: int):
        self.budget = max(0, int(budget_bytes))
        self.used = 0
        self._items: "collections.OrderedDict[Tuple[int, ...], Saved]" = collections.OrderedDict()
        self._pinned: Dict[Tuple[int, ...], int] = {}
        self._lock = threading.Lock()
        self.hits = self.misses = self.evictions = 0
        self.seconds = 0.0

    def __len__(self) -> int:
        return len(self._items)

    def put(self, saved: Optional[Saved], pending: bool = False) -> bool:
        if saved is None or self.budget == 0 or saved.n_bytes > self.budget:
            return False
        with self._lock:
            key = saved.ids
            if key in self._items:
                self._items.move_to_end(key)
                return True
            # a newer state evicts the states it wholly covers
            for k in [k for k in self._items if len(k) <= len(key) and key[:len(k)] == k and k not in self._pinned]:
                self._drop(k)
            self._items[key] = saved
            self.used += saved.n_bytes
            if pending:
                self._pinned[key] = self._pinned.get(key, 0) + 1
            self._evict()
            return key in self._items

    def settle(self, ids: Sequence[int]) -> None:
        """The async copy of a pending state finished: it may be evicted again."""
        with self._lock:
            k = tuple(ids)
            if k in self._pinned:
                self._pinned[k] -= 1
                if self._pinned[k] <= 0:
                    del self._pinned[k]
            self._evict()

    def _drop(self, key) -> None:
        s = self._items.pop(key)
        self.used -= s.n_bytes
        self.evictions += 1

    def _evict(self) -> None:
        for k in list(self._items):
            if self.used <= self.budget:
                break
            if k in self._pinned:
                continue
            self._drop(k)

    def lookup(self, ids: Sequence[int], at_least: int = 1) -> Tuple[Optional[Saved], int]:
        """Best saved state for a prompt: (state, positions keepable)."""
        with self._lock:
            best, best_n = None, 0
            for k, s in self._items.items():
                n = common_prefix(k, ids)
                if n > best_n:
                    best, best_n = s, n
            if best is None or best_n < at_least:
                self.misses += 1
                return None, 0
            self._items.move_to_end(best.ids)
            self.hits += 1
            return best, best_n

    def clear(self) -> None:
        with self._lock:
            self._items.clear()
            self._pinned.clear()
            self.used = 0

    def stats(self) -> Dict[str, float]:
        return {"entries": len(self._items), "bytes": self.used, "budget": self.budget, "hits": self.hits,
                "misses": self.misses, "evictions": self.evictions, "seconds": self.seconds}
