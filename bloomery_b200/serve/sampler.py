"""Token sampling over one row of logits (host oracle of the CUDA sampler).

Chain, as the reference states it (``crates/sampler/src/lib.rs:1-16,190-346``):
penalties (repeat: ``l <= 0 ? l*r : l/r`` once per distinct token of the window, then
``- (count*frequency + presence)``) -> top-k -> min-p (``logit >= max + ln(min_p)``) and
top-p (shortest best-first prefix whose mass, normalised over *all* top-k survivors and
untempered, reaches top_p) -> temperature -> softmax in f64 -> one draw ``u * total`` over
the running sums, ``u`` from xoshiro256** seeded through splitmix64 (53-bit uniform).
Every stage keeps at least one candidate.  Candidates are ordered (logit descending, id
ascending), the engine's greedy tie rule, so ``top_k = 1`` answers what greedy answers.
``temperature <= 0`` is the arg-max after the penalties.
"""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

MASK64 = (1 << 64) - 1


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 64
    seed: int = 0

    @classmethod
    def greedy(cls) -> "SamplingParams":
        return cls(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_last_n=0)

    @property
    def penalizes(self) -> bool:
        return self.repeat_last_n != 0 and (self.repeat_penalty != 1.0 or self.frequency_penalty != 0.0
                                            or self.presence_penalty != 0.0)


class Xoshiro256:
    """xoshiro256** seeded by splitmix64; ``next_f64`` is uniform in [0, 1) from the top 53 bits."""

    def __init__(self, seed: int):
        z = seed & MASK64
        s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & MASK64
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
            s.append(x ^ (x >> 31))
        self.s = s

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & MASK64

    def next_u64(self) -> int:
        s = self.s
        out = (self._rotl((s[1] * 5) & MASK64, 7) * 9) & MASK64
        t = (s[1] << 17) & MASK64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return out

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


def greedy_pick(row: np.ndarray) -> int:
    """Strictly greater wins, equal wins at the lower id, NaN never wins, all-NaN/-inf -> 0."""
    r = np.where(np.isnan(row), -np.inf, row)
    if r.size == 0:
        return 0
    m = r.max()
    if m == -np.inf:
        return 0
    return int(np.flatnonzero(r == m)[0])


def _sanitize(row: np.ndarray) -> np.ndarray:
    r = np.where(np.isnan(row), np.float32(-np.inf), row).astype(np.float32)
    return r + np.float32(0.0)          # -0.0 -> +0.0


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None):
        self.params = params or SamplingParams()
        self.rng = Xoshiro256(self.params.seed)
        self.candidates: List[Tuple[int, float]] = []

    def penalized(self, logits: np.ndarray, recent: Sequence[int]) -> np.ndarray:
        p = self.params
        row = _sanitize(logits).copy()
        window = list(recent)[-p.repeat_last_n:] if p.repeat_last_n > 0 else []
        counts = {}
        for t in window:
            if 0 <= t < row.size:
                counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            l = row[t]
            l = np.float32(l * np.float32(p.repeat_penalty)) if l <= 0 else np.float32(l / np.float32(p.repeat_penalty))
            l = np.float32(l - np.float32(np.float32(c) * np.float32(p.frequency_penalty) + np.float32(p.presence_penalty)))
            row[t] = -np.inf if np.isnan(l) else l
        return row

    def sample(self, logits: np.ndarray, recent: Sequence[int] = ()) -> int:
        p = self.params
        logits = np.asarray(logits, dtype=np.float32)
        self.candidates = []
        if logits.size == 0:
            return 0
        pen = p.penalizes and len(recent) > 0
        row = self.penalized(logits, recent) if pen else logits
        if p.temperature <= 0:
            i = greedy_pick(row)
            self.candidates = [(i, float(row[i]))]
            return i
        row = _sanitize(row)
        n = row.size
        k = p.top_k
        if 0 < k < n:
            # the k best under (logit desc, id asc): take everything >= the k-th value, order, cut
            kth = np.partition(row, n - k)[n - k]
            idx = np.flatnonzero(row >= kth)
        else:
            idx = np.arange(n)
        order = np.lexsort((idx, -row[idx].astype(np.float64)))
        idx = idx[order]
        if 0 < k < n:
            idx = idx[:k]
        vals = row[idx]
        mx = vals[0]
        if not np.isfinite(mx):
            self.candidates = [(int(idx[0]), float(vals[0]))]
            return int(idx[0])
        w1 = np.exp((vals - mx).astype(np.float64))
        norm = float(w1.sum()) if p.top_p < 1.0 else 0.0
        keep = len(idx)
        if p.min_p > 0:
            floor = np.float32(mx + np.float32(math.log(p.min_p)))
            keep = max(1, int(np.count_nonzero(vals >= floor)))     # sorted: survivors are a prefix
        if p.top_p < 1.0:
            mass = np.cumsum(w1[:keep] / norm)
            hit = np.flatnonzero(mass >= float(np.float32(p.top_p)))
            if hit.size:
                keep = int(hit[0]) + 1
        idx, vals = idx[:keep], vals[:keep]
        self.candidates = [(int(i), float(v)) for i, v in zip(idx, vals)]
        if keep == 1:
            return int(idx[0])
        inv_t = 1.0 / float(np.float32(p.temperature))
        w = np.exp((vals - vals[0]).astype(np.float64) * inv_t)
        cum = np.cumsum(w)
        u = self.rng.next_f64() * float(cum[-1])
        i = min(int(np.searchsorted(cum, u, side="right")), keep - 1)
        return int(idx[i])
