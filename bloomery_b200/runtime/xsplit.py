"""Prompt-time split of a layer's host-resident experts: which of them are copied to the card for this prompt unit and
which stay with the host's own expert pass, as a pure function of the unit's routed counts and of priced constants.

The balance (the reference's ``crates/runtime/src/xsplit.rs`` states the same one): after a layer's routing the card's
side (copies of the experts it takes, then their products) and the host's side (its union pass over the experts left to
it) run side by side and the layer waits for the longer.  An expert routed ``m`` rows of the unit costs the host
``max(W, c * m)`` (its weights cross the host's DRAM once whatever ``m``), and costs the card its copy at the rate the
lane has BESIDE the union (the union's weight reads hold the host's DRAM for their share of its window) plus
``f + k * m``.  Walking the host experts hottest first, an expert moves to the card while the card's side after it stays
under the host's side without it; the walk stops short of the crossing, so the same counts always give the same split,
and no constant is a timing taken during the prompt.

Here the rule prices the two prompt paths of the tiered engine (``runtime/tiered.py``): the pass path (rows in passes of
8, cold experts on the host leg) and the stream path (the layer's stacks copied into the card ring, every product on the
card).  :func:`stream_gate` is the least prompt width at which the rule would move the hottest host expert at all: a
prompt narrower than that streams nothing, so it takes the pass path.
"""
from __future__ import annotations

import dataclasses
from typing import List, Sequence, Tuple


@dataclasses.dataclass(frozen=True)
class Costs:
    lane_b_per_us: float        # pinned host -> card copy rate with the host's DRAM otherwise idle [B/us]
    expert_bytes: int           # one expert's gate + up + down in the resident layout [B]
    host_us_fixed: float        # W: the host's cost of an expert whatever its rows [us]
    host_us_per_row: float      # c [us / routed row]
    card_us_fixed: float        # f: the card's fixed cost of one more expert in the grouped product [us]
    card_us_per_row: float      # k [us / routed row]
    n_expert: int
    top_k: int

    def check(self) -> None:
        for name in ("lane_b_per_us", "expert_bytes"):
            if not getattr(self, name) > 0:
                raise ValueError(f"{name} must be above 0")
        for name in ("host_us_fixed", "host_us_per_row", "card_us_fixed", "card_us_per_row"):
            v = getattr(self, name)
            if not (v >= 0 and v == v and v != float("inf")):
                raise ValueError(f"{name} must be finite and 0 or more")
        if self.n_expert < 1 or not 1 <= self.top_k <= self.n_expert:
            raise ValueError("top_k of n_expert experts")


@dataclasses.dataclass(frozen=True)
class Split:
    streamed: Tuple[int, ...]   # host experts copied to the card for this unit, hottest first
    kept: Tuple[int, ...]       # routed host experts left to the host's pass
    card_us: float              # the card's side after the streamed ones
    host_us: float              # the host's side without them
    beside_b_per_us: float      # the copy rate the split was priced at


def host_us(c: Costs, rows: int) -> float:
    return max(c.host_us_fixed, c.host_us_per_row * rows) if rows > 0 else 0.0


def burst_share(c: Costs, rows: int, listed: int) -> float:
    """The share of its own window the union spends reading weights (its fixed costs against its whole cost): what a
    copy beside it loses of the lane."""
    fixed = c.host_us_fixed * listed
    whole = fixed + c.host_us_per_row * rows
    return fixed / whole if whole > 0 else 0.0


def rank(counts: Sequence[int], host: Sequence[int]) -> List[int]:
    """The routed host experts hottest first, the lower id first on a tie."""
    return sorted((e for e in host if counts[e] > 0), key=lambda e: (-counts[e], e))


def split(counts: Sequence[int], host: Sequence[int], c: Costs, card_base_us: float = 0.0) -> Split:
    """``counts[e]``: rows of the unit routed to expert e; ``host``: the experts that are not on the card;
    ``card_base_us``: what the card's side already holds (its resident experts' products)."""
    c.check()
    if len(counts) != c.n_expert:
        raise ValueError(f"{len(counts)} counts for a layer of {c.n_expert} experts")
    seen = set()
    for e in host:
        if not 0 <= e < c.n_expert or e in seen:
            raise ValueError(f"host expert {e}: each expert of the layer at most once")
        seen.add(e)
    ranked = rank(counts, host)
    rows = sum(counts[e] for e in ranked)
    rate = c.lane_b_per_us * (1.0 - burst_share(c, rows, len(ranked)))
    card, union = float(card_base_us), sum(host_us(c, counts[e]) for e in ranked)
    moved = 0
    if rate > 0:
        for e in ranked:
            m = counts[e]
            card_next = card + c.expert_bytes / rate + c.card_us_fixed + c.card_us_per_row * m
            union_next = union - host_us(c, m)
            if card_next > union_next:
                break
            card, union, moved = card_next, union_next, moved + 1
    return Split(tuple(ranked[:moved]), tuple(ranked[moved:]), card, union, rate)


def stream_gate(c: Costs, n_host: int, limit: int = 1 << 16) -> int:
    """The least prompt width (rows) whose even routing over the layer's experts moves at least one host expert to the
    card; ``limit`` + 1 when none up to ``limit`` does.  Even routing gives every expert ``rows * top_k / n_expert``
    rows: the most cautious unit, no expert hotter than the rest."""
    c.check()
    if not 0 < n_host <= c.n_expert:
        raise ValueError("n_host of the layer's experts")
    host = list(range(n_host))

    def streams(rows: int) -> bool:
        per = rows * c.top_k // c.n_expert
        if per <= 0:
            return False
        return bool(split([per] * c.n_expert, host, c).streamed)

    if not streams(limit):
        return limit + 1
    lo, hi = 1, limit                      # the union grows with the width and the copy does not: one crossing
    while lo < hi:
        mid = (lo + hi) // 2
        if streams(mid):
            hi = mid
        else:
            lo = mid + 1
    return lo
