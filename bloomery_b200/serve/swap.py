"""More request slots than the engine holds sequences: :class:`SwapEngine` serves N logical slots over an engine of
P < N sequences, and the slots take the engine in turns.

The engines of this package hold every slot natively (each slot owns pages of the paged KV pool, spilled to the host
when the pool is short), so this adapter is for the case where that is not wanted: a long ``--slot-ctx`` whose KV only
fits a few times, with more clients than that connected.  The reference's counterpart is ``crates/serve/src/swap.rs``
(``SwapEngine``, ``ParkTable``, ``QUANTUM``); there the engine holds ONE sequence, here any P.

Rules.

* The engine thread asks :meth:`SwapEngine.turn` once a round which live slots run.  A slot that holds the engine keeps
  it for :data:`QUANTUM` tokens; after that it yields when another live slot waits, the one that waited longest next.
  With at most P live slots nobody ever yields.
* A slot that leaves the engine is parked: under ``park="states"`` its snapshot goes into the :class:`ParkTable`
  (a byte budget; states of idle slots -- their request finished -- leave first when a live one needs room), under
  ``park="ids"`` only its ids are kept and its next turn feeds them again.  A live state that finds no room is kept by
  its ids too: the request goes on, it pays a prompt pass at its next turn.
* A slot that comes back restores its parked state, and feeds whatever the state does not cover.
* Every call names a logical slot; the adapter never steps more than P of them in one call.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Set

from .engine import Engine, Saved

QUANTUM = 64          # tokens a slot runs before the next waiting slot's turn


class ParkTable:
    """Snapshots of the slots that hold no engine sequence, at most ``budget`` bytes of them."""

    def __init__(self, budget: int):
        self.budget = int(budget)
        self.held: Dict[int, Saved] = {}
        self.idle: Set[int] = set()
        self.evicted = 0
        self.refused = 0

    def bytes(self) -> int:
        return sum(s.n_bytes for s in self.held.values())

    def put(self, slot: int, saved: Saved, idle: bool) -> bool:
        """Keep ``saved`` for ``slot``.  Idle states leave (oldest first) to make room; a live state never leaves for
        another.  False when it does not fit."""
        self.take(slot)
        need = saved.n_bytes
        if need > self.budget:
            self.refused += 1
            return False
        while self.bytes() + need > self.budget:
            victim = next((s for s in self.held if s in self.idle), None)
            if victim is None:
                self.refused += 1
                return False
            self.take(victim)
            self.evicted += 1
        self.held[slot] = saved
        if idle:
            self.idle.add(slot)
        return True

    def take(self, slot: int) -> Optional[Saved]:
        self.idle.discard(slot)
        return self.held.pop(slot, None)

    def mark(self, slot: int, idle: bool) -> None:
        if slot in self.held:
            (self.idle.add if idle else self.idle.discard)(slot)


class SwapEngine(Engine):
    def __init__(self, inner: Engine, n_slots: int, park: str = "states", budget: int = 4 << 30, quantum: int = QUANTUM):
        if park not in ("states", "ids"):
            raise ValueError(f"park takes states or ids, got {park!r}")
        if n_slots < inner.n_slots:
            raise ValueError(f"{n_slots} slots over an engine of {inner.n_slots}: nothing to take turns for")
        self.inner = inner
        self.n_slots = n_slots
        self.n_engine = inner.n_slots
        self.park, self.quantum = park, quantum
        self.table = ParkTable(budget if park == "states" else 0)
        self.tokenizer, self.slot_ctx, self.n_vocab = inner.tokenizer, inner.slot_ctx, inner.n_vocab
        self.model_name = inner.model_name
        self.max_rows = getattr(inner, "max_rows", 8)
        self.device_sampling = getattr(inner, "device_sampling", False)
        self.ids: List[List[int]] = [[] for _ in range(n_slots)]      # what every logical slot's sequence holds
        self.where: List[Optional[int]] = [None] * n_slots            # logical -> engine slot
        self.owner: List[Optional[int]] = [None] * self.n_engine      # engine slot -> logical
        self.used = [0] * n_slots                                     # tokens since the slot took the engine
        self.since = [0] * n_slots                                    # the ticket a waiting slot drew when it started to wait
        self.last = [0] * n_slots                                     # the round the slot last ran in
        self.live: Set[int] = set()
        self.holders: List[int] = []
        self.round = self.tickets = 0
        self.parks = self.refeeds = self.restores = 0

    # ---- whose turn ---------------------------------------------------------------------------------------------
    def _ticket(self) -> int:
        self.tickets += 1
        return self.tickets

    def turn(self, live: Iterable[int]) -> Set[int]:
        """The live slots that run this round (at most as many as the engine holds sequences)."""
        self.round += 1
        now = list(dict.fromkeys(live))
        for s in now:
            if s not in self.live:
                self.since[s] = self._ticket()
        for s in self.live - set(now):
            self.table.mark(s, idle=True)
        self.live = set(now)
        holders = [s for s in self.holders if s in self.live]
        waiting = sorted((s for s in now if s not in holders), key=lambda s: (self.since[s], s))
        # waiting slots beyond the free sequences get in only when a holder yields: those past their quantum do, the
        # one that ran longest first, and queue behind the slots already waiting
        short = max(0, len(waiting) - (self.n_engine - len(holders)))
        spent = sorted((s for s in holders if self.used[s] >= self.quantum), key=lambda s: (-self.used[s], s))[:short]
        keep: List[int] = [s for s in holders if s not in spent]
        for s in spent:
            self.since[s] = self._ticket()
            waiting.append(s)
        while len(keep) < self.n_engine and waiting:
            s = waiting.pop(0)
            self.used[s] = 0
            keep.append(s)
        self.holders = keep
        for s in keep:
            self.last[s] = self.round
        return set(keep)

    # ---- moving states ------------------------------------------------------------------------------------------
    def _park(self, slot: int) -> None:
        p = self.where[slot]
        ids = self.ids[slot]
        if self.park == "states" and ids:
            saved = self.inner.snapshot(p, ids)
            if saved is not None:
                self.table.put(slot, saved, idle=slot not in self.live)
        self.inner.reset(p)
        self.where[slot], self.owner[p] = None, None
        self.parks += 1

    def _bring(self, slot: int, pinned: Sequence[int] = ()) -> int:
        """The engine slot of logical ``slot``, making room and putting its state back when it holds none."""
        p = self.where[slot]
        if p is not None:
            return p
        free = [q for q, o in enumerate(self.owner) if o is None]
        if free:
            p = free[0]
        else:
            victims = [o for o in self.owner if o is not None and o not in pinned and o != slot]
            if not victims:
                raise RuntimeError(f"slot {slot}: every engine sequence is pinned by this call")
            # idle slots first, then the one that ran longest ago
            victim = min(victims, key=lambda o: (o in self.live, self.last[o], o))
            p = self.where[victim]
            self._park(victim)
        self.where[slot], self.owner[p] = p, slot
        ids = self.ids[slot]
        have = 0
        saved = self.table.take(slot)
        if saved is not None and ids:
            n = 0
            while n < min(len(ids), len(saved.ids)) and saved.ids[n] == ids[n]:
                n += 1
            if n:
                have = self.inner.restore(p, saved, n)
                self.restores += 1
        if have < len(ids):
            self.inner.cut(p, have)
            self.inner.prefill(p, ids[have:], have)
            self.refeeds += 1
        return p

    # ---- the engine calls ---------------------------------------------------------------------------------------
    def prefill(self, slot, ids, start):
        p = self._bring(slot)
        self.inner.prefill(p, ids, start)
        self.ids[slot] = self.ids[slot][:start] + list(ids)

    def step(self, rows, want_logits=True, draft_slots=None, sampling=None):
        slots = list(dict.fromkeys(r[0] for r in rows))
        if len(slots) > self.n_engine:
            raise RuntimeError(f"a round of {len(slots)} slots over an engine of {self.n_engine}: ask turn() who runs")
        phys = {s: self._bring(s, slots) for s in slots}
        kw = {}
        if draft_slots is not None:
            kw["draft_slots"] = {phys[s] for s in draft_slots if s in phys}
        if sampling is not None:
            kw["sampling"] = sampling
        out = self.inner.step([(phys[s], tok, pos) for s, tok, pos in rows], want_logits=want_logits, **kw)
        for s, tok, pos in rows:
            self.ids[s] = self.ids[s][:pos] + [tok]
            self.used[s] += 1
            self.last[s] = self.round
        return out

    def cut(self, slot, n):
        self.ids[slot] = self.ids[slot][:n]
        if self.where[slot] is not None:
            self.inner.cut(self.where[slot], n)

    def reset(self, slot):
        self.ids[slot] = []
        self.table.take(slot)
        if self.where[slot] is not None:
            self.inner.reset(self.where[slot])

    def share_prefix(self, src, dst, n, have=0):
        # pages are shared between two sequences the engine holds; a parked donor has nothing to share
        if self.where[src] is None:
            return 0
        p = self._bring(dst, (src,))
        got = self.inner.share_prefix(self.where[src], p, n, have)
        if got > have:
            self.ids[dst] = self.ids[src][:got]
        return got

    def snapshot(self, slot, ids):
        if self.where[slot] is None:
            held = self.table.held.get(slot)
            if held is not None and tuple(held.ids[:len(ids)]) == tuple(ids) and len(held.ids) == len(ids):
                return held
        return self.inner.snapshot(self._bring(slot), ids)

    def restore(self, slot, saved, n):
        p = self._bring(slot)
        got = self.inner.restore(p, saved, n)
        self.ids[slot] = list(saved.ids[:got])
        return got

    def embed(self, ids):
        return self.inner.embed(ids)

    def props(self):
        out = dict(self.inner.props())
        out["turns"] = {"slots": self.n_slots, "engine_sequences": self.n_engine, "park": self.park, "quantum": self.quantum,
                        "parked_bytes": self.table.bytes(), "park_budget": self.table.budget, "parks": self.parks,
                        "restores": self.restores, "refeeds": self.refeeds, "evicted_idle_states": self.table.evicted,
                        "states_without_room": self.table.refused}
        return out

    def close(self):
        self.inner.close()

    def __getattr__(self, name):
        # anything else (the decode engine behind a GPU engine, residency reset, ...) is the inner engine's
        if name == "inner":
            raise AttributeError(name)
        return getattr(self.inner, name)
