"""Experts as the elastic tenant of the card: they are what the card gives up when a later allocation does not fit
and what it takes back when there is room.

* :func:`with_room` runs an allocating operation; on an out-of-memory refusal it asks the body for the shortfall
  (``give_back``), then runs the operation once more.
* :func:`settle_to_margin` is the move a load makes after its warm-up, once every buffer serving uses exists: give
  back what the card holds past its margin, or fill what it has free.
* every give-back and fill is counted (:class:`ElasticStats`) so a binary can print it as a record line; a steady
  state after warm-up keeps the give-back count at zero.

A body offers two moves (``give_back(n_bytes) -> bytes freed``, ``fill(n_bytes) -> bytes taken``) and a size
(``unit_bytes``, the bytes one step of either move is worth).  :class:`TieredBody` is the body of a
:class:`bloomery_b200.runtime.tiered.TieredEngine`: one step is one resident expert slot in every routed layer
(``TieredExperts.resize``); the slots that go are the coldest by the routing heat, their experts fall to the host leg.
Nothing here names a model.  (The reference: ``crates/gpu/src/room/elastic.rs`` -- ``ElasticBody``, ``with_room``,
``settle_to_margin``.)
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional, TypeVar

T = TypeVar("T")


@dataclasses.dataclass
class ElasticStats:
    give_backs: int = 0
    bytes_given: int = 0
    fills: int = 0
    bytes_filled: int = 0
    retries: int = 0

    def record(self) -> dict:
        return dataclasses.asdict(self)


class NoRoom(MemoryError):
    """The operation was refused twice: the body had nothing (more) to give."""


def _is_oom(exc: BaseException) -> bool:
    import torch
    oom = getattr(torch.cuda, "OutOfMemoryError", ())
    return isinstance(exc, (MemoryError,) + ((oom,) if oom else ())) or "out of memory" in str(exc).lower()


def with_room(op: Callable[[], T], body, need_bytes: int, stats: Optional[ElasticStats] = None) -> T:
    """Run ``op``; when it is refused for memory, have ``body`` give back ``need_bytes`` (rounded up to its unit) and run
    it once more.  A second refusal, or a body that frees nothing, raises :class:`NoRoom`."""
    try:
        return op()
    except BaseException as exc:                 # noqa: BLE001 - only memory refusals are handled, the rest re-raised
        if not _is_oom(exc):
            raise
        freed = body.give_back(max(need_bytes, body.unit_bytes))
        if stats is not None:
            stats.retries += 1
            if freed:
                stats.give_backs += 1
                stats.bytes_given += freed
        if not freed:
            raise NoRoom(f"the card has no room for {need_bytes} bytes and the experts have nothing to give back") from exc
        try:
            return op()
        except BaseException as exc2:            # noqa: BLE001
            if _is_oom(exc2):
                raise NoRoom(f"no room for {need_bytes} bytes even after {freed} bytes of experts went to the host") from exc2
            raise


def settle_to_margin(body, free_bytes: int, margin_bytes: int, stats: Optional[ElasticStats] = None) -> int:
    """With ``free_bytes`` free on the card and ``margin_bytes`` to be left free: give back the shortfall, or fill what
    is free past the margin in whole units.  Returns the signed change of the experts' bytes on the card."""
    if free_bytes < margin_bytes:
        freed = body.give_back(margin_bytes - free_bytes)
        if stats is not None and freed:
            stats.give_backs += 1
            stats.bytes_given += freed
        return -freed
    spare = free_bytes - margin_bytes
    if spare >= body.unit_bytes:
        taken = body.fill(spare)
        if stats is not None and taken:
            stats.fills += 1
            stats.bytes_filled += taken
        return taken
    return 0


class TieredBody:
    """The experts of a tiered engine as an elastic body: a unit is one resident slot in every routed layer."""

    def __init__(self, engine):
        self.engine = engine

    @property
    def unit_bytes(self) -> int:
        return self.engine.tiered.slot_bytes()

    def _resize(self, n_slots: int) -> int:
        e = self.engine
        t = e.tiered
        before = t.card_bytes()
        if n_slots == t.n_slots:
            return 0
        heat = e.heat.cpu() if hasattr(e, "heat") else None
        t.resize(n_slots, heat)
        e.graphs.clear()                      # the captured passes hold the old slot arrays' addresses
        return abs(before - t.card_bytes())

    def give_back(self, n_bytes: int) -> int:
        t = self.engine.tiered
        steps = -(-n_bytes // self.unit_bytes)
        return self._resize(max(0, t.n_slots - steps))

    def fill(self, n_bytes: int) -> int:
        t = self.engine.tiered
        if not t.keep_host:
            return 0                           # no RAM-resident source to fill from
        steps = n_bytes // self.unit_bytes
        return self._resize(min(t.spec.n_expert, t.n_slots + steps))
