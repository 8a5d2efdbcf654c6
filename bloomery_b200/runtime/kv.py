"""Paged KV pool: fixed-size pages of 64 positions, per-slot block tables, prefix sharing.

The reference reserves each slot's whole context as a virtual range and backs pages
lazily (``crates/gpu/src/room/mod.rs:1-52``, ``room/kv.rs:1-8``) and shares a prefix
between slots copy-on-write (``Room::share``, ``room/mod.rs:22-31``).  Here the same
capabilities sit on a block table that the kernels read from device memory: pages are
handed out on demand, a shared prefix is a run of page ids present in two tables with
a reference count, and a slot that appends into a shared page first takes its own copy.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

PAGE = 64


class OutOfPages(RuntimeError):
    pass


def snap_ready(snap) -> None:
    """Wait until a snapshot's device-to-host copies have landed (call before any host-side read of its tensors)."""
    ev = snap.pop("_ev", None) if isinstance(snap, dict) else None
    if ev is not None:
        ev.synchronize()


class KvPool:
    def __init__(self, n_layer: int, n_kv: int, head_dim: int, n_pages: int, n_slots: int, max_pages_per_slot: int,
                 device, dtype=torch.float16, v_dim: Optional[int] = None):
        self.n_layer, self.n_kv, self.head_dim = n_layer, n_kv, head_dim
        self.n_pages, self.n_slots, self.max_pages = n_pages, n_slots, max_pages_per_slot
        self.device = torch.device(device)
        # [layer][page][kv head][position in page][dim]
        self.k = torch.zeros(n_layer, n_pages, n_kv, PAGE, head_dim, dtype=dtype, device=self.device)
        # a latent cache (MLA) keeps one row per position that serves as key and value: v_dim = 0
        self.v = torch.zeros(n_layer, n_pages, n_kv, PAGE, head_dim if v_dim is None else v_dim, dtype=dtype,
                             device=self.device)
        self.table_host = torch.full((n_slots, max_pages_per_slot), -1, dtype=torch.int32,
                                     pin_memory=self.device.type == "cuda")
        self.table = torch.full((n_slots, max_pages_per_slot), -1, dtype=torch.int32, device=self.device)
        self.free: List[int] = list(range(n_pages - 1, -1, -1))
        self.refs: List[int] = [0] * n_pages
        self.pages: List[List[int]] = [[] for _ in range(n_slots)]
        self.dirty = False
        # host spill: when the pool runs dry, the least recently used slot that the current pass does not touch
        # is copied to pinned host memory and its pages are reused; it comes back the next time it is needed
        # (the reference backs such pages with host memory in place: crates/gpu/src/room/mod.rs ``Backing::Spill``)
        self.spilled: Dict[int, tuple] = {}
        self.protect: set = set()
        self.stamp = [0] * n_slots
        self.clock = 0
        self.n_spills = 0
        self.n_unspills = 0
        self.allow_spill = True
        self.floor_positions = 0        # a pool that holds fewer positions than this never spills (BLOOMERY_KV_FLOOR)

    @property
    def bytes(self) -> int:
        return (self.k.numel() + self.v.numel()) * self.k.element_size()

    def free_pages(self) -> int:
        return len(self.free)

    def touch(self, slot: int) -> None:
        self.clock += 1
        self.stamp[slot] = self.clock

    def _spill_one(self) -> bool:
        victims = [s for s in range(self.n_slots) if self.pages[s] and s not in self.protect
                   and all(self.refs[p] == 1 for p in self.pages[s])]
        if not victims or not self.allow_spill or self.n_pages * PAGE < self.floor_positions:
            return False
        s = min(victims, key=lambda v: self.stamp[v])
        n = len(self.pages[s]) * PAGE
        # stream order keeps this safe: the copy out is enqueued before anything that rewrites the pages
        snap = self.snapshot(s, n)
        self.release(s)
        self.spilled[s] = (snap, n)
        self.n_spills += 1
        return True

    def _take(self) -> int:
        if not self.free and not self._spill_one():
            raise OutOfPages("KV pool exhausted")
        pg = self.free.pop()
        self.refs[pg] = 1
        return pg

    def _drop(self, pg: int) -> None:
        self.refs[pg] -= 1
        if self.refs[pg] == 0:
            self.free.append(pg)

    def ensure(self, slot: int, n_positions: int) -> None:
        """Back positions [0, n_positions) of a slot with pages.  The slot itself is never the spill victim of
        its own request: when only its pages could be taken, the pool is out of pages."""
        need = (n_positions + PAGE - 1) // PAGE
        if need > self.max_pages:
            raise OutOfPages(f"slot {slot}: {n_positions} positions exceed the slot context")
        mine = slot not in self.protect
        self.protect.add(slot)
        try:
            if slot in self.spilled:
                snap, n = self.spilled.pop(slot)
                self.restore(slot, snap, n)
                self.n_unspills += 1
            self.touch(slot)
            pl = self.pages[slot]
            while len(pl) < need:
                pg = self._take()
                self.table_host[slot, len(pl)] = pg
                pl.append(pg)
                self.dirty = True
        finally:
            if mine:
                self.protect.discard(slot)

    def own(self, slot: int, position: int) -> None:
        """Copy-on-write: make the page holding ``position`` private before it is written."""
        i = position // PAGE
        pl = self.pages[slot]
        if i < len(pl) and self.refs[pl[i]] > 1:
            mine = slot not in self.protect
            self.protect.add(slot)
            try:
                new = self._take()
            finally:
                if mine:
                    self.protect.discard(slot)
            self.k[:, new].copy_(self.k[:, pl[i]])
            self.v[:, new].copy_(self.v[:, pl[i]])
            self._drop(pl[i])
            pl[i] = new
            self.table_host[slot, i] = new
            self.dirty = True

    def truncate(self, slot: int, n_positions: int) -> None:
        """Keep positions [0, n_positions); later pages go back to the pool (``cut``)."""
        keep = (n_positions + PAGE - 1) // PAGE
        if slot in self.spilled:
            snap, n = self.spilled[slot]
            if keep == 0:
                del self.spilled[slot]
            else:
                self.spilled[slot] = (snap, min(n, keep * PAGE))
            return
        pl = self.pages[slot]
        while len(pl) > keep:
            self._drop(pl.pop())
            self.table_host[slot, len(pl)] = -1
            self.dirty = True

    def release(self, slot: int) -> None:
        self.truncate(slot, 0)

    def share_prefix(self, src: int, dst: int, n_positions: int, have: int = 0) -> int:
        """Map the whole pages of ``src`` covering [0, n_positions) into ``dst``; returns positions shared.
        Only whole pages can be mapped, so the result is rounded down to a page; when that is no more than the
        ``have`` positions ``dst`` already holds of the same prefix, ``dst`` is left untouched and 0 is returned."""
        if (n_positions // PAGE) * PAGE <= have:
            return 0
        if src in self.spilled:
            self.ensure(src, 1)              # bring the source back before its pages are mapped twice
        full = min(n_positions // PAGE, len(self.pages[src]))
        if full * PAGE <= have:
            return 0
        self.release(dst)
        self.spilled.pop(dst, None)
        for i in range(full):
            pg = self.pages[src][i]
            self.refs[pg] += 1
            self.pages[dst].append(pg)
            self.table_host[dst, i] = pg
        self.dirty = True
        return full * PAGE

    def sync_table(self) -> None:
        """Push the host table to the device if it changed (small copy, outside any capture)."""
        if self.dirty:
            if self.device.type == "cuda":
                # snapshot first: the host keeps editing table_host while the copy is in flight
                snap = torch.empty_like(self.table_host, pin_memory=True).copy_(self.table_host)
                self.table.copy_(snap, non_blocking=True)
            else:
                self.table.copy_(self.table_host)
            self.dirty = False

    # snapshots for the host prompt cache -------------------------------------------------
    def snapshot(self, slot: int, n_positions: int, stream: Optional[torch.cuda.Stream] = None) -> Dict[str, torch.Tensor]:
        """Copy a slot's first ``n_positions`` K/V rows to pinned host memory."""
        n_pg = (n_positions + PAGE - 1) // PAGE
        idx = torch.tensor(self.pages[slot][:n_pg], dtype=torch.long, device=self.device)
        pin = self.device.type == "cuda"
        k = torch.empty((self.n_layer, n_pg, self.n_kv, PAGE, self.head_dim), dtype=self.k.dtype, pin_memory=pin)
        v = torch.empty((self.n_layer, n_pg, self.n_kv, PAGE, self.v.shape[-1]), dtype=self.v.dtype, pin_memory=pin)
        k.copy_(self.k.index_select(1, idx), non_blocking=True)
        v.copy_(self.v.index_select(1, idx), non_blocking=True)
        snap = {"k": k, "v": v, "n": torch.tensor(n_positions)}
        if pin:
            # the two copies run behind the caller on the stream: anyone who reads the host bytes waits on this first
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            snap["_ev"] = ev
        return snap

    def restore(self, slot: int, snap: Dict[str, torch.Tensor], n_positions: int) -> None:
        n_positions = min(n_positions, int(snap["n"]))
        if (n_positions + PAGE - 1) // PAGE < snap["k"].shape[1]:
            snap_ready(snap)                 # a partial restore slices on the host: the bytes must have landed
        self.spilled.pop(slot, None)
        self.release(slot)
        self.ensure(slot, n_positions)
        n_pg = (n_positions + PAGE - 1) // PAGE
        idx = torch.tensor(self.pages[slot][:n_pg], dtype=torch.long, device=self.device)
        self.k.index_copy_(1, idx, snap["k"][:, :n_pg].to(self.device, non_blocking=True))
        self.v.index_copy_(1, idx, snap["v"][:, :n_pg].to(self.device, non_blocking=True))
