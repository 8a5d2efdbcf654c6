"""Expert placement at run time: cold routed experts in pinned host RAM, the most-called
ones promoted into HBM slots on a side stream, cold hits served by the CPU leg.

Pieces (in the reference: ``crates/runtime/src/swaprule.rs`` rule,
``crates/gpu/src/host/{swap,lane}.rs`` machine, ``host/{mod,step,handoff}.rs`` host tier):

* :class:`ResidencyRule` -- pure host logic.  Heat of every expert is a decayed count of the
  routed ids seen on kept rows; every ``every`` rows the hottest off-card experts are paired
  with the coldest on-card ones and a pair is admitted when the newcomer leads by ``margin``
  and was called at least ``min_count`` times, at most ``cap`` pairs per boundary.  The
  default ``mid`` = every 4 rows, cap 24, margin 3, min_count 2, decay 0.9, one spare slot per
  layer (``swaprule.rs:63-77``).  Same history => same decisions.
* :class:`TieredExperts` -- per layer: all experts in pinned host memory (resident layouts,
  read in place by the C++ CPU leg), ``n_slots`` HBM slots plus one spare, and a device
  ``slot_map`` (expert id -> slot or -1) that the kernels read, so promotions never need a
  graph recapture.  A promotion copies the newcomer into the spare slot with
  ``cudaMemcpyAsync`` on a copy stream; it *lands* at the boundary ``delay`` rounds later
  whatever the copy's progress (the main stream waits on the copy's event), by rewriting
  two words of the slot map; the victim's slot becomes the new spare.
* :class:`HostTier` -- the pinned, device-mapped hand-off page and the C++ service thread.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..formats.resident import WT
from ..ops._lib import I, L, check, cuda, host, p, stream
from ..ops.decode import QWeight

PRESETS = {
    "off": None,
    "low": dict(every=8, cap=8, margin=4.0, min_count=3, decay=0.9),
    "mid": dict(every=4, cap=24, margin=3.0, min_count=2, decay=0.9),
    "high": dict(every=2, cap=48, margin=1.5, min_count=1, decay=0.8),
}


@dataclasses.dataclass
class Flip:
    layer: int
    newcomer: int
    victim: int


class ResidencyRule:
    def __init__(self, n_layer: int, n_expert: int, resident: Sequence[Sequence[int]], every: int = 4, cap: int = 24,
                 margin: float = 3.0, min_count: int = 2, decay: float = 0.9):
        self.n_layer, self.E = n_layer, n_expert
        self.every, self.cap, self.margin, self.min_count, self.decay = every, cap, margin, min_count, decay
        self.heat = [[0.0] * n_expert for _ in range(n_layer)]
        self.on_card = [set(r) for r in resident]
        self.rows = 0
        self.total_flips = 0

    def observe(self, layer: int, counts: Sequence[int]) -> None:
        """Add one boundary's routed-id counts of a layer (already summed over its kept rows)."""
        h = self.heat[layer]
        d = self.decay
        for e in range(self.E):
            h[e] = h[e] * d + counts[e]

    def kept(self, n_rows: int) -> bool:
        """Account kept rows; true when a decision boundary was crossed."""
        before = self.rows // self.every
        self.rows += n_rows
        return self.rows // self.every != before

    def decide(self) -> List[Flip]:
        flips: List[Flip] = []
        for layer in range(self.n_layer):
            h = self.heat[layer]
            on = self.on_card[layer]
            off = sorted((e for e in range(self.E) if e not in on), key=lambda e: (-h[e], e))
            cold = sorted(on, key=lambda e: (h[e], e))
            for new, old in zip(off, cold):
                if len(flips) >= self.cap:
                    break
                if h[new] < self.min_count or h[new] < h[old] + self.margin:
                    break
                flips.append(Flip(layer, new, old))
        for f in flips:
            self.on_card[f.layer].discard(f.victim)
            self.on_card[f.layer].add(f.newcomer)
        self.total_flips += len(flips)
        return flips


class HostTier:
    """The hand-off page (pinned + mapped into the device) and the C++ service thread."""

    def __init__(self, n_layer: int, hidden: int, inter: int, n_used: int, device, max_rows: int = 8):
        self.lib = host()
        self.lib.blh_host_tier_page_words.restype = ctypes.c_long
        self.lib.blh_host_tier_create.restype = ctypes.c_void_p
        words = int(self.lib.blh_host_tier_page_words(I(hidden), I(max_rows)))
        self.page = torch.zeros(words, dtype=torch.int32, pin_memory=True)
        self.max_rows = max_rows
        self.device = torch.device(device)
        # pinned memory from torch is mapped (cudaHostAllocDefault on UVA systems): its host
        # pointer is valid on the device
        self.page_dev_ptr = self.page.data_ptr()
        self.handle = ctypes.c_void_p(self.lib.blh_host_tier_create(I(n_layer), I(hidden), I(inter), I(n_used), I(max_rows),
                                                                    ctypes.c_void_p(self.page.data_ptr())))
        if not self.handle:
            raise RuntimeError("host tier refused the shape")
        self.seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.pending = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.cold_total = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.wait_ns = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.extra = torch.zeros(max_rows, hidden, dtype=torch.float32, device=self.device)
        self.started = False

    def set_layer(self, layer: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, gtype: str, dtype: str, E: int):
        self.lib.blh_host_tier_set_layer(self.handle, I(layer), p(gate), p(up), p(down), I(WT[gtype]), I(WT[dtype]), I(E))

    def start(self) -> None:
        if not self.started:
            self.lib.blh_host_tier_start(self.handle)
            self.started = True

    def stop(self) -> None:
        if self.started:
            self.lib.blh_host_tier_stop(self.handle)
            self.started = False

    def stats(self) -> Dict[str, float]:
        a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        self.lib.blh_host_tier_stats(self.handle, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return {"handoffs": a.value, "cold_slots_served": b.value, "host_busy_s": c.value / 1e9,
                "card_wait_s": float(self.wait_ns.item()) / 1e9, "cold_slots_routed": int(self.cold_total.item())}

    def handoff(self, ids, wts, slot_map, xq, xds, M: int, n_used: int, K: int, E: int, layer: int) -> None:
        check(cuda().bl_host_handoff(p(ids), p(wts), p(slot_map), p(xq), p(xds), I(M), I(n_used), I(K), I(E), I(layer),
                                     I(self.max_rows), ctypes.c_void_p(self.page_dev_ptr), p(self.seq), p(self.pending),
                                     p(self.cold_total), stream()), "bl_host_handoff")

    def wait(self, M: int, K: int, fault, layer: int) -> None:
        check(cuda().bl_host_wait(ctypes.c_void_p(self.page_dev_ptr), p(self.seq), p(self.pending), p(self.extra), I(M), I(K),
                                  I(self.max_rows), p(fault), I(layer), p(self.wait_ns), stream()), "bl_host_wait")

    def close(self) -> None:
        if self.handle:
            self.lib.blh_host_tier_destroy(self.handle)
            self.handle = None


class TieredExperts:
    """Expert stacks of every MoE layer split between pinned host RAM and HBM slots."""

    def __init__(self, spec, weights, n_slots: int, device, rule: Optional[str] = "mid", delay: int = 2,
                 keep_host: bool = True):
        """``keep_host=False``: the cold experts are not kept in RAM (a drive-backed arena serves them); promotion
        has no source then, so the residency rule is off."""
        self.spec = spec
        self.device = torch.device(device)
        self.keep_host = keep_host
        E = spec.n_expert
        self.n_slots = max(0, min(n_slots, E))
        self.layers = [il for il in range(spec.n_layer) if spec.layer_is_moe(il)]
        self.host: Dict[int, Dict[str, QWeight]] = {}
        self.card: Dict[int, Dict[str, QWeight]] = {}
        self.slot_map: Dict[int, torch.Tensor] = {}
        self.slot_of: Dict[int, Dict[int, int]] = {}
        self.spare: Dict[int, int] = {}
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.pending: List[Tuple[int, Flip, int, Optional[torch.cuda.Event]]] = []   # (lands_at_round, flip, slot, event)
        self.round = 0
        self.delay = delay
        self.bytes_promoted = 0
        for il in self.layers:
            b = f"blk.{il}."
            hq, cq = {}, {}
            for part in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                full = weights.q.pop(b + part + ".weight")
                if keep_host:
                    pinned = full.data.cpu().pin_memory() if self.device.type == "cuda" else full.data.cpu()
                    hq[part] = QWeight(pinned, full.qtype, full.k)
                slots = torch.zeros(self.n_slots + 1, *full.data.shape[1:], dtype=torch.uint8, device=self.device)
                if self.n_slots:
                    slots[:self.n_slots].copy_(full.data[:self.n_slots])
                cq[part] = QWeight(slots, full.qtype, full.k)
                weights.n_bytes -= full.n_bytes - slots.numel()
                del full
            self.host[il], self.card[il] = hq, cq
            sm = torch.full((E,), -1, dtype=torch.int32)
            sm[:self.n_slots] = torch.arange(self.n_slots, dtype=torch.int32)
            self.slot_map[il] = sm.to(self.device)
            self.slot_of[il] = {e: e for e in range(self.n_slots)}
            self.spare[il] = self.n_slots
        preset = PRESETS.get(rule or "off") if keep_host else None
        self.rule = ResidencyRule(spec.n_layer, E, [list(range(self.n_slots)) if il in self.host else [] for il in range(spec.n_layer)],
                                  **preset) if preset and self.n_slots else None
        self._heat_seen: Dict[int, torch.Tensor] = {}

    def card_bytes(self) -> int:
        return sum(q.data.numel() for c in self.card.values() for q in c.values())

    def slot_bytes(self) -> int:
        """Bytes of one resident slot in every routed layer (gate, up and down matrices; the types may differ by layer)."""
        return sum(int(q.data[0].numel()) for il in self.layers for q in self.card[il].values())

    def resize(self, n_slots: int, heat: Optional[torch.Tensor] = None) -> None:
        """Change the number of resident slots of every routed layer (between passes, no captured pass alive).
        Shrinking keeps the hottest residents by ``heat`` ([layer, expert] routed counts; slot order when absent) and
        hands the rest to the host leg; growing copies the hottest host experts in.  Flips in flight are dropped: their
        newcomers never became visible in the slot map."""
        E = self.spec.n_expert
        n_slots = max(0, min(n_slots, E))
        if not self.keep_host and n_slots > self.n_slots:
            raise ValueError("no RAM-resident experts to fill new slots from")
        self.pending = []
        for il in self.layers:
            res = dict(self.slot_of[il])                                   # expert -> slot
            h = heat[il].tolist() if heat is not None else None
            rank = (lambda e: (-h[e], e)) if h is not None else (lambda e: (res.get(e, E), e))
            keep = sorted(res, key=rank)[:n_slots]
            more = []
            if n_slots > len(keep):
                more = sorted((e for e in range(E) if e not in res), key=(lambda e: (-h[e], e)) if h is not None else (lambda e: e))
                more = more[:n_slots - len(keep)]
            new_card, order = {}, keep + more
            for part, old in self.card[il].items():
                slots = torch.zeros(n_slots + 1, *old.data.shape[1:], dtype=torch.uint8, device=self.device)
                for i, e in enumerate(keep):
                    slots[i].copy_(old.data[res[e]])
                for i, e in enumerate(more):
                    slots[len(keep) + i].copy_(self.host[il][part].data[e], non_blocking=True)
                new_card[part] = QWeight(slots, old.qtype, old.k)
            self.card[il] = new_card
            sm = torch.full((E,), -1, dtype=torch.int32)
            for i, e in enumerate(order):
                sm[e] = i
            self.slot_map[il].copy_(sm.to(self.device))
            self.slot_of[il] = {e: i for i, e in enumerate(order)}
            self.spare[il] = n_slots
            if self.rule is not None:
                self.rule.on_card[il] = set(order)
        self.n_slots = n_slots
        if self.rule is not None and n_slots == 0:
            self.rule = None

    def host_bytes(self) -> int:
        return sum(q.data.numel() for c in self.host.values() for q in c.values())

    def attach_host_tier(self, tier: HostTier) -> None:
        for il in self.layers:
            h = self.host[il]
            if not h:
                continue
            tier.set_layer(il, h["ffn_gate_exps"].data, h["ffn_up_exps"].data, h["ffn_down_exps"].data,
                           h["ffn_gate_exps"].qtype, h["ffn_down_exps"].qtype, self.spec.n_expert)

    # ---- boundary: called between passes, on the engine's stream ------------------------------
    def boundary(self, heat: torch.Tensor, kept_rows: int) -> int:
        """Land due flips, then (at a decision boundary) read the heat and start new copies."""
        self.round += 1
        landed = 0
        still = []
        for lands_at, flip, slot, ev in self.pending:
            if lands_at > self.round:
                still.append((lands_at, flip, slot, ev))
                continue
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)   # lands now, whatever the copy's progress
            sm = self.slot_map[flip.layer]
            old_slot = self.slot_of[flip.layer].pop(flip.victim)
            sm[flip.victim] = -1
            sm[flip.newcomer] = slot
            self.slot_of[flip.layer][flip.newcomer] = slot
            self.spare[flip.layer] = old_slot
            landed += 1
        self.pending = still
        if self.rule is None or not self.rule.kept(kept_rows):
            return landed
        counts = heat.cpu()
        for il in self.layers:
            prev = self._heat_seen.get(il)
            cur = counts[il]
            self.rule.observe(il, (cur - prev if prev is not None else cur).tolist())
            self._heat_seen[il] = cur.clone()
        busy_layers = {f.layer for _, f, _, _ in self.pending}
        for f in self.rule.decide():
            if f.layer in busy_layers:          # one spare per layer: one flip in flight per layer
                self.rule.on_card[f.layer].discard(f.newcomer)
                self.rule.on_card[f.layer].add(f.victim)
                continue
            busy_layers.add(f.layer)
            slot = self.spare[f.layer]
            ev = None
            if self.copy_stream is not None:
                self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(self.copy_stream):
                    for part in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                        self.card[f.layer][part].data[slot].copy_(self.host[f.layer][part].data[f.newcomer], non_blocking=True)
                        self.bytes_promoted += self.host[f.layer][part].data[f.newcomer].numel()
                    ev = torch.cuda.Event()
                    ev.record(self.copy_stream)
            else:
                for part in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                    self.card[f.layer][part].data[slot].copy_(self.host[f.layer][part].data[f.newcomer])
            self.pending.append((self.round + self.delay, f, slot, ev))
        return landed

    def reset(self) -> None:
        """Forget the heat (``POST /residency/reset``); the current map stays."""
        if self.rule is not None:
            self.rule.heat = [[0.0] * self.rule.E for _ in range(self.rule.n_layer)]
