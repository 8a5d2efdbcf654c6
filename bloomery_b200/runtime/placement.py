"""Pure placement planner: from a tensor inventory and a budget per card to where every tensor
lives, how many routed experts per layer stay on the card, how much context fits, and what each
tensor-parallel rank holds.  No device is touched; the server prints the result as its ``plan`` /
``need`` lines and builds the engine from it.

The reference's planner works the same way (``crates/placement/src/placement.rs:1-36``: per-tensor
device / format / bytes, card budgets and margins, the expert rule ``n_l`` per layer, tier cards,
the TP rank plan, context fitting, the need record).

Rules followed here:
  * the trunk (everything but routed experts) always lives on the card(s); a trunk that does not
    fit is a refusal, never a silent spill;
  * with experts on the host, every MoE layer keeps the same number ``n_l`` of resident expert
    slots (a multiple of 4, plus one spare slot for promotions), the largest that fits after
    trunk, KV for the asked context, work buffers and the margin;
  * context: an asked context is never cut (refusal names the largest that fits); an unasked one
    is the trained limit or the largest multiple of 1,024 that fits, at least 4,096;
  * tensor parallel: attention heads and routed experts divide over the ranks, norms / router /
    embedding / head are replicated; KV divides with the KV heads (never below one head per rank).
"""
from __future__ import annotations

import dataclasses
import re
from typing import Dict, List, Optional, Sequence, Tuple

WORK_BYTES = 2 << 30          # activations, split-K scratch, graphs, allocator slack per card
EXPERT_RE = re.compile(r"blk\.(\d+)\.ffn_(gate|up|down)_exps\.weight$")


class NoFit(ValueError):
    """The ask does not fit the budget; ``largest_ctx`` is what would."""

    def __init__(self, msg: str, largest_ctx: int = 0):
        super().__init__(msg)
        self.largest_ctx = largest_ctx


@dataclasses.dataclass
class TensorPlace:
    name: str
    n_bytes: int
    where: str                 # "card" (every card of the plan, sharded or replicated per `split`), "host", "card+host"
    split: str = "whole"       # whole | heads | experts | replicated


@dataclasses.dataclass
class Plan:
    world: int
    places: List[TensorPlace]
    trunk_bytes: int                    # per card
    expert_bytes_per_layer: int         # all routed experts of one MoE layer (whole model)
    n_moe_layers: int
    n_expert: int
    resident_per_layer: int             # expert slots on the card per MoE layer (== n_expert/world when all fit)
    spare_slots: int
    kv_bytes: int                       # per card
    slot_ctx: int
    n_slots: int
    card_bytes: int                     # per card, everything
    host_bytes: int
    budget: int

    @property
    def ctx_total(self) -> int:
        return self.slot_ctx * self.n_slots

    def need(self) -> Dict[str, object]:
        return {"card_bytes": self.card_bytes, "host_bytes": self.host_bytes, "budget": self.budget,
                "fits": self.card_bytes <= self.budget}

    def word(self) -> str:
        base = "a" if self.world == 1 else f"tp{self.world}"
        if self.host_bytes:
            base += f"+host[{self.resident_per_layer}/{self.n_expert}]"
        return base


def _classify(name: str) -> str:
    if EXPERT_RE.search(name):
        return "experts"
    if re.search(r"attn_(q|k|v|output|q_b|k_b|v_b)\.weight$", name):
        return "heads"
    return "replicated"


def plan(inventory: Sequence[Tuple[str, int]], *, n_layer: int, n_expert: int, first_dense: int, kv_bytes_per_token: int,
         n_kv_heads: int, ctx_train: int, budget: int, margin: int = 1 << 30, world: int = 1, ctx_ask: int = 0,
         n_slots: int = 1, host_experts: str = "none", n_host_layers: int = 0, work_bytes: int = WORK_BYTES) -> Plan:
    """``inventory`` = (tensor name, bytes as resident).  ``host_experts``: none | all | fit | first (first
    ``n_host_layers`` layers' experts on the host, expressed as an equal number of slots per layer)."""
    if world < 1 or n_slots < 1:
        raise ValueError("at least one card and one slot")
    trunk = experts = 0
    places: List[TensorPlace] = []
    for name, nb in inventory:
        kind = _classify(name)
        if kind == "experts":
            experts += nb
        elif kind == "heads":
            trunk += (nb + world - 1) // world
        else:
            trunk += nb
        places.append(TensorPlace(name, nb, "card", kind if world > 1 or kind == "experts" else "whole"))
    n_moe = max(0, n_layer - first_dense) if n_expert else 0
    per_layer = experts // n_moe if n_moe else 0
    per_expert_layer = per_layer // n_expert if n_expert else 0
    kv_share = max(1, min(world, n_kv_heads)) if n_kv_heads else world
    kv_tok = (kv_bytes_per_token + kv_share - 1) // kv_share
    room = budget - margin - work_bytes - trunk
    if room < 0:
        raise NoFit(f"the trunk of {trunk >> 20} MiB per card does not fit {budget >> 20} MiB "
                    f"(margin {margin >> 20} MiB, work {work_bytes >> 20} MiB); more cards divide the attention heads")
    all_experts_card = (experts + world - 1) // world

    def ctx_that_fits(after_experts: int) -> int:
        return max(0, after_experts) // max(1, kv_tok)

    if host_experts == "none":
        resident, spare, experts_card = (n_expert // world if n_expert else 0), 0, all_experts_card
    elif host_experts == "all":
        resident, spare, experts_card = 0, 0, 0
    elif host_experts == "first":
        resident = n_expert * max(0, n_moe - min(n_moe, n_host_layers)) // max(1, n_moe) // 4 * 4
        spare = 1 if 0 < resident < n_expert else 0
        experts_card = (resident + spare) * per_expert_layer * n_moe
    elif host_experts == "fit":
        want_ctx = (ctx_ask or 4096 * n_slots)
        left = room - want_ctx * kv_tok
        per_slot_all_layers = per_expert_layer * n_moe
        fit_slots = max(0, left) // max(1, per_slot_all_layers)
        if fit_slots >= n_expert // world + 0 and n_expert:
            resident, spare = n_expert // world, 0
        else:
            resident = max(0, (fit_slots - 1)) // 4 * 4
            spare = 1 if resident > 0 else 0
        experts_card = (resident + spare) * per_expert_layer * n_moe if resident < n_expert // max(1, world) else all_experts_card
    else:
        raise ValueError(f"host_experts {host_experts!r}")
    fit_tokens = ctx_that_fits(room - experts_card)
    if experts_card > room:
        raise NoFit(f"routed experts of {experts_card >> 20} MiB per card do not fit beside a trunk of {trunk >> 20} MiB in "
                    f"{budget >> 20} MiB; keep experts on the host (--cpu-moe, -fit on) or add cards")
    if ctx_ask:
        total = ctx_ask
        if total > fit_tokens:
            raise NoFit(f"a context of {ctx_ask} does not fit; the largest that fits is {fit_tokens // 1024 * 1024}",
                        largest_ctx=fit_tokens // 1024 * 1024)
    else:
        total = min(ctx_train * n_slots, fit_tokens // 1024 * 1024)
        if total < 4096:
            raise NoFit("not even a context of 4,096 fits beside the weights", largest_ctx=fit_tokens // 1024 * 1024)
    slot_ctx = min(ctx_train, total // n_slots) // 64 * 64
    kv_bytes = slot_ctx * n_slots * kv_tok
    host_bytes = 0
    if n_expert and resident < n_expert // max(1, world):
        host_bytes = experts                      # the host keeps every routed expert; the card holds copies of the resident ones
        for p in places:
            if p.split == "experts":
                p.where = "card+host" if resident else "host"
    return Plan(world=world, places=places, trunk_bytes=trunk, expert_bytes_per_layer=per_layer, n_moe_layers=n_moe,
                n_expert=n_expert, resident_per_layer=resident, spare_slots=spare, kv_bytes=kv_bytes, slot_ctx=slot_ctx,
                n_slots=n_slots, card_bytes=trunk + experts_card + kv_bytes + work_bytes, host_bytes=host_bytes, budget=budget)


def rank_inventory(inventory: Sequence[Tuple[str, int]], world: int, rank: int) -> List[Tuple[str, int]]:
    """What one tensor-parallel rank holds (bytes): head-split and expert-split tensors divide, the rest is whole."""
    out = []
    for name, nb in inventory:
        kind = _classify(name)
        out.append((name, nb // world if kind in ("heads", "experts") else nb))
    return out
