"""Decode engine for models whose routed experts do not all fit in HBM: a budgeted number of
experts per layer stay resident in slots, the rest live in pinned host RAM; a routed slot
whose expert is not resident is served by the CPU leg through the in-graph hand-off, and the
residency rule keeps promoting the most-called experts (``runtime/residency.py``).

Per MoE layer the chain becomes
  router | route | hand-off (go) | gate·up of resident slots | wait | down + combine (+ host rows)
so the card computes its resident experts while the CPU computes the cold ones (the
reference's ``router -> handoff -> go -> [card experts] -> wait -> add``,
``crates/gpu/src/host/mod.rs:12-27``).  ``--cpu-moe`` is this engine with zero resident slots.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import decode as K
from .engine import DecodeEngine
from ..ops.decode import QWeight
from .residency import HostTier, TieredExperts


class TieredEngine(DecodeEngine):
    def __init__(self, weights, resident_per_layer: int, residency: Optional[str] = "mid", nvme=None, **kw):
        """``nvme``: a :class:`bloomery_b200.runtime.nvtier.NvmeTier` over a side file of this model's experts; the
        host leg then reads cold experts from its arena (paged from the drive) instead of RAM-resident stacks."""
        spec = weights.spec
        self.nvme = nvme
        self.tiered = TieredExperts(spec, weights, resident_per_layer, weights.device, rule=residency,
                                    keep_host=nvme is None)
        super().__init__(weights, **kw)
        self.tier = HostTier(spec.n_layer, spec.hidden, spec.moe_inter, spec.n_used, self.device)
        self.tiered.attach_host_tier(self.tier)
        if nvme is not None:
            nvme.attach(self.tier)
            self.gemm_threshold = 0          # no RAM-resident stacks to stream from: prompts take the pass path
        self.tier.start()

    def _moe(self, il: int, M: int, x: torch.Tensor) -> int:
        s, w, t = self.spec, self.w, self.tiered
        b = f"blk.{il}."
        sm = t.slot_map[il]
        card = t.card[il]
        ids, wts = self.r_ids_all[il], self.r_wts_all[il]
        # the routing launch's last block writes ids / weights / heat (completion ticket), so no routing launch follows
        K.router(x, w.f[b + "ffn_norm.weight"], s.rms_eps, w.q[b + "ffn_gate_inp.weight"], M, self.r_logits,
                 self.xq, self.xds, None, self.fault, il, rule=self._rule(il), ids=ids, wts=wts, heat=self.heat[il],
                 ticket=self.tickets[8 * max(1, s.n_kv):])
        self.tier.handoff(ids, wts, sm, self.xq, self.xds, M, s.n_used, s.hidden, s.n_expert, il)
        staged = card["ffn_gate_exps"].data.shape[0] > 0 and card["ffn_gate_exps"].qtype == card["ffn_up_exps"].qtype and \
            K.moe_fits_stage(card["ffn_gate_exps"], card["ffn_down_exps"], s.n_used)
        if staged:
            K.gate_up_staged(self.xq, self.xds, ids, sm, card["ffn_gate_exps"], card["ffn_up_exps"], s.n_expert, s.n_used, M,
                             self.actq, self.actds, None, self.fault, il, down=card["ffn_down_exps"])
        else:
            K.gate_up_sel(self.xq, self.xds, ids, sm, card["ffn_gate_exps"], card["ffn_up_exps"], s.n_expert,
                          s.n_used, M, self.actq, self.actds, None, self.fault, il)
        self.tier.wait(M, s.hidden, self.fault, il)
        (K.down_staged if staged else K.down_combine)(self.actq, self.actds, ids, wts, sm, card["ffn_down_exps"], s.n_expert,
                                                      s.n_used, M, x, self.tier.extra, x, self.fault, il)
        return 5

    def _new_gemm_prefill(self):
        """Prompts take the GEMM path with the layer's whole expert stacks streamed from pinned host memory into a
        two-half card ring on the copy stream, one layer ahead of the compute (the reference's prompt-time expert
        stream: ``crates/gpu/src/host/xstream.rs``; there only the hottest host experts move, here the whole layer,
        which the GEMM then reads as one stack)."""
        from .prefill import GemmPrefill
        pre = GemmPrefill(self, ubatch=self.ubatch)
        pre.expert_source = ExpertStreamer(self.tiered, self.device).get
        return pre

    def set_prompt_costs(self, costs) -> int:
        """Derive ``gemm_threshold`` (the prompt width from which the layer's stacks are streamed to the card instead of
        the rows taking the pass path with the host leg) from priced constants: the least width at which the split rule
        of ``runtime/xsplit.py`` moves any host expert to the card.  Returns the threshold."""
        from .xsplit import stream_gate
        s = self.spec
        n_host = max(1, s.n_expert - self.tiered.n_slots)
        gate = stream_gate(costs, n_host)
        if self.nvme is None:                # experts on a drive have no pinned stacks to stream from
            self.gemm_threshold = max(2, gate)
        return gate

    def _after_pass(self, n_rows: int) -> None:
        self.tiered.boundary(self.heat, n_rows)

    def memory_report(self):
        r = super().memory_report()
        r.update({"experts_card": self.tiered.card_bytes(), "experts_host": self.tiered.host_bytes()})
        return r

    def stats(self):
        out = self.tier.stats()
        out["flips"] = self.tiered.rule.total_flips if self.tiered.rule else 0
        out["bytes_promoted"] = self.tiered.bytes_promoted
        if self.nvme is not None:
            out["nvme"] = self.nvme.stats()
        return out

    def close(self) -> None:
        self.tier.stop()
        self.tier.close()


class ExpertStreamer:
    """Double-buffered host -> card copies of whole expert stacks, layer by layer."""

    PARTS = ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")

    def __init__(self, tiered: TieredExperts, device):
        self.t = tiered
        self.device = device
        self.copy = torch.cuda.Stream(device=device)
        size = {p: max(tiered.host[il][p].data.numel() for il in tiered.layers) for p in self.PARTS}
        self.halves = [{p: torch.empty(size[p], dtype=torch.uint8, device=device) for p in self.PARTS} for _ in range(2)]
        self.ready = {}            # layer -> (half index, event)
        self.bytes = 0

    def _issue(self, il: int, half: int) -> None:
        cur = torch.cuda.current_stream(self.device)
        gate = torch.cuda.Event()
        gate.record(cur)                            # everything that read this half before is enqueued before here
        self.copy.wait_event(gate)
        with torch.cuda.stream(self.copy):
            for p_ in self.PARTS:
                src = self.t.host[il][p_].data
                self.halves[half][p_][:src.numel()].copy_(src.reshape(-1), non_blocking=True)
                self.bytes += src.numel()
            ev = torch.cuda.Event()
            ev.record(self.copy)
        self.ready[il] = (half, ev)

    def get(self, il: int):
        layers = self.t.layers
        k = layers.index(il)
        if il not in self.ready:
            self._issue(il, k % 2)
        half, ev = self.ready.pop(il)
        torch.cuda.current_stream(self.device).wait_event(ev)
        nxt = layers[(k + 1) % len(layers)]          # the next layer (or the first one of the next micro-batch)
        if nxt not in self.ready and len(layers) > 1:
            self._issue(nxt, (half + 1) % 2)
        out = []
        for p_ in self.PARTS:
            h = self.t.host[il][p_]
            out.append(QWeight(self.halves[half][p_][:h.data.numel()].view(h.data.shape), h.qtype, h.k))
        return out
