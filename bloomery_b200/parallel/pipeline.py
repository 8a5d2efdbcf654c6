"""Pipeline (stage) axis: the model as a list of stages, each a contiguous layer range with its own GPU,
weights, KV cache and captured graphs; the boundary between two stages is the hidden rows of the pass.

Used for capacity (a model that does not fit one card), not speed: a pass walks the stages in order.
The contract is the reference's (``crates/gpu/src/model.rs`` ``Stage`` / ``load_blocks`` :740, design
decision "two stages = one stage, bit for bit"): the same kernels run on the same rows, so picks and
logits equal the one-stage engine's exactly.  Here the boundary crosses with a device-to-device copy
over NVLink ordered by events (the reference moves it through the host).
"""
from __future__ import annotations

import re
from typing import Iterator, List, Optional, Sequence, Tuple

import torch

from ..models.spec import ModelSpec
from ..models.weights import TensorItem, Weights
from ..runtime.engine import MAX_ROWS, DecodeEngine

_BLK = re.compile(r"blk\.(\d+)\.")


def stage_items(items: Iterator[TensorItem], spec: ModelSpec, lo: int, hi: int, first: bool, last: bool) -> Iterator[TensorItem]:
    """The tensors one stage needs: its layers, the embedding on the first stage, norm + head (and a tied
    embedding, and the draft layers) on the last."""
    for it in items:
        name = it[0]
        m = _BLK.match(name)
        if m:
            il = int(m.group(1))
            if lo <= il < hi or (last and il >= spec.n_layer):
                yield it
        elif name.startswith("token_embd"):
            if first or last:
                yield it
        elif last:
            yield it


def split_layers(n_layer: int, n_stages: int, shares: Optional[Sequence[float]] = None) -> List[Tuple[int, int]]:
    """Contiguous layer ranges, by equal count or by the given shares (``-ts`` style)."""
    shares = list(shares) if shares else [1.0] * n_stages
    tot = sum(shares)
    cuts, acc = [0], 0.0
    for s in shares[:-1]:
        acc += s
        cuts.append(min(n_layer, max(cuts[-1] + 1, round(n_layer * acc / tot))))
    cuts.append(n_layer)
    return [(cuts[i], cuts[i + 1]) for i in range(n_stages)]


class _KvAll:
    """Slot operations applied to every stage's KV pool."""

    def __init__(self, stages):
        self.stages = stages

    def share_prefix(self, src, dst, n, have=0):
        return min(st.kv.share_prefix(src, dst, n, have) for st in self.stages)

    def sync_table(self):
        for st in self.stages:
            with torch.cuda.device(st.device):
                st.kv.sync_table()

    def snapshot(self, slot, n):
        from ..runtime.kv import snap_ready
        snaps = [st.kv.snapshot(slot, n) for st in self.stages]
        for sn in snaps:
            snap_ready(sn)                   # the bytes are read on the host right below
        return {"stages": snaps, "k": torch.cat([s["k"].reshape(-1).view(torch.uint8).cpu() for s in snaps])}

    def restore(self, slot, saved, n):
        for st, sn in zip(self.stages, saved["stages"]):
            st.kv.restore(slot, sn, n)

    def ensure(self, slot, n):
        for st in self.stages:
            st.kv.ensure(slot, n)


class PipelineEngine:
    def __init__(self, spec: ModelSpec, items_of_stage, devices: Sequence, ranges: Optional[List[Tuple[int, int]]] = None,
                 **engine_kw):
        """``items_of_stage(lo, hi, first, last)`` yields that stage's tensors (e.g. ``stage_items`` over a file)."""
        n = len(devices)
        self.spec = spec
        self.ranges = ranges or split_layers(spec.n_layer, n)
        self.stages: List[DecodeEngine] = []
        for i, ((lo, hi), dev) in enumerate(zip(self.ranges, devices)):
            first, last = i == 0, i == n - 1
            with torch.cuda.device(dev):
                w = Weights.from_items(spec, items_of_stage(lo, hi, first, last), dev)
                self.stages.append(DecodeEngine(w, layers=(lo, hi), stage_first=first, stage_last=last, **engine_kw))
        head = self.stages[-1]
        self.device = head.device
        self.n_slots, self.slot_ctx = head.n_slots, head.slot_ctx
        self.kv = _KvAll(self.stages)
        self.launches_per_step = 0
        self.n_mtp = 0
        self._ev = [torch.cuda.Event() for _ in self.stages]

    @property
    def logits(self):
        return self.stages[-1].logits

    @property
    def slot_len(self):
        return self.stages[-1].slot_len

    def step(self, rows: Sequence[Tuple[int, int, int]], head: bool = True) -> List[int]:
        if len(rows) > MAX_ROWS:
            raise ValueError(f"{len(rows)} rows exceed a pass of {MAX_ROWS}")
        prev = None
        for i, st in enumerate(self.stages):
            last = i == len(self.stages) - 1
            with torch.cuda.device(st.device):
                M = st.set_rows(rows)
                if st.use_graphs:
                    st._graph(M, head and last, False)      # capture (and its warm-up pass, which rewrites x) comes first
                if prev is not None:
                    cur = torch.cuda.current_stream(st.device)
                    cur.wait_event(self._ev[i - 1])
                    st.x[:M].copy_(prev.x[:M], non_blocking=True)      # the stage boundary: hidden rows of the pass
                st.launch(M, head and last, False)
                self._ev[i].record(torch.cuda.current_stream(st.device))
                for slot, _, pos in rows:
                    st.slot_len[slot] = max(st.slot_len[slot], pos + 1)
                if last and head:
                    out = st.read_tokens(len(rows))
                    word = out[M] & 0xFFFFFFFF
                    for other in self.stages[:-1]:                      # a fault word of an earlier stage counts too
                        with torch.cuda.device(other.device):
                            w2 = int(other.fault.item()) & 0xFFFFFFFF
                        word = min(word, w2)
                    if word != 0xFFFFFFFF:
                        from ..runtime.engine import EngineFault
                        for s2 in self.stages:
                            s2.poisoned = word
                        raise EngineFault(word)
                    return out[:len(rows)]
            prev = st
        return []

    def prefill(self, slot: int, tokens: Sequence[int], start: int = 0, gemm: Optional[bool] = None) -> int:
        last, n, i = 0, len(tokens), 0
        while i < n:
            chunk = tokens[i:i + MAX_ROWS]
            is_last = i + len(chunk) >= n
            out = self.step([(slot, int(t), start + i + j) for j, t in enumerate(chunk)], head=is_last)
            if is_last:
                last = out[len(chunk) - 1]
            i += len(chunk)
        return last

    def cut(self, slot: int, n_positions: int) -> None:
        for st in self.stages:
            with torch.cuda.device(st.device):
                st.cut(slot, n_positions)

    def reset(self, slot: int) -> None:
        for st in self.stages:
            with torch.cuda.device(st.device):
                st.reset(slot)

    def memory_report(self):
        out = {}
        for i, st in enumerate(self.stages):
            for k, v in st.memory_report().items():
                out[f"stage{i}.{k}"] = v
        return out
