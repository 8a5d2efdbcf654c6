"""Router traces and the census of where picks were served.

A trace file records, for every kept position and MoE layer, the expert ids and weights the router
chose; the residency rule can be replayed offline against it and two engines can be compared pick by
pick.  The census counts how many picks each tier served (the reference:
``crates/gpu/src/host/route_trace.rs``, ``census.rs``).

File layout (little endian): magic ``BLRT`` u32 version=1, u32 n_layer, u32 top_k, then records of
``u32 position, u32 layer, top_k x i32 id, top_k x f32 weight``.
"""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

MAGIC = b"BLRT"


class RouteTraceWriter:
    def __init__(self, path: str, n_layer: int, top_k: int):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.f = open(path, "wb")
        self.n_layer, self.top_k = n_layer, top_k
        self.f.write(MAGIC + struct.pack("<III", 1, n_layer, top_k))
        self.n = 0

    def add(self, position: int, layer: int, ids: Sequence[int], weights: Sequence[float]) -> None:
        if len(ids) != self.top_k or len(weights) != self.top_k:
            raise ValueError("a trace record holds exactly top_k picks")
        self.f.write(struct.pack(f"<II{self.top_k}i{self.top_k}f", position, layer, *[int(i) for i in ids],
                                 *[float(w) for w in weights]))
        self.n += 1

    def close(self) -> None:
        self.f.close()


def read_trace(path: str) -> Tuple[int, int, Iterator[Tuple[int, int, List[int], List[float]]]]:
    f = open(path, "rb")
    head = f.read(16)
    if len(head) < 16 or head[:4] != MAGIC:
        raise ValueError(f"{path}: not a route trace")
    ver, n_layer, top_k = struct.unpack("<III", head[4:])
    if ver != 1:
        raise ValueError(f"{path}: trace version {ver}")
    rec = struct.Struct(f"<II{top_k}i{top_k}f")

    def it():
        with f:
            while True:
                b = f.read(rec.size)
                if not b:
                    return
                if len(b) < rec.size:
                    raise ValueError(f"{path}: truncated record")
                v = rec.unpack(b)
                yield v[0], v[1], list(v[2:2 + top_k]), list(v[2 + top_k:])
    return n_layer, top_k, it()


class Census:
    """Counts of picks by where they were served."""

    PLACES = ("card", "host", "peer", "spare")

    def __init__(self, n_layer: int):
        self.counts: List[Dict[str, int]] = [{p: 0 for p in self.PLACES} for _ in range(n_layer)]

    def add(self, layer: int, place: str, n: int = 1) -> None:
        self.counts[layer][place] += n

    def add_picks(self, layer: int, ids: Sequence[int], slot_map: Optional[Sequence[int]]) -> None:
        """``slot_map[e] >= 0`` = resident on this card; ``-1`` = served by the host tier."""
        for e in ids:
            if e < 0:
                self.add(layer, "peer")
            elif slot_map is None or slot_map[e] >= 0:
                self.add(layer, "card")
            else:
                self.add(layer, "host")

    def totals(self) -> Dict[str, int]:
        return {p: sum(c[p] for c in self.counts) for p in self.PLACES}

    def share(self, place: str) -> float:
        t = self.totals()
        n = sum(t.values())
        return t[place] / n if n else 0.0


def trace_engine(engine, prompt: Sequence[int], n_new: int, path: str) -> int:
    """Run ``engine`` eagerly over ``prompt`` then ``n_new`` greedy tokens, recording every routed pick.
    Returns the number of records.  (Eager on purpose: the ids of a layer are read back before the next
    layer overwrites them.)"""
    import torch
    s = engine.spec
    w = RouteTraceWriter(path, s.n_layer, s.n_used)
    orig = engine._moe

    state = {"pos": []}

    def traced(il, M, x):
        n = orig(il, M, x)
        torch.cuda.current_stream().synchronize()
        ids, wts = engine.r_ids_all[il][:M].cpu().tolist(), engine.r_wts_all[il][:M].cpu().tolist()
        for m, p in enumerate(state["pos"][:M]):
            w.add(p, il, ids[m], wts[m])
        return n

    was_graphs = engine.use_graphs
    engine.use_graphs, engine._moe = False, traced
    try:
        engine.reset(0)
        tok = None
        for i in range(0, len(prompt), 8):
            chunk = list(prompt[i:i + 8])
            state["pos"] = list(range(i, i + len(chunk)))
            tok = engine.step([(0, t, i + j) for j, t in enumerate(chunk)])[-1]
        pos = len(prompt)
        for _ in range(n_new):
            state["pos"] = [pos]
            tok = engine.step([(0, tok, pos)])[0]
            pos += 1
    finally:
        engine._moe, engine.use_graphs = orig, was_graphs
        w.close()
    return w.n
