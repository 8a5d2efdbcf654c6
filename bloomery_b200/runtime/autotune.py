"""Load-time race of equal kernel variants and the store of what they cost.

A variant set is a few ways to run the same site that produce the same bits (launch shaping only:
programmatic dependent launch on/off, graph replay vs eager).  At load each is timed on the
device with the weights cold in L2 and the fastest wins; results are kept in a JSON store keyed by
card, driver, build and shape so the next start skips the race (the reference:
``crates/gpu/src/autotune.rs:1-45``, ``crates/runtime/src/costs.rs``).
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
from typing import Callable, Dict, Optional, Tuple


class CostStore:
    def __init__(self, path: Optional[str]):
        self.path = path
        self.data: Dict[str, Dict[str, float]] = {}
        if path and os.path.exists(path):
            try:
                doc = json.load(open(path))
                if isinstance(doc, dict) and doc.get("version") == 1:
                    self.data = doc.get("costs", {})
            except (OSError, ValueError):
                self.data = {}             # an unreadable store is an empty store

    @staticmethod
    def key(card: str, driver: str, build: str, shape: Dict[str, object]) -> str:
        blob = json.dumps({"card": card, "driver": driver, "build": build, "shape": shape}, sort_keys=True)
        return hashlib.sha256(blob.encode()).hexdigest()[:24]

    def get(self, key: str) -> Optional[Dict[str, float]]:
        return self.data.get(key)

    def put(self, key: str, costs: Dict[str, float]) -> None:
        self.data[key] = dict(costs)
        if not self.path:
            return
        d = os.path.dirname(os.path.abspath(self.path))
        os.makedirs(d, exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=d, prefix=".costs.")
        with os.fdopen(fd, "w") as f:
            json.dump({"version": 1, "costs": self.data}, f)
        os.replace(tmp, self.path)          # readers never see a half-written store


def best_of(costs: Dict[str, float]) -> str:
    """Smallest cost wins; ties go to the name that sorts first, so a rerun picks the same variant."""
    return min(sorted(costs), key=lambda k: costs[k])


def race(variants: Dict[str, Callable[[], None]], time_one: Callable[[Callable[[], None]], float], reps: int = 5,
         flush: Optional[Callable[[], None]] = None) -> Tuple[str, Dict[str, float]]:
    """Time every variant ``reps`` times (median), flushing between runs; returns (winner, costs)."""
    costs: Dict[str, float] = {}
    for name, fn in variants.items():
        fn()                                  # warm-up: module load, attribute set-up
        ts = []
        for _ in range(reps):
            if flush is not None:
                flush()
            ts.append(time_one(fn))
        ts.sort()
        costs[name] = ts[len(ts) // 2]
    return best_of(costs), costs


def cuda_timer(stream=None) -> Callable[[Callable[[], None]], float]:
    import torch

    def time_one(fn) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    return time_one


def tune_decode_launch(engine, store: Optional[CostStore] = None, build: str = "") -> Dict[str, object]:
    """Race programmatic dependent launch on/off for one decode step of ``engine`` (equal bits either way)
    and leave the winner switched on.  Returns what was decided and why."""
    import torch
    from ..ops import decode as K
    s = engine.spec
    card = torch.cuda.get_device_name(engine.device)
    driver = str(torch.version.cuda)
    key = CostStore.key(card, driver, build, {"arch": s.arch, "layers": s.n_layer, "hidden": s.hidden, "experts": s.n_expert})
    known = store.get(key) if store else None
    if known:
        win = best_of(known)
        K.set_pdl(win == "pdl")
        return {"winner": win, "costs": known, "raced": False}
    flush_buf = torch.empty(192 << 20, dtype=torch.uint8, device=engine.device)
    engine.kv.ensure(0, 64)
    engine.kv.sync_table()

    def variant(pdl: bool):
        def run():
            K.set_pdl(pdl)
            engine.graphs.clear()
            engine.set_rows([(0, 0, 0)])
            engine.launch(1, True, False)
        return run
    win, costs = race({"pdl": variant(True), "plain": variant(False)}, cuda_timer(), flush=lambda: flush_buf.fill_(1))
    K.set_pdl(win == "pdl")
    engine.graphs.clear()
    engine.reset(0)
    if store:
        store.put(key, costs)
    return {"winner": win, "costs": costs, "raced": True}
