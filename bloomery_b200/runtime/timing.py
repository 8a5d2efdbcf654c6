"""Timing aids that cost nothing when they are off.

* :class:`PromptTiming` keeps one CUDA event per (layer, unit) mark of a prompt micro-batch when armed and
  nothing when not (the reference: ``crates/gpu/src/prompt_timing.rs:1-8``).
* :class:`HostProfile` is the CPU-side profiler of ``BLOOMERY_PROFILE=0|1|2``: level 0 is one attribute test per
  call site, level 1 a clock pair per call, level 2 splits rows by stage (``crates/model/src/profile.rs:1-45``).
* ``save_heat`` / ``load_heat`` keep the routing heat of a model between runs, so the residency rule starts
  warm (the reference's warm profile: ``crates/runtime/src/warmprof.rs``).
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional, Tuple


class PromptTiming:
    def __init__(self):
        self.armed = False
        self.marks: List[Tuple[int, str, object]] = []

    def arm(self, on: bool = True) -> None:
        self.armed = on
        self.marks = []

    def mark(self, layer: int, unit: str) -> None:
        if not self.armed:
            return
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((layer, unit, ev))

    def report(self) -> Dict[str, float]:
        """Milliseconds per unit, summed over layers (synchronises on the last mark)."""
        out: Dict[str, float] = {}
        if len(self.marks) < 2:
            return out
        self.marks[-1][2].synchronize()
        for (l0, u0, e0), (l1, u1, e1) in zip(self.marks, self.marks[1:]):
            out[u1] = out.get(u1, 0.0) + e0.elapsed_time(e1)
        return out


class HostProfile:
    def __init__(self, level: Optional[int] = None):
        if level is None:
            from ..utils import levers
            level = int(levers.get("BLOOMERY_PROFILE"))
        self.level = level
        self.totals: Dict[str, float] = {}
        self.calls: Dict[str, int] = {}

    def span(self, name: str, detail: bool = False):
        """Context manager; a no-op object when the level does not ask for this span."""
        if self.level == 0 or (detail and self.level < 2):
            return _NOOP
        return _Span(self, name)

    def report(self) -> Dict[str, Dict[str, float]]:
        return {k: {"seconds": v, "calls": self.calls[k]} for k, v in sorted(self.totals.items())}


class _Noop:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NOOP = _Noop()


class _Span:
    def __init__(self, prof: HostProfile, name: str):
        self.p, self.name = prof, name

    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        dt = time.perf_counter() - self.t0
        self.p.totals[self.name] = self.p.totals.get(self.name, 0.0) + dt
        self.p.calls[self.name] = self.p.calls.get(self.name, 0) + 1
        return False


def save_heat(heat, path: str, model: str = "") -> None:
    """``heat``: int tensor [n_layer, n_expert] of routed counts."""
    doc = {"version": 1, "model": model, "heat": [[int(v) for v in row] for row in heat.cpu().tolist()]}
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(doc, f)
    os.replace(tmp, path)


def load_heat(path: str, n_layer: int, n_expert: int, model: str = ""):
    """The saved counts as a list of rows, or None when the file is missing, unreadable or of another shape / model."""
    try:
        doc = json.load(open(path))
    except (OSError, ValueError):
        return None
    h = doc.get("heat")
    if doc.get("version") != 1 or (model and doc.get("model") not in ("", model)) or not isinstance(h, list):
        return None
    if len(h) != n_layer or any(not isinstance(r, list) or len(r) != n_expert for r in h):
        return None
    return h
