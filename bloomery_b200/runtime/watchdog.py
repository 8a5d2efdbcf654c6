"""Watchdog of the engine thread: names a wedged wait, never kills.

The engine thread brackets every bounded wait (a step's readback, a prompt unit, a host-tier
round) with ``enter``/``leave``.  A helper thread wakes once a second; a bracket older than the
bound is reported once -- a ``watchdog`` record with the site's name and age -- and the model is
marked wedged so ``/health`` can answer 503.  It does not interrupt anything: the bounded waits on
the device side end by themselves with a status (the reference: ``crates/gpu/src/watchdog.rs:1-33``,
``ENGINE_BOUND`` = 60 s in ``crates/gpu/src/host/mod.rs:462``).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Tuple


class Watchdog:
    def __init__(self, model: str = "model", bound_s: float = 60.0, period_s: float = 1.0,
                 report: Optional[Callable[[str, float], None]] = None, clock=time.monotonic):
        self.model, self.bound_s, self.period_s = model, bound_s, period_s
        self._report = report
        self._clock = clock
        self._lock = threading.Lock()
        self._open: Dict[int, Tuple[str, float, bool]] = {}      # token -> (site, since, reported)
        self._next = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.wedged: List[Tuple[str, float]] = []

    def start(self) -> "Watchdog":
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name=f"watchdog:{self.model}", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.period_s + 1)
            self._thread = None

    def enter(self, site: str) -> int:
        with self._lock:
            self._next += 1
            self._open[self._next] = (site, self._clock(), False)
            return self._next

    def leave(self, token: int) -> None:
        with self._lock:
            self._open.pop(token, None)

    class _Guard:
        def __init__(self, wd, site):
            self.wd, self.site = wd, site

        def __enter__(self):
            self.tok = self.wd.enter(self.site)

        def __exit__(self, *exc):
            self.wd.leave(self.tok)
            return False

    def guard(self, site: str) -> "Watchdog._Guard":
        return Watchdog._Guard(self, site)

    def is_wedged(self) -> bool:
        with self._lock:
            return any(rep for _, _, rep in self._open.values())

    def poll(self) -> List[Tuple[str, float]]:
        """One pass of the helper thread (callable directly from tests)."""
        now = self._clock()
        fresh = []
        with self._lock:
            for tok, (site, since, reported) in list(self._open.items()):
                if not reported and now - since > self.bound_s:
                    self._open[tok] = (site, since, True)
                    fresh.append((site, now - since))
        for site, age in fresh:
            self.wedged.append((site, age))
            if self._report is not None:
                self._report(site, age)
        return fresh

    def _run(self) -> None:
        while not self._stop.wait(self.period_s):
            self.poll()


class Waits:
    """Totals of the time the engine thread spent waiting, by kind (``/metrics``; the reference's
    ``crates/gpu/src/waits.rs``).  Plain adds under the GIL: readers see a recent total."""

    KINDS = ("card", "host_tier", "h2d", "prompt_cache")

    def __init__(self):
        self.ns = {k: 0 for k in self.KINDS}
        self.n = {k: 0 for k in self.KINDS}

    def add(self, kind: str, seconds: float) -> None:
        self.ns[kind] = self.ns.get(kind, 0) + int(seconds * 1e9)
        self.n[kind] = self.n.get(kind, 0) + 1

    def timed(self, kind: str):
        w = self

        class _T:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                w.add(kind, time.perf_counter() - self.t0)
                return False
        return _T()

    def metrics(self) -> Dict[str, float]:
        out = {}
        for k in self.ns:
            out[f"wait_{k}_seconds_total"] = self.ns[k] / 1e9
            out[f"wait_{k}_total"] = self.n[k]
        return out


class CaptureLock:
    """Per-device reader/writer lock: stream captures hold it shared, anything that synchronises the
    whole context or creates handles holds it exclusive, so a capture is never invalidated by a
    sync issued from another thread (the reference: ``crates/gpu/src/capsync.rs:1-40``)."""

    def __init__(self):
        self._cond = threading.Condition()
        self._shared = 0
        self._exclusive = False
        self._waiting_exclusive = 0

    def acquire_shared(self) -> None:
        with self._cond:
            while self._exclusive or self._waiting_exclusive:
                self._cond.wait()
            self._shared += 1

    def release_shared(self) -> None:
        with self._cond:
            self._shared -= 1
            if self._shared == 0:
                self._cond.notify_all()

    def acquire_exclusive(self) -> None:
        with self._cond:
            self._waiting_exclusive += 1
            while self._exclusive or self._shared:
                self._cond.wait()
            self._waiting_exclusive -= 1
            self._exclusive = True

    def release_exclusive(self) -> None:
        with self._cond:
            self._exclusive = False
            self._cond.notify_all()

    def capture(self):
        lk = self

        class _S:
            def __enter__(self):
                lk.acquire_shared()

            def __exit__(self, *exc):
                lk.release_shared()
                return False
        return _S()

    def sync(self):
        lk = self

        class _X:
            def __enter__(self):
                lk.acquire_exclusive()

            def __exit__(self, *exc):
                lk.release_exclusive()
                return False
        return _X()


_DEVICE_LOCKS: Dict[str, CaptureLock] = {}
_DEVICE_LOCKS_GUARD = threading.Lock()


def device_lock(device) -> CaptureLock:
    with _DEVICE_LOCKS_GUARD:
        return _DEVICE_LOCKS.setdefault(str(device), CaptureLock())
