"""Per-key limits on the requests a key makes, and the routes a key reaches.

A line of the key file is ``KEY [scope=S[,S]] [inflight=N] [rate=N/s | rate=N/m] [burst=B]``:

* ``scope=``: ``inference`` (generation, token counts, the tokenizer, embeddings, stored responses), ``read``
  (``GET /props``, ``/slots``, ``/metrics``) or ``admin`` (every route; the default), comma-separated; ``inference`` and
  ``read`` both reach the model list and lookups; slot actions, ``/residency/reset`` and ``/shutdown`` need ``admin``.  A
  route outside the scope answers 403 (``permission_error``);
* ``inflight=N``: the most generating requests the key may have open at once;
* ``rate=N/s`` or ``rate=N/m`` with ``burst=B`` (``N`` unless set): a bucket of ``B`` requests that refills ``N`` a second
  or a minute, each generating request taking one.

A request past either limit is answered 429 with ``Retry-After`` and starts nothing; a key with neither field is limited
by nothing; every key counts apart.  Only routes that start a generation take a place (chat, completions, messages,
responses, embeddings); reading a stored response, tokenising or listing models never does, so they can be used while a
generation holds the key's last place.  (The reference: ``crates/serve/src/admit.rs``.)
"""
from __future__ import annotations

import math
import threading
import time
from typing import Callable, Dict, Optional, Tuple

MOST = 1_000_000          # the largest N or B a field takes


class LimitError(ValueError):
    """A key-file line whose limit fields do not parse; the message names the field, never the key."""


SCOPES = ("inference", "read", "admin")
_INFERENCE_PREFIXES = ("/completion", "/completions", "/v1/completions", "/v1/chat/completions", "/chat/completions", "/v1/messages",
                       "/v1/responses", "/v1/embeddings", "/embeddings", "/embedding", "/tokenize", "/detokenize",
                       "/apply-template", "/v1/systemone")
_READ_PATHS = ("/props", "/slots", "/metrics")
_LOOKUP_PREFIXES = ("/v1/models", "/models", "/api/tags", "/api/show")


def route_scope(method: str, path: str) -> str:
    """The scope a request needs: ``public`` (health), ``lookup`` (model list: any scope), ``inference``, ``read`` or
    ``admin``."""
    path = path.rstrip("/") or "/"
    if path in ("/health", "/v1/health") or method == "OPTIONS":
        return "public"
    if any(path == p_ or path.startswith(p_ + "/") for p_ in _LOOKUP_PREFIXES):
        return "lookup"
    if method == "GET" and path in _READ_PATHS:
        return "read"
    if any(path == p_ or path.startswith(p_ + "/") for p_ in _INFERENCE_PREFIXES):
        return "inference"
    return "admin"                             # slot actions, /residency/reset, /shutdown, anything unnamed


class Limits:
    def __init__(self, inflight: Optional[int] = None, rate: Optional[Tuple[int, bool]] = None, burst: Optional[int] = None,
                 scopes: Optional[frozenset] = None):
        self.inflight = inflight
        self.rate = rate                      # (count, per_minute)
        self.burst = burst if burst is not None else (rate[0] if rate else None)
        self.scopes = scopes if scopes is not None else frozenset(("admin",))

    def reaches(self, method: str, path: str) -> bool:
        need = route_scope(method, path)
        if need == "public" or "admin" in self.scopes:
            return True
        if need == "lookup":
            return bool(self.scopes & {"inference", "read"})
        return need in self.scopes

    def same(self, other: "Limits") -> bool:
        return (self.inflight, self.rate, self.burst, self.scopes) == (other.inflight, other.rate, other.burst, other.scopes)

    @property
    def interval(self) -> float:
        n, per_minute = self.rate
        return (60.0 if per_minute else 1.0) / n

    @staticmethod
    def _count(name: str, shown: str, text: str) -> int:
        if not text.isdigit() or not 1 <= int(text) <= MOST:
            raise LimitError(f"{name}={shown}: takes a whole number from 1 to {MOST}")
        return int(text)

    @classmethod
    def parse(cls, fields) -> "Limits":
        inflight = rate = burst = scopes = None
        seen = set()
        for name, value in fields:
            if name in seen:
                raise LimitError(f"{name}: named twice")
            seen.add(name)
            if name == "scope":
                got = [v for v in value.split(",")]
                if not value or any(v not in SCOPES for v in got):
                    raise LimitError(f"scope={value}: takes inference, read or admin, comma-separated")
                scopes = frozenset(got)
            elif name == "inflight":
                inflight = cls._count(name, value, value)
            elif name == "burst":
                burst = cls._count(name, value, value)
            elif name == "rate":
                n, sep, unit = value.partition("/")
                if not sep:
                    raise LimitError(f"rate={value}: takes N/s or N/m, a count a second or a minute")
                if unit not in ("s", "m"):
                    raise LimitError(f"rate={value}: the unit is s or m")
                rate = (cls._count(name, value, n), unit == "m")
            else:
                raise LimitError(f"{name}: not a field of a key line (scope, inflight, rate, burst)")
        if burst is not None and rate is None:
            raise LimitError("burst: needs a rate beside it")
        return cls(inflight, rate, burst, scopes)


def parse_key_line(line: str) -> Tuple[str, Limits]:
    """``KEY name=value ...`` -> (key, limits)."""
    parts = line.split()
    fields = []
    for f in parts[1:]:
        name, sep, value = f.partition("=")
        if not sep:
            raise LimitError(f"{name}: fields are name=value")
        fields.append((name, value))
    return parts[0], Limits.parse(fields)


class Admission:
    """Counts every key apart.  ``admit(key)`` returns a release callable, or raises :class:`Refused`."""

    def __init__(self, limits: Dict[str, Limits], clock: Callable[[], float] = time.monotonic):
        self.limits = limits
        self.clock = clock
        self.lock = threading.Lock()
        self.open: Dict[str, int] = {}
        self.bucket: Dict[str, Tuple[float, float]] = {}       # key -> (tokens, time of that count)

    def admit(self, key: str) -> Callable[[], None]:
        lim = self.limits.get(key)
        if lim is None or (lim.inflight is None and lim.rate is None):
            return lambda: None
        with self.lock:
            now = self.clock()
            if lim.inflight is not None and self.open.get(key, 0) >= lim.inflight:
                raise Refused(f"this key has {lim.inflight} requests in flight, its limit", 1)
            if lim.rate is not None:
                tokens, at = self.bucket.get(key, (float(lim.burst), now))
                tokens = min(float(lim.burst), tokens + (now - at) / lim.interval)
                if tokens < 1.0:
                    wait = (1.0 - tokens) * lim.interval
                    self.bucket[key] = (tokens, now)
                    n, per_minute = lim.rate
                    raise Refused(f"this key is limited to {n} requests a {'minute' if per_minute else 'second'}",
                                  max(1, math.ceil(wait)))
                self.bucket[key] = (tokens - 1.0, now)
            self.open[key] = self.open.get(key, 0) + 1
        done = [False]

        def release() -> None:
            with self.lock:
                if not done[0]:
                    done[0] = True
                    self.open[key] = max(0, self.open.get(key, 0) - 1)
        return release


class Refused(Exception):
    def __init__(self, message: str, retry_after: int):
        super().__init__(message)
        self.retry_after = retry_after
