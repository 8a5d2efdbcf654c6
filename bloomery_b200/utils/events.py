"""Start events: one JSON object per line on stdout for whoever started the server
(``crates/serve/src/event.rs:1-11``): ``pick``, ``bound`` (listener up, answers ``loading``),
``ready`` (first moment requests are served), ``error`` (before every non-zero exit),
``stopped``.  Human-readable lines stay on stderr."""
from __future__ import annotations

import json
import sys
import threading

SCHEMA = "bloomery.event/1"
_enabled = False
_lock = threading.Lock()
_sink = None


def enable(sink=None) -> None:
    global _enabled, _sink
    _enabled, _sink = True, sink


def emit(event: str, **fields) -> None:
    if not _enabled:
        return
    line = json.dumps({"schema": SCHEMA, "event": event, **fields}, separators=(",", ":"))
    with _lock:
        out = _sink or sys.stdout
        out.write(line + "\n")
        out.flush()
