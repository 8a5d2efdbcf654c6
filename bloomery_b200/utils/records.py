"""Typed log lines with a schema and a reader (``crates/record/src/lib.rs:1-22``): each line
is ``kind<TAB>json`` on stderr; ``--records-schema`` prints the table of kinds."""
from __future__ import annotations

import json
import sys
import time
from typing import Dict, Iterable, Iterator, List, Tuple

KINDS: Dict[str, List[str]] = {
    "plan": ["model", "devices", "weights_bytes", "kv_bytes", "ctx", "slots", "place"],
    "need": ["weights_bytes", "kv_bytes_per_token", "host_bytes", "fits", "bytes", "pinned", "cache_ram", "cards", "threads",
             "allowed"],
    "ctx": ["asked", "served", "trained", "rule"],
    "parallel": ["slots", "slot_ctx", "source"],
    "setup": ["phase", "seconds", "winner", "raced", "resident_per_layer", "host", "page_cache"],
    "watchdog": ["model", "site", "seconds"],
    "step_stats": ["steps", "card_wait_s", "kv_free_pages", "kv_spills", "free_bytes"],
    "request": ["id", "route", "slot", "prompt_tokens", "cached_tokens", "predicted_tokens", "prompt_ms",
                "predicted_ms", "status"],
    "progress": ["slot", "tokens", "tok_per_s"],
    "residency": ["layer", "flips", "resident_hits", "host_hits"],
    "fault": ["layer", "site", "message"],
}


def schema() -> str:
    return json.dumps({"schema": "bloomery.record/1", "kinds": KINDS}, indent=1)


_taps: List = []


def tap(fn) -> None:
    """Hand every record line written from now on to ``fn`` as well (the start screen reads the lines as printed)."""
    if fn not in _taps:
        _taps.append(fn)


def write(kind: str, _out=None, **fields) -> None:
    if kind not in KINDS:
        raise KeyError(f"unknown record kind {kind!r}")
    unknown = set(fields) - set(KINDS[kind])
    if unknown:
        raise KeyError(f"record {kind!r} has no field(s) {sorted(unknown)}")
    out = _out or sys.stderr
    line = f"{kind}\t{json.dumps({'t': round(time.time(), 3), **fields}, separators=(',', ':'))}\n"
    out.write(line)
    out.flush()
    for fn in _taps:
        fn(line)


def read(lines: Iterable[str]) -> Iterator[Tuple[str, dict]]:
    """Yield (kind, fields) of every well-formed record line; other lines are skipped."""
    for ln in lines:
        kind, sep, body = ln.rstrip("\n").partition("\t")
        if not sep or kind not in KINDS:
            continue
        try:
            yield kind, json.loads(body)
        except json.JSONDecodeError:
            continue
