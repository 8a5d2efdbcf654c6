"""The start screen and the live view: views for a person over the record lines the start printed and over the requests
the server has answered, drawn on stderr when it is a terminal.

The start screen is drawn once, below the record lines, when the server begins to serve.  It is armed (:func:`arm`) when
``BLOOMERY_SCREEN`` is on and stderr is a terminal; piped stderr is never armed, so it carries the record lines alone.
It reads the lines' text as printed and nothing else: every value on it is a record's, a byte count shown in GiB to one
decimal.  A row is read from the last line of its record's kind; a fact whose record the start did not print is left
off; a record the start printed whose value does not read as a number is named on an ``unread`` row, never left off as
if it had not been printed.  ``NO_COLOR`` (set and not empty) and ``TERM=dumb`` draw it without colour; ``TERM=dumb`` or
a locale that does not name UTF-8 draws it in plain ASCII; ``COLORTERM=truecolor`` (or ``24bit``) draws its colours as
they are, any other terminal gets the nearest of the 256-colour cube.

The screen is a wordmark, a status line with the address, then two panels: where the model went (the cards, the host,
with a bar of each one's share) and how it serves (the placement, the context and slots, the prompt cache).  Wide
terminals set the panels side by side, narrow ones stack them; widths below four columns are refused.  Its last row names
the keys: ``Ctrl+C``, ``BLOOMERY_SCREEN=off`` and ``d`` for the live view.

The live view (:class:`Ring`, :func:`live_view`) keeps the last request lines the worker printed and draws them with the
counters of ``/metrics``; ``d`` toggles it while stdin is a terminal (:func:`watch_keys`).

Counterpart of the reference's ``crates/serve/src/screen.rs`` and ``crates/serve/src/live/`` (ring, parts, view, term).
"""
from __future__ import annotations

import collections
import dataclasses
import json
import os
import sys
import threading
from typing import Callable, Deque, Dict, Iterable, List, Mapping, Optional, Tuple

ORANGE, GREY, WHITE = (255, 140, 40), (140, 140, 140), (235, 235, 235)
MIN_WIDTH, SIDE_BY_SIDE = 4, 96


@dataclasses.dataclass(frozen=True)
class Style:
    color: bool
    truecolor: bool
    utf8: bool

    @staticmethod
    def of(env: Mapping[str, str]) -> "Style":
        term = env.get("TERM")
        dumb = term == "dumb"
        color = not dumb and not env.get("NO_COLOR")
        locale = next((env[k] for k in ("LC_ALL", "LC_CTYPE", "LANG") if env.get(k)), "")
        utf8 = not dumb and ("utf-8" in locale.lower() or "utf8" in locale.lower())
        return Style(color, env.get("COLORTERM") in ("truecolor", "24bit"), utf8)

    def paint(self, text: str, rgb: Tuple[int, int, int]) -> str:
        if not self.color or not text:
            return text
        if self.truecolor:
            return f"\x1b[38;2;{rgb[0]};{rgb[1]};{rgb[2]}m{text}\x1b[0m"
        cube = 16 + 36 * round(rgb[0] / 255 * 5) + 6 * round(rgb[1] / 255 * 5) + round(rgb[2] / 255 * 5)
        return f"\x1b[38;5;{cube}m{text}\x1b[0m"


def gib(n: float) -> str:
    return f"{n / (1 << 30):.1f} GiB"


def last_records(lines: Iterable[str]) -> Dict[str, dict]:
    """The fields of the last line of each record kind, from the lines as printed (``kind<TAB>json``)."""
    out: Dict[str, dict] = {}
    for ln in lines:
        kind, sep, body = ln.rstrip("\n").partition("\t")
        if not sep:
            continue
        try:
            fields = json.loads(body)
        except json.JSONDecodeError:
            out[kind] = {"_unread": body[:60]}
            continue
        if isinstance(fields, dict):
            out[kind] = fields
    return out


def _num(rec: dict, key: str, unread: List[str], kind: str) -> Optional[float]:
    if key not in rec:
        return None
    v = rec[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        unread.append(f"{kind}.{key}={v!r}")
        return None
    return float(v)


def _bar(share: float, width: int, style: Style) -> str:
    width = max(1, width)
    full = max(0, min(width, round(share * width)))
    on, off = ("█", "░") if style.utf8 else ("#", ".")
    return style.paint(on * full, ORANGE) + style.paint(off * (width - full), GREY)


def panels(recs: Dict[str, dict], style: Style, width: int) -> Tuple[List[str], List[str], List[str]]:
    """(where the model went, how it serves, unread values) as plain rows of at most ``width`` columns."""
    unread: List[str] = []
    where: List[str] = ["where the model went"]
    how: List[str] = ["how it serves"]
    for kind, rec in recs.items():
        if "_unread" in rec:
            unread.append(f"{kind}: {rec['_unread']}")
    plan, need, ctx, par, setup = (recs.get(k, {}) for k in ("plan", "need", "ctx", "parallel", "setup"))
    weights, kv = _num(plan, "weights_bytes", unread, "plan"), _num(plan, "kv_bytes", unread, "plan")
    host = _num(need, "host_bytes", unread, "need")
    devices = plan.get("devices")
    total = (weights or 0.0) + (host or 0.0)
    bar_w = max(4, min(24, width - 34))
    if weights is not None:
        n_dev = len(devices) if isinstance(devices, list) and devices else 1
        label = f"cards x{n_dev}" if n_dev > 1 else "card"
        where.append(f"  {label:<10} {gib(weights):>10}  {_bar(weights / total if total else 1.0, bar_w, style)}")
    if host:
        where.append(f"  {'host':<10} {gib(host):>10}  {_bar(host / total if total else 0.0, bar_w, style)}")
    if kv is not None:
        where.append(f"  {'context':<10} {gib(kv):>10}")
    per_layer = setup.get("resident_per_layer")
    if per_layer is not None:
        where.append(f"  experts resident per layer: {per_layer}")
    if plan.get("place") not in (None, ""):
        how.append(f"  placement  {plan['place']}")
    served = _num(ctx, "served", unread, "ctx")
    if served is not None:
        rule = ctx.get("rule")
        how.append(f"  context    {int(served):,}" + (f" ({rule})" if rule else ""))
    slots = _num(par, "slots", unread, "parallel")
    if slots is not None:
        src = par.get("source")
        how.append(f"  slots      {int(slots)}" + (f" (from {src})" if src else ""))
    cache = _num(need, "cache_ram", unread, "need")
    if cache is not None:
        how.append(f"  prompt cache {gib(cache)}" if cache > 0 else "  prompt cache off")
    return where, how, unread


def draw(lines: Iterable[str], address: str, width: int, style: Style, live_keys: bool = False) -> str:
    """The whole screen as text for a terminal ``width`` columns wide."""
    if width < MIN_WIDTH:
        raise ValueError(f"a screen of {width} columns: at least {MIN_WIDTH}")
    recs = last_records(lines)
    where, how, unread = panels(recs, style, width)
    dot = "●" if style.utf8 else "*"
    rule = ("─" if style.utf8 else "-") * min(width, 72)
    out = [style.paint("bloomery", ORANGE) + style.paint("  b200", GREY), style.paint(rule, GREY),
           f"{style.paint(dot, ORANGE)} serving on {style.paint(address, WHITE)}", ""]
    where = where if len(where) > 1 else []
    how = how if len(how) > 1 else []
    if width >= SIDE_BY_SIDE and where and how:
        left_w = width // 2
        import re
        bare = lambda s: re.sub(r"\x1b\[[0-9;]*m", "", s)                                   # noqa: E731
        for i in range(max(len(where), len(how))):
            left = where[i] if i < len(where) else ""
            out.append(left + " " * max(1, left_w - len(bare(left))) + (how[i] if i < len(how) else ""))
    else:
        out += where + ([""] if where and how else []) + how
    if unread:
        out += ["", "unread"] + [f"  {u}" for u in unread]
    keys = ["Ctrl+C stops", "BLOOMERY_SCREEN=off hides this"] + (["d shows the live view"] if live_keys else [])
    out += ["", style.paint("  ".join(keys), GREY)]
    return "\n".join(ln if style.color else ln[:width] for ln in out) + "\n"


# ------------------------------------------------------------------------------------------------- arming and notes
_armed = False
_lines: List[str] = []
_lock = threading.Lock()


def arm(env: Mapping[str, str], is_terminal: bool, lever: str = "on") -> bool:
    """Arm the screen for this start: the lever is on and stderr is a terminal."""
    global _armed
    with _lock:
        _armed = lever != "off" and bool(is_terminal)
        _lines.clear()
    return _armed


def note(line: str) -> None:
    """A record line the start printed (kept for the screen and the live view whether or not the screen is armed)."""
    with _lock:
        _lines.append(line)
        del _lines[:-512]


def records() -> List[str]:
    with _lock:
        return list(_lines)


def draw_if_armed(address: str, env: Optional[Mapping[str, str]] = None, out=None, live_keys: bool = False) -> bool:
    if not _armed:
        return False
    env = os.environ if env is None else env
    out = out or sys.stderr
    try:
        width = os.get_terminal_size(out.fileno()).columns
    except (OSError, ValueError, AttributeError):
        width = 80
    try:
        out.write(draw(records(), address, width, Style.of(env), live_keys))
        out.flush()
    except ValueError:
        return False
    return True


# ------------------------------------------------------------------------------------------------------- live view
class Ring:
    """The last ``n`` request lines the worker printed, newest last."""

    def __init__(self, n: int = 32):
        self._items: Deque[str] = collections.deque(maxlen=n)
        self._lock = threading.Lock()

    def push(self, line: str) -> None:
        with self._lock:
            self._items.append(line.rstrip("\n"))

    def lines(self) -> List[str]:
        with self._lock:
            return list(self._items)


def live_view(ring: Ring, counters: Mapping[str, float], width: int, style: Style, rows: int = 12) -> str:
    """The live view: a line of counters, then the newest request lines, each cut to the width."""
    if width < MIN_WIDTH:
        raise ValueError(f"a view of {width} columns: at least {MIN_WIDTH}")
    head = "  ".join(f"{k} {v:g}" for k, v in counters.items())
    body = ring.lines()[-rows:] or ["no request has ended yet"]
    cut = lambda s: s if len(s) <= width else s[:max(1, width - 1)] + ("…" if style.utf8 else ">")      # noqa: E731
    return "\n".join([style.paint(cut("live  " + head), ORANGE)] + [cut(ln) for ln in body]
                     + [style.paint(cut("d hides this view"), GREY)]) + "\n"


def watch_keys(on_key: Callable[[str], None], stdin=None, stop: Optional[threading.Event] = None) -> Optional[threading.Thread]:
    """Read single keys from a terminal stdin on a thread and hand each to ``on_key``; None when stdin is no terminal (a
    server under a supervisor takes no keys)."""
    stdin = stdin or sys.stdin
    try:
        if not stdin.isatty():
            return None
        import termios
        import tty
        fd = stdin.fileno()
        saved = termios.tcgetattr(fd)
    except (OSError, ValueError, AttributeError, ImportError):
        return None
    stop = stop or threading.Event()

    def loop():
        import select
        try:
            tty.setcbreak(fd)
            while not stop.is_set():
                ready, _, _ = select.select([fd], [], [], 0.25)
                if ready:
                    ch = os.read(fd, 1).decode(errors="ignore")
                    if ch:
                        on_key(ch)
        except (OSError, ValueError):
            pass
        finally:
            try:
                termios.tcsetattr(fd, termios.TCSADRAIN, saved)
            except (OSError, ValueError, termios.error):
                pass
    th = threading.Thread(target=loop, name="live-keys", daemon=True)
    th.start()
    return th
