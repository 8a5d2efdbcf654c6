"""Request-side rules of a model's think span: the effort word, the budget in generated ids, and the loop check.

* ``reasoning_effort`` takes OpenAI's words (``none``, ``minimal``, ``low``, ``medium``, ``high``, ``xhigh``) and ``max``.
  ``none`` turns thinking off before the template (it reads ``enable_thinking: false`` and the whole output lands in
  ``content``); every other word asks for reasoning (``enable_thinking: true``).  A ``chat_template_kwargs``
  ``enable_thinking`` in the same request wins when it agrees and is a 400 naming both fields when it asks the opposite.
* ``reasoning_budget``: the think span's budget in generated ids; ``0`` closes it at once, ``-1`` or absent leaves it
  alone.  When the span has used its budget the closing tag is written for the model (:class:`ThinkSpan.force_close`).
* ``reasoning_loop``: ``true`` ends a generation whose open think span repeats a cycle of up to 1,024 ids over at least
  256 ids and one whole cycle (:func:`find_loop`).

The reference keeps the same rules in ``crates/serve/src/reasoning.rs`` (span split and budget) and its generation loop.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Sequence

import numpy as np

EFFORTS = ("none", "minimal", "low", "medium", "high", "xhigh", "max")
MAX_CYCLE, MIN_SPAN = 1024, 256


class ReasoningError(ValueError):
    """A request whose reasoning fields cannot be served as asked (the API answers 400 with this message)."""


def effort_kwargs(effort: Any, kwargs: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    """The template kwargs of a request that names ``reasoning_effort`` (None = not named)."""
    out = dict(kwargs or {})
    if effort is None:
        return out
    if not isinstance(effort, str) or effort not in EFFORTS:
        raise ReasoningError(f"reasoning_effort takes one of {', '.join(EFFORTS)}")
    want = effort != "none"
    given = out.get("enable_thinking")
    if given is not None and bool(given) != want:
        raise ReasoningError(f"chat_template_kwargs.enable_thinking={str(bool(given)).lower()} beside reasoning_effort={effort!r} "
                             f"ask for opposite thinking")
    out["enable_thinking"] = want
    out["reasoning_effort"] = effort
    return out


def budget_from(body: Dict[str, Any], forced_tool: bool = False) -> int:
    v = body.get("reasoning_budget")
    if v is None:
        return -1
    if isinstance(v, bool) or not isinstance(v, int) or v < -1:
        raise ReasoningError("reasoning_budget takes a whole number of ids, -1 for no budget")
    if v >= 0 and forced_tool:
        raise ReasoningError("reasoning_budget beside a forced tool_choice: a forced call leaves no think span to budget")
    return v


def loop_flag(body: Dict[str, Any]) -> bool:
    v = body.get("reasoning_loop")
    if v is None or v is False:
        return False
    if v is not True:
        raise ReasoningError("reasoning_loop takes true or false")
    return True


def find_loop(ids: Sequence[int], max_cycle: int = MAX_CYCLE, min_span: int = MIN_SPAN) -> int:
    """The shortest cycle length L <= ``max_cycle`` such that the last max(``min_span``, L) + L ids repeat with period L
    (at least ``min_span`` ids and one whole cycle of repetition), or 0."""
    n = len(ids)
    if n < min_span + 1:
        return 0
    a = np.asarray(ids[-(max(min_span, max_cycle) + max_cycle):], dtype=np.int64)
    m = a.size
    for L in range(1, min(max_cycle, m // 2) + 1):
        span = max(min_span, L)
        if span + L > m:
            break
        tail = a[m - span:]
        if np.array_equal(tail, a[m - span - L:m - L]):
            return L
    return 0


class ThinkSpan:
    """Where a generation stands relative to its think span, from the text written so far."""

    def __init__(self, open_tag: str = "<think>", close_tag: str = "</think>", started: bool = False, budget: int = -1,
                 watch_loop: bool = False):
        self.open_tag, self.close_tag = open_tag, close_tag
        self.started, self.budget, self.watch_loop = started, budget, watch_loop
        self.ids_inside = 0
        self.closed = False
        self.forced = False
        self.first_inside: Optional[int] = None         # index in the generated ids where the span began

    @property
    def active(self) -> bool:
        return self.budget >= 0 or self.watch_loop

    def inside(self, text: str) -> bool:
        if self.closed:
            return False
        if self.close_tag in text:
            self.closed = True
            return False
        return self.started or self.open_tag in text

    def note(self, text: str, n_generated: int) -> None:
        """Call after every generated id with the text so far."""
        if self.inside(text):
            if self.first_inside is None:
                self.first_inside = max(0, n_generated - 1)
            self.ids_inside += 1

    def force_close(self, text: str) -> bool:
        """True once: the span is open and has used its budget (a budget of 0 closes it before its first id)."""
        if self.budget < 0 or self.forced or not self.inside(text):
            return False
        if self.ids_inside >= self.budget:
            self.forced = True
            return True
        return False

    def looping(self, text: str, generated: Sequence[int]) -> int:
        """Cycle length when the open span repeats itself, else 0 (checked every 32 ids: the scan is not free)."""
        if not self.watch_loop or self.first_inside is None or not self.inside(text):
            return 0
        if self.ids_inside < MIN_SPAN + 1 or self.ids_inside % 32:
            return 0
        return find_loop(generated[self.first_inside:])
