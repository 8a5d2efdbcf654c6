"""``POST /v1/systemone`` answered by a generative model: the decision models' request (a state and questions of type
``choice``, ``score`` or ``noul``) asked as a chat whose reply a JSON schema holds, and answered in the decision models'
body with their formulas.

The schema text goes in the system message and the state in the user message.  The reply is one JSON object with one
member a question; each question is one pick of the structured-output walk, and the row that pick reads is the question's
evidence: the logit of the token each option's remaining text starts with, read where the walk picks
(``Request.pick_rows`` in ``serve/worker.py``).  Those logits are the options' scores:

* probabilities: a softmax in f32 over the question's options only, each then the f64 of that f32; every printed number
  is ``round(x, 4)``;
* ``choice``: the model's own pick; ``confidence`` ``max(0, (p_max - u) / (1 - u))`` with ``u`` the uniform probability;
* ``score``: ``sum(i * p_i)``; ``confidence`` ``max(0, 1 - dist / dist_uniform)`` with ``dist`` the mean distance of the
  levels to the most probable one and ``dist_uniform`` that of the uniform distribution to the middle level;
* ``noul``: the probability of ``true``.

Options that one token does not tell apart (two start with the same token once their shared prefix is written) are asked
by letter: the enum holds ``A``, ``B``, ... in option order, the schema text shows each beside its option, and the answer
names the options, never a letter.  More such options than 26 letters is a 400.

Counterpart of the reference's ``crates/serve/src/systemone.rs`` (the route on a generative seat),
``crates/decision/src/request.rs`` (the request's checks) and ``crates/decision/src/answer.rs`` (the formulas and the
body's shape).
"""
from __future__ import annotations

import dataclasses
import json
import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

KINDS = ("noul", "choice", "score")
SCORE_LEVELS = (2, 10)
LETTERS = "ABCDEFGHIJKLMNOPQRSTUVWXYZ"


class SystemOneError(ValueError):
    """A request this route refuses; ``status`` is the HTTP answer (400 unless the server lacks the input's kind: 501)."""

    def __init__(self, message: str, status: int = 400):
        super().__init__(message)
        self.status = status


@dataclasses.dataclass
class Question:
    id: str
    kind: str
    instructions: Optional[str]
    options: List[str]                      # choice: option ids in request order; score: "0".."n-1"; noul: true, false
    texts: List[str]                        # what each option means, shown in the schema text
    literals: List[str] = dataclasses.field(default_factory=list)    # each option as the reply writes it
    by_letter: bool = False


def read_request(body: Any) -> Tuple[str, List[Question]]:
    """The state as text and the questions in request order; a refusal names the question."""
    if not isinstance(body, dict):
        raise SystemOneError("the body is not an object")
    if "state" not in body:
        raise SystemOneError("state is required")
    qs = body.get("questions")
    if not isinstance(qs, dict) or not qs:
        raise SystemOneError("at least one question is required")
    if body.get("videos"):
        raise SystemOneError("the request carries videos; this server does not support video input for decisions", 501)
    if body.get("images") or _has_image_part(body["state"]):
        raise SystemOneError("the request carries images; this server has no image encoder", 501)
    out: List[Question] = []
    for qid, q in qs.items():
        def refuse(what: str):
            return SystemOneError(f"question {qid!r}: {what}")
        if not isinstance(q, dict):
            raise refuse("the question is not an object")
        kind = q.get("type")
        if kind not in KINDS:
            raise refuse("type must be noul, choice, or score")
        crit = q.get("criteria")
        ins = q.get("instructions")
        if ins is not None and not isinstance(ins, str):
            ins = json.dumps(ins, ensure_ascii=False)
        if kind != "noul" and not crit:
            raise refuse("criteria must not be empty")
        if kind == "choice":
            if not isinstance(crit, dict):
                raise refuse("choice criteria must be an object of option id to description")
            out.append(Question(qid, kind, ins, list(crit), [_text(v) for v in crit.values()]))
        elif kind == "score":
            if not isinstance(crit, list):
                raise refuse("score criteria must be an array of level descriptions")
            if not SCORE_LEVELS[0] <= len(crit) <= SCORE_LEVELS[1]:
                raise refuse(f"criteria must be an array of {SCORE_LEVELS[0]} to {SCORE_LEVELS[1]} levels, not {len(crit)}")
            out.append(Question(qid, kind, ins, [str(i) for i in range(len(crit))], [_text(v) for v in crit]))
        else:
            if crit and not isinstance(crit, dict):
                raise refuse("noul criteria must be an object (overriding true or false), or empty")
            crit = crit or {}
            out.append(Question(qid, kind, ins, ["true", "false"], [_text(crit.get("true", "yes")), _text(crit.get("false", "no"))]))
    state = body["state"]
    return (state if isinstance(state, str) else json.dumps(state, ensure_ascii=False)), out


def _text(v: Any) -> str:
    return v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)


def _has_image_part(state: Any) -> bool:
    msgs = state.get("messages") if isinstance(state, dict) else state
    if not isinstance(msgs, list):
        return False
    for m in msgs:
        c = m.get("content") if isinstance(m, dict) else None
        if isinstance(c, list) and any(isinstance(p, dict) and p.get("type") == "image_url" for p in c):
            return True
    return False


def _common(texts: Sequence[str]) -> str:
    first = texts[0]
    k = len(first)
    for t in texts[1:]:
        j = 0
        while j < k and j < len(t) and first[j] == t[j]:
            j += 1
        k = j
    return first[:k]


def first_tokens(literals: Sequence[str], encode: Callable[[str], List[int]]) -> Optional[List[int]]:
    """The token each option's text starts with once the prefix all of them share is written, or None when two options
    start with the same one (or one has nothing left to write) and a single pick cannot tell them apart."""
    lead = len(_common(literals))
    toks = []
    for lit in literals:
        ids = encode(lit[lead:]) if lit[lead:] else []
        if not ids:
            return None
        toks.append(int(ids[0]))
    return toks if len(set(toks)) == len(toks) else None


def plan(questions: List[Question], encode: Callable[[str], List[int]]) -> Dict[str, Any]:
    """Decide how each question is written (its options' own ids, or letters) and build the reply's schema."""
    props: Dict[str, Any] = {}
    for q in questions:
        if q.kind == "choice":
            q.literals = [json.dumps(o, ensure_ascii=False) for o in q.options]
            if len(q.options) > 1 and first_tokens(q.literals, encode) is None:
                if len(q.options) > len(LETTERS):
                    raise SystemOneError(f"question {q.id!r}: {len(q.options)} options that one token does not tell apart are more "
                                         f"than the {len(LETTERS)} letters they could be asked by")
                q.by_letter = True
                q.literals = [json.dumps(LETTERS[i]) for i in range(len(q.options))]
                if first_tokens(q.literals, encode) is None:
                    raise SystemOneError(f"question {q.id!r}: the letters do not tokenize apart on this vocabulary")
            props[q.id] = {"enum": [json.loads(lit) for lit in q.literals]}
        elif q.kind == "score":
            q.literals = list(q.options)
            props[q.id] = {"enum": [int(o) for o in q.options]}
        else:
            q.literals = ["true", "false"]
            props[q.id] = {"type": "boolean"}
    return {"type": "object", "properties": props, "required": [q.id for q in questions], "additionalProperties": False}


def schema_text(questions: List[Question]) -> str:
    """The system message: what each member of the reply means and which values it takes."""
    lines = ["Answer every question about the state the user gives with one JSON object: one member a question, in this "
             "order, each holding one of the values listed for it."]
    for q in questions:
        head = f"- {json.dumps(q.id, ensure_ascii=False)} ({q.kind})" + (f": {q.instructions}" if q.instructions else "")
        if q.kind == "choice":
            shown = [(LETTERS[i] if q.by_letter else o) for i, o in enumerate(q.options)]
            vals = "; ".join((f"{s} = {o}: {t}" if q.by_letter else f"{o}: {t}") for s, o, t in zip(shown, q.options, q.texts))
            lines.append(f"{head}\n  options: {vals}")
        elif q.kind == "score":
            lines.append(f"{head}\n  levels: " + "; ".join(f"{o} = {t}" for o, t in zip(q.options, q.texts)))
        else:
            lines.append(f"{head}\n  true = {q.texts[0]}; false = {q.texts[1]}")
    return "\n".join(lines)


def value_starts(questions: List[Question], reply: Dict[str, Any]) -> Dict[str, int]:
    """Where each question's value starts in the canonical reply text (``{"a": v, "b": w}``)."""
    pos, out = 1, {}
    for i, q in enumerate(questions):
        pos += len(json.dumps(q.id, ensure_ascii=False)) + 2
        out[q.id] = pos
        pos += len(json.dumps(reply[q.id], ensure_ascii=False)) + 2
    return out


def probabilities(scores: Sequence[float]) -> List[float]:
    s = np.asarray(scores, dtype=np.float32)
    if not np.all(np.isfinite(s)):
        raise SystemOneError("a score is not finite: the model could not evaluate the decision", 500)
    e = np.exp(s - s.max(), dtype=np.float32)
    return [float(x) for x in (e / e.sum(dtype=np.float32)).astype(np.float32)]


def confidence_choice(p: Sequence[float]) -> float:
    if len(p) < 2:
        return 1.0
    u = 1.0 / len(p)
    return max(0.0, (max(p) - u) / (1.0 - u))


def confidence_score(p: Sequence[float]) -> float:
    n = len(p)
    if n < 2:
        return 1.0
    mode = 0
    for i, x in enumerate(p):
        if x > p[mode]:
            mode = i
    dist = sum(x * abs(i - mode) for i, x in enumerate(p))
    dist_uniform = sum(abs(i - (n - 1) / 2.0) / n for i in range(n))
    return max(0.0, 1.0 - dist / dist_uniform)


def r4(x: float) -> float:
    return round(float(x), 4)


def answer(q: Question, picked: Any, scores: Sequence[float]) -> Dict[str, Any]:
    """One question's entry of the body from the model's pick and its options' scores (in option order)."""
    p = probabilities(scores)
    if q.kind == "choice":
        lit = json.dumps(picked, ensure_ascii=False)
        choice = q.options[q.literals.index(lit)] if lit in q.literals else q.options[int(np.argmax(p))]
        return {"type": "choice", "choice": choice, "confidence": r4(confidence_choice(p)),
                "probabilities": {o: r4(x) for o, x in zip(q.options, p)}}
    if q.kind == "score":
        return {"type": "score", "score": r4(math.fsum(i * x for i, x in enumerate(p))), "confidence": r4(confidence_score(p)),
                "legend": {o: t for o, t in zip(q.options, q.texts)}, "probabilities": {o: r4(x) for o, x in zip(q.options, p)}}
    return {"type": "noul", "noul": r4(p[0])}


def answers(questions: List[Question], document: str, rows: Sequence[Tuple[int, np.ndarray]],
            encode: Callable[[str], List[int]]) -> Dict[str, Any]:
    """Every question's entry.  ``document`` is the reply's JSON text; ``rows`` the ``(offset in the document, logits
    row)`` of each pick the walk made."""
    try:
        reply = json.loads(document)
    except json.JSONDecodeError:
        raise SystemOneError("the reply is not a whole JSON object: the token limit cut it", 500) from None
    if not isinstance(reply, dict) or any(q.id not in reply for q in questions):
        raise SystemOneError("the reply does not answer every question", 500)
    starts = value_starts(questions, reply)
    by_offset = {int(o): r for o, r in rows}
    out: Dict[str, Any] = {}
    for q in questions:
        if len(q.options) == 1:
            out[q.id] = answer(q, reply[q.id], [0.0])
            continue
        toks = first_tokens(q.literals, encode)
        at = starts[q.id] + len(_common(q.literals))
        row = by_offset.get(at)
        if toks is None or row is None:
            raise SystemOneError(f"question {q.id!r}: no pick was read where its options part", 500)
        out[q.id] = answer(q, reply[q.id], [float(row[t]) for t in toks])
    return out
