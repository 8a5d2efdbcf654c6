"""Structured output as a program over text segments, walked token by token.

A JSON schema (the subset below) compiles to a list of segments: literal text, a JSON string, a JSON number, a fork
among segment lists, and an array that repeats its item.  A :class:`Walk` keeps the set of places the output may be at
(one per fork option that still matches what was written, like the heads of an NFA) and answers, for a candidate token's
text, whether some place accepts all of it.  Where every place agrees that literal text comes next the walk names it
(:meth:`Walk.forced_text`): the server then takes the canonical tokens of that text without reading the logits at all
(the jump arm) -- keys, punctuation and closing brackets of an object cost no sampling.  Once the program is spent only
an end-of-generation token is allowed.

The output is canonical JSON: ``", "`` and ``": "`` separators, no other whitespace, properties in schema order.

Schema subset: ``type`` object (its ``required`` properties in order, then each optional one in order, each of which may
be left out) / array (``items``, ``minItems``, ``maxItems``) / string (``maxLength``, ``enum``) / number / integer /
boolean / null, ``const``, ``enum``, ``anyOf`` / ``oneOf``, a ``$ref`` into the schema itself (``#/$defs/...``, not
recursive).  Any other keyword (``pattern``, ``minLength``, ``minimum``, ``allOf``, ...), a ``$ref`` outside the schema,
more than 4,096 schemas or 128 nested levels raise :class:`Unsupported` naming it, and the caller falls back to the
prefix validator of ``serve/chat.py``.

The reference's counterpart is ``crates/serve/src/constrain/program.rs`` (parts, compile, walk with heads, the fixed-next
shortcut); this one walks characters of token texts instead of precompiled id tries.
"""
from __future__ import annotations

import json
import re
from typing import Any, List, Optional, Sequence, Set, Tuple

_NUM_FULL = re.compile(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?\Z")
_NUM_PREFIX = re.compile(r"-?((0|[1-9]\d*)((\.\d*)|((\.\d+)?[eE][+-]?\d*))?)?\Z")
_INT_FULL = re.compile(r"-?(0|[1-9]\d*)\Z")
_INT_PREFIX = re.compile(r"-?(0|[1-9]\d*)?\Z")
_ESCAPES = '"\\/bfnrt'


class Unsupported(ValueError):
    """The schema uses something the segment program does not express."""


def _merge(segs: List[tuple]) -> Tuple[tuple, ...]:
    out: List[tuple] = []
    for s in segs:
        if s[0] == "lit" and not s[1]:
            continue
        if s[0] == "lit" and out and out[-1][0] == "lit":
            out[-1] = ("lit", out[-1][1] + s[1])
        else:
            out.append(s)
    return tuple(out)


_ANNOTATIONS = ("title", "description", "default", "examples", "$schema", "$id", "$comment", "$defs", "definitions", "strict", "name")
_KEYWORDS = {"object": ("properties", "required", "additionalProperties"), "array": ("items", "minItems", "maxItems"),
             "string": ("maxLength",), "number": (), "integer": (), "boolean": (), "null": ()}
MAX_SCHEMAS, MAX_DEPTH = 4096, 128


def compile_schema(schema: Any, root: Any = None, _depth: int = 0, _count: Optional[List[int]] = None,
                   _refs: Tuple[str, ...] = ()) -> Tuple[tuple, ...]:
    """Schema -> segments.  ``root``: the document ``$ref`` pointers resolve in (the schema itself at the top)."""
    if not isinstance(schema, dict):
        raise Unsupported("a schema is an object")
    root = schema if root is None else root
    _count = [0] if _count is None else _count
    _count[0] += 1
    if _count[0] > MAX_SCHEMAS or _depth > MAX_DEPTH:
        raise Unsupported(f"the schema writes out to more than {MAX_SCHEMAS} schemas or past {MAX_DEPTH} nested levels")
    sub = lambda s_, refs=_refs: compile_schema(s_, root, _depth + 1, _count, refs)       # noqa: E731
    if "$ref" in schema:
        ref = schema["$ref"]
        if not isinstance(ref, str) or not ref.startswith("#/"):
            raise Unsupported(f"$ref {ref!r} points outside the schema")
        if ref in _refs:
            raise Unsupported(f"$ref {ref!r} is recursive")
        node: Any = root
        for part in ref[2:].split("/"):
            part = part.replace("~1", "/").replace("~0", "~")
            if not isinstance(node, dict) or part not in node:
                raise Unsupported(f"$ref {ref!r} names nothing in the schema")
            node = node[part]
        extra = [k for k in schema if k != "$ref" and k not in _ANNOTATIONS]
        if extra:
            raise Unsupported(f"{extra[0]!r} beside a $ref")
        return sub(node, _refs + (ref,))
    if "const" in schema:
        return (("lit", json.dumps(schema["const"], ensure_ascii=False)),)
    if "enum" in schema:
        opts = schema["enum"]
        if not isinstance(opts, list) or not opts:
            raise Unsupported("enum takes a non-empty list")
        return (("alt", tuple((("lit", json.dumps(v, ensure_ascii=False)),) for v in opts)),)
    for word in ("anyOf", "oneOf"):
        if word in schema:
            if not isinstance(schema[word], list) or not schema[word]:
                raise Unsupported(f"{word} takes a non-empty list")
            return (("alt", tuple(sub(s_) for s_ in schema[word])),)
    t = schema.get("type")
    if isinstance(t, list):
        return (("alt", tuple(sub({**schema, "type": x}) for x in t)),)
    if t not in _KEYWORDS:
        raise Unsupported(f"schema type {t!r}")
    unknown = [k for k in schema if k != "type" and k not in _ANNOTATIONS and k not in _KEYWORDS[t]]
    if unknown:
        raise Unsupported(f"the keyword {unknown[0]!r} is outside the served subset")
    if t == "object":
        props = schema.get("properties")
        if not isinstance(props, dict):
            raise Unsupported("an object needs its properties listed")
        if schema.get("additionalProperties") not in (None, False):
            raise Unsupported("additionalProperties other than false")
        req = schema.get("required", [])
        if not isinstance(req, list) or any(r not in props for r in req):
            raise Unsupported("required names a property the object does not list")
        member = lambda key, lead: [("lit", lead + json.dumps(key, ensure_ascii=False) + ": ")] + list(sub(props[key]))     # noqa: E731
        need = [k for k in props if k in req]
        optional = [k for k in props if k not in req]
        segs: List[tuple] = [("lit", "{")]
        for i, key in enumerate(need):
            segs += member(key, ", " if i else "")

        def tail(keys) -> List[tuple]:
            """Optional members after something was written: each may be left out."""
            out: List[tuple] = []
            for key in keys:
                out.append(("alt", (_merge(member(key, ", ")), ())))
            return out
        if need or not optional:
            segs += tail(optional)
        else:
            # nothing required: the first member written takes no comma, so fork on which optional one comes first
            firsts = [_merge(member(key, "") + tail(optional[i + 1:])) for i, key in enumerate(optional)]
            segs.append(("alt", tuple(firsts) + ((),)))
        segs.append(("lit", "}"))
        return _merge(segs)
    if t == "array":
        item = sub(schema.get("items") if "items" in schema else _raise("an array needs items"))
        lo, hi = int(schema.get("minItems", 0)), schema.get("maxItems")
        return (("lit", "["), ("arr", item, lo, None if hi is None else int(hi), 0))
    if t == "string":
        return (("str", schema.get("maxLength")),)
    if t == "number":
        return (("num", False),)
    if t == "integer":
        return (("num", True),)
    if t == "boolean":
        return (("alt", ((("lit", "true"),), (("lit", "false"),))),)
    return (("lit", "null"),)


def _raise(msg: str):
    raise Unsupported(msg)


Head = Tuple[Tuple[tuple, ...], int, Any]      # (segments, index, state inside the segment)


def _start(seg: tuple) -> Any:
    return {"lit": 0, "str": (0, 0), "num": "", "raw": 0}.get(seg[0])


def _closure(heads) -> Set[Head]:
    """Expand forks and arrays until every head stands on literal text, a string, a number or the end."""
    out: Set[Head] = set()
    todo = list(heads)
    while todo:
        segs, i, st = todo.pop()
        if i >= len(segs):
            out.add((segs, i, None))
            continue
        s = segs[i]
        if s[0] == "alt":
            for opt in s[1]:
                ns = tuple(opt) + segs[i + 1:]
                todo.append((ns, 0, _start(ns[0]) if ns else None))
        elif s[0] == "arr":
            _, item, lo, hi, count = s
            rest = segs[i + 1:]
            if count >= lo:
                ns = _merge([("lit", "]")] + list(rest))
                todo.append((ns, 0, 0))
            if hi is None or count < hi:
                ns = _merge([("lit", ", " if count else "")] + list(item)) + (("arr", item, lo, hi, count + 1),) + rest
                todo.append((ns, 0, _start(ns[0])))
        else:
            out.add((segs, i, st))
    return out


def _next(segs, i) -> Set[Head]:
    return _closure([(segs, i + 1, _start(segs[i + 1]) if i + 1 < len(segs) else None)])


def _feed(head: Head, ch: str) -> Set[Head]:
    segs, i, st = head
    if i >= len(segs):
        return set()
    s = segs[i]
    if s[0] == "lit":
        if s[1][st] != ch:
            return set()
        return _next(segs, i) if st + 1 == len(s[1]) else {(segs, i, st + 1)}
    if s[0] == "str":
        phase, n = st
        if phase == 0:
            return {(segs, i, (1, 0))} if ch == '"' else set()
        if phase == 2:
            return {(segs, i, (1, n + 1))} if ch in _ESCAPES else set()
        if ch == '"':
            return _next(segs, i)
        if ch == "\\":
            return {(segs, i, (2, n))}
        if ord(ch) < 0x20 or (s[1] is not None and n + 1 > s[1]) or (ch == "<" and len(s) > 2 and s[2]):
            return set()
        return {(segs, i, (1, n + 1))}
    if s[0] == "raw":
        # one line of bare text inside a call's markup: no line break and no "<" (which could open or close a tag)
        if ch not in "\n\r<" and ord(ch) >= 0x20:
            return {(segs, i, 1)}
        out_raw: Set[Head] = set()
        for h in _next(segs, i):
            out_raw |= _feed(h, ch)
        return out_raw
    if s[0] == "num":
        full, prefix = (_INT_FULL, _INT_PREFIX) if s[1] else (_NUM_FULL, _NUM_PREFIX)
        cand = st + ch
        if prefix.match(cand) and len(cand) <= 40:
            return {(segs, i, cand)}
        if full.match(st):                       # the number is whole: this character belongs to what follows
            out: Set[Head] = set()
            for h in _next(segs, i):
                out |= _feed(h, ch)
            return out
        return set()
    return set()


class Walk:
    def __init__(self, program: Tuple[tuple, ...]):
        self.heads: Set[Head] = _closure([(program, 0, _start(program[0]) if program else None)])

    def _after(self, heads: Set[Head], text: str) -> Set[Head]:
        for ch in text:
            nxt: Set[Head] = set()
            for h in heads:
                nxt |= _feed(h, ch)
            heads = nxt
            if not heads:
                break
        return heads

    def accepts(self, piece: str) -> bool:
        return bool(piece) and bool(self._after(self.heads, piece))

    def take(self, piece: str) -> None:
        self.heads = self._after(self.heads, piece)

    @property
    def dead(self) -> bool:
        return not self.heads

    @property
    def spent(self) -> bool:
        """The output so far is a whole value (a number at the very end counts when it is whole)."""
        for segs, i, st in self.heads:
            if i >= len(segs):
                return True
            if i == len(segs) - 1 and segs[i][0] == "num" and (_INT_FULL if segs[i][1] else _NUM_FULL).match(st):
                return True
        return False

    def forced_text(self) -> str:
        """Literal text that every head writes next ('' when they disagree or stand in a string or number)."""
        texts = []
        for segs, i, st in self.heads:
            if i >= len(segs) or segs[i][0] != "lit":
                return ""
            texts.append(segs[i][1][st:])
        if not texts:
            return ""
        common = texts[0]
        for t in texts[1:]:
            k = 0
            while k < len(common) and k < len(t) and common[k] == t[k]:
                k += 1
            common = common[:k]
        return common


class ProgramConstraint:
    """The request-side face: the same ``allowed`` / ``done`` / ``closed`` calls as the prefix validator, answered by a
    walk that follows the text written so far, plus ``forced_text`` for the jump arm."""

    def __init__(self, schema: dict):
        self.schema = schema
        self.program = compile_schema(schema)
        self._text = ""
        self._walk = Walk(self.program)

    def _at(self, text: str) -> Walk:
        if text != self._text:
            if text.startswith(self._text):
                self._walk.take(text[len(self._text):])
            else:
                self._walk = Walk(self.program)
                self._walk.take(text)
            self._text = text
        return self._walk

    def allowed(self, text: str, piece: str) -> bool:
        return self._at(text).accepts(piece)

    def done(self, text: str) -> bool:
        return self._at(text).spent

    def closed(self, text: str) -> bool:
        w = self._at(text)
        return w.spent and all(i >= len(segs) for segs, i, _ in w.heads)

    def forced_text(self, text: str) -> str:
        return self._at(text).forced_text()


FRAMINGS = ("hermes", "qwenxml", "glmxml", "dsml", "dsml_spaced")


def call_opener(framing: str) -> str:
    """The text that opens a call (or a block of calls) in a framing."""
    if framing in ("dsml", "dsml_spaced"):
        from .chat import _dsml_tags
        return _dsml_tags(framing == "dsml_spaced")[0]
    return "<tool_call>"


def _no_lt(segs: Sequence[tuple]) -> Tuple[tuple, ...]:
    """The same program inside a tool call's markup, where the reply is scanned for tags: a free string takes no ``<``,
    and a ``<`` in fixed text (a constant, an option, a property name) is written as its JSON escape."""
    out: List[tuple] = []
    for s in segs:
        if s[0] == "lit":
            out.append(("lit", s[1].replace("<", "\\u003c")))
        elif s[0] == "str":
            out.append(("str", s[1], True))
        elif s[0] == "alt":
            out.append(("alt", tuple(_no_lt(o) for o in s[1])))
        elif s[0] == "arr":
            out.append(("arr", _no_lt(s[1])) + tuple(s[2:]))
        else:
            out.append(s)
    return tuple(out)


def _tool_fn(tool: Any) -> Tuple[str, dict]:
    fn = tool.get("function", tool) if isinstance(tool, dict) else None
    if not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
        raise Unsupported("a tool needs a function with a name")
    params = fn.get("parameters")
    if params is None or params == {}:
        params = {"type": "object", "properties": {}}
    return fn["name"], params


def _call_segments(name: str, params: dict, framing: str) -> Tuple[tuple, ...]:
    """One call of ``name`` in the template's framing, its arguments held to ``params``."""
    if not isinstance(params, dict) or "anyOf" in params or "oneOf" in params or "$ref" in params:
        raise Unsupported(f"the forced tool {name!r} has parameters with a root anyOf or $ref")
    if params.get("type") != "object":
        raise Unsupported(f"the forced tool {name!r} has parameters that are not an object")
    if "<" in name or "\n" in name:
        raise Unsupported(f"the tool name {name!r} cannot be written inside a call's markup")
    if framing == "hermes":
        head = '<tool_call>\n{"name": ' + json.dumps(name, ensure_ascii=False) + ', "arguments": '
        return _merge([("lit", head)] + list(_no_lt(compile_schema(params))) + [("lit", "}\n</tool_call>")])
    # the <function=...><parameter=...> markup: a value on lines of its own, a string bare, anything else as JSON
    props = params.get("properties") or {}
    req = params.get("required", [])
    if not isinstance(props, dict) or not isinstance(req, list) or any(r not in props for r in req):
        raise Unsupported(f"the forced tool {name!r} lists its properties and required names")

    def value(schema: Any) -> List[tuple]:
        if isinstance(schema, dict) and schema.get("type") == "string" and "enum" not in schema and "const" not in schema:
            if any(k not in _ANNOTATIONS and k not in ("type", "maxLength") for k in schema):
                raise Unsupported("a string keyword outside the served subset")
            return [("raw",)]
        if isinstance(schema, dict) and isinstance(schema.get("enum"), list) and all(isinstance(v, str) for v in schema["enum"]):
            if any("<" in v or "\n" in v for v in schema["enum"]):
                raise Unsupported("a raw option with a < or a line break")
            return [("alt", tuple((("lit", v),) for v in schema["enum"]))]
        if isinstance(schema, dict) and ("anyOf" in schema or "oneOf" in schema):
            raise Unsupported("an anyOf in a tool argument written raw")
        return list(compile_schema(schema, params))

    def member(key: str) -> List[tuple]:
        if "<" in key or ">" in key or "\n" in key:
            raise Unsupported(f"the property name {key!r} cannot be written inside a call's markup")
        return [("lit", f"<parameter={key}>\n")] + value(props[key]) + [("lit", "\n</parameter>\n")]
    if framing in ("dsml", "dsml_spaced"):
        # a block of one invoke; a parameter says whether its value is bare text (string="true") or JSON
        from .chat import _dsml_tags
        b_open, b_close, i_open, i_close, p_open, p_close = _dsml_tags(framing == "dsml_spaced")
        if '"' in name:
            raise Unsupported(f"the tool name {name!r} cannot be written inside a call's markup")

        def param(key: str) -> List[tuple]:
            if '"' in key or "<" in key or "\n" in key:
                raise Unsupported(f"the property name {key!r} cannot be written inside a call's markup")
            v = value(props[key])
            sch = props[key]
            bare = isinstance(sch, dict) and ((sch.get("type") == "string" and "enum" not in sch and "const" not in sch)
                                              or (isinstance(sch.get("enum"), list) and all(isinstance(x, str) for x in sch["enum"])))
            flag = "true" if bare else "false"
            return [("lit", f'{p_open}{key}" string="{flag}">')] + v + [("lit", f"{p_close}\n")]
        segs = [("lit", f'{b_open}\n{i_open}{name}">\n')]
        for key in props:
            segs += param(key) if key in req else [("alt", (_merge(param(key)), ()))]
        segs.append(("lit", f"{i_close}\n{b_close}"))
        return _merge(segs)
    if framing == "glmxml":
        # <tool_call>NAME, then an <arg_key> / <arg_value> pair a member, a string bare (it holds no "<")
        def pair(key: str) -> List[tuple]:
            if "<" in key or "\n" in key:
                raise Unsupported(f"the property name {key!r} cannot be written inside a call's markup")
            return [("lit", f"<arg_key>{key}</arg_key>\n<arg_value>")] + value(props[key]) + [("lit", "</arg_value>\n")]
        segs = [("lit", f"<tool_call>{name}\n")]
        for key in props:
            segs += pair(key) if key in req else [("alt", (_merge(pair(key)), ()))]
        segs.append(("lit", "</tool_call>"))
        return _merge(segs)
    segs: List[tuple] = [("lit", f"<tool_call>\n<function={name}>\n")]
    for key in props:
        segs += member(key) if key in req else [("alt", (_merge(member(key)), ()))]
    segs.append(("lit", "</function>\n</tool_call>"))
    return _merge(segs)


def forced_call_program(tools: Any, choice: Any, framing: str) -> Tuple[tuple, ...]:
    """The program of a reply that must be one tool call: ``choice`` is ``"required"`` (any of ``tools``) or a function's
    name.  Raises :class:`Unsupported` naming what cannot be forced (the caller answers 400 with it)."""
    if framing not in FRAMINGS:
        raise Unsupported(f"a forced call is not written in this template's framing ({framing})")
    if not isinstance(tools, list) or not tools:
        raise Unsupported("a forced tool_choice needs tools")
    fns = [_tool_fn(t) for t in tools]
    if choice != "required":
        fns = [f for f in fns if f[0] == choice]
        if not fns:
            raise Unsupported(f"tool_choice names {choice!r}, which is not among the tools")
    calls = [_call_segments(n, p, framing) for n, p in fns]
    return calls[0] if len(calls) == 1 else (("alt", tuple(calls)),)


class ForcedCall(ProgramConstraint):
    """A reply held to one tool call.  While a think span the template opened is still open the model writes freely
    (it may not end there); the call starts after the span's close, with the line breaks a model puts between them."""

    def __init__(self, program: Tuple[tuple, ...], think_open: bool = False, close_tag: str = "</think>"):
        self.schema = None
        self.program = (("alt", ((("lit", "\n\n"),), (("lit", "\n"),), ())),) + tuple(program) if think_open else tuple(program)
        self.think_open, self.close_tag = think_open, close_tag
        self._text = ""
        self._walk = Walk(self.program)

    def _split(self, text: str) -> Optional[str]:
        """The part of the output the program governs (None: still inside the think span)."""
        if not self.think_open:
            return text
        at = text.find(self.close_tag)
        return None if at < 0 else text[at + len(self.close_tag):]

    def allowed(self, text: str, piece: str) -> bool:
        own = self._split(text)
        if own is None:
            whole = text + piece
            at = whole.find(self.close_tag)
            if at < 0:
                return True
            rest = whole[at + len(self.close_tag):]          # the piece closes the span: what follows it starts the call
            return not rest or Walk(self.program).accepts(rest)
        return super().allowed(own, piece)

    def done(self, text: str) -> bool:
        own = self._split(text)
        return own is not None and super().done(own)

    def closed(self, text: str) -> bool:
        own = self._split(text)
        return own is not None and super().closed(own)

    def forced_text(self, text: str) -> str:
        own = self._split(text)
        return "" if own is None else super().forced_text(own)


class AfterThink:
    """A document constraint behind a think span the template opened: the span is closed at once (the server writes the
    closing tag for the model), and the inner constraint governs what follows it, after the line breaks a model puts
    between the two."""

    def __init__(self, inner, close_tag: str = "</think>"):
        self.inner, self.close_tag = inner, close_tag

    def _own(self, text: str) -> Optional[str]:
        at = text.find(self.close_tag)
        return None if at < 0 else text[at + len(self.close_tag):]

    def allowed(self, text: str, piece: str) -> bool:
        own = self._own(text)
        if own is None:
            return self.close_tag.startswith(text + piece) or (text + piece).startswith(self.close_tag)
        if not own.strip("\n") and not piece.strip("\n"):
            return len(own + piece) <= 2                              # at most a blank line before the document
        lead = len(own) - len(own.lstrip("\n"))
        if not own.strip("\n"):
            piece, own = (own + piece).lstrip("\n"), ""
            return len((own + piece)) > 0 and self.inner.allowed("", piece)
        return self.inner.allowed(own[lead:], piece)

    def done(self, text: str) -> bool:
        own = self._own(text)
        return own is not None and self.inner.done(own.lstrip("\n"))

    def closed(self, text: str) -> bool:
        own = self._own(text)
        return own is not None and self.inner.closed(own.lstrip("\n"))

    def forced_text(self, text: str) -> str:
        own = self._own(text)
        inner = getattr(self.inner, "forced_text", None)
        if own is None or inner is None or (own and not own.strip("\n")):
            return ""
        return inner(own.lstrip("\n"))


class WatchedCall:
    """A free reply whose tool calls are watched: text is unconstrained until the model writes its framing's call opener;
    from there the call follows the program a forced call compiles, until it closes, and the reply is free again.  The
    reply may end anywhere outside a call and nowhere inside one."""

    def __init__(self, program: Tuple[tuple, ...], opener: str = "<tool_call>"):
        self.program = tuple(program)
        self.OPENER = opener
        self._text = ""
        self._state: Tuple[str, Optional[Walk]] = ("", None)          # (tail of the free text, walk of the open call)

    def _step(self, state, chunk: str):
        tail, walk = state
        for ch in chunk:
            if walk is not None:
                heads = walk._after(walk.heads, ch)
                if not heads:
                    return None                                        # the call left its program
                nw = Walk.__new__(Walk)
                nw.heads = heads
                walk = None if all(i >= len(segs) for segs, i, _ in heads) else nw
                continue
            tail = (tail + ch)[-len(self.OPENER):]
            if tail == self.OPENER:
                walk = Walk(self.program)
                walk.take(self.OPENER)
                tail = ""
                if walk.dead:
                    return None
        return tail, walk

    def _at(self, text: str):
        if text != self._text:
            if self._state is None and text.startswith(self._text):
                self._text = text                                      # gave up watching: stays given up while the text grows
                return None
            base, state = (self._text, self._state) if text.startswith(self._text) else ("", ("", None))
            self._state = self._step(state, text[len(base):])
            self._text = text
        return self._state

    def free(self, text: str) -> bool:
        """No call is open: the pick needs no mask (a reply that once left its program is no longer watched)."""
        state = self._at(text)
        return state is None or state[1] is None

    def allowed(self, text: str, piece: str) -> bool:
        state = self._at(text)
        return bool(piece) and (state is None or self._step(state, piece) is not None)

    def done(self, text: str) -> bool:
        return self.free(text)

    def closed(self, text: str) -> bool:
        return False                                                   # the reply ends when the model ends it

    def forced_text(self, text: str) -> str:
        state = self._at(text)
        return state[1].forced_text() if state is not None and state[1] is not None else ""


def watched_calls(tools: Any, framing: str) -> Optional[WatchedCall]:
    """The watch over a free reply's calls, or None where the calls stay unwatched: a framing the programs do not write,
    or a tool schema outside the served subset."""
    try:
        program = forced_call_program(tools, "required", framing)
    except Unsupported:
        return None
    return WatchedCall(program, call_opener(framing))


# what the prefix validator of serve/chat.py reads beside the program's own subset (free-form objects, open additional
# properties): a keyword outside both is honoured by neither path, so the request is refused by that keyword's name
_FALLBACK_KEYWORDS = {"type", "properties", "required", "additionalProperties", "items", "minItems", "maxItems", "enum", "const",
                      "anyOf", "oneOf", "maxLength", "$ref"} | set(_ANNOTATIONS)


def unserved_keyword(schema: Any, _depth: int = 0) -> Optional[str]:
    """The first schema keyword no constraint of this server enforces (``pattern``, ``minLength``, ``minimum``, ``allOf``,
    ``minProperties``, ...), or None."""
    if not isinstance(schema, dict) or _depth > MAX_DEPTH:
        return None
    for k, v in schema.items():
        if k not in _FALLBACK_KEYWORDS:
            return k
        if k in ("properties", "$defs", "definitions") and isinstance(v, dict):
            for sub in v.values():
                bad = unserved_keyword(sub, _depth + 1)
                if bad:
                    return bad
        elif k == "items":
            bad = unserved_keyword(v, _depth + 1)
            if bad:
                return bad
        elif k in ("anyOf", "oneOf") and isinstance(v, list):
            for sub in v:
                bad = unserved_keyword(sub, _depth + 1)
                if bad:
                    return bad
    return None


def constraint_for(schema: Optional[dict]):
    """A segment program when the schema compiles to one, else None (the caller keeps its prefix validator)."""
    if not schema:
        return None
    try:
        return ProgramConstraint(schema)
    except Unsupported:
        return None
