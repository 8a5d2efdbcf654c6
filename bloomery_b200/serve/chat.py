"""Chat surface: Jinja chat templates with Hugging Face semantics, client-text guard marks,
tool-call parsers (hermes JSON, Qwen XML, Mistral, GLM XML), the reasoning split and the
structured-output constraint.

Counterparts in the reference: ``crates/jinja`` (HF-semantics subset with strict errors),
``crates/serve/src/{guard,hermes,qwenxml,glmxml,mistral,reasoning}.rs`` and
``constrain/{schema,program}.rs``.  The template engine here is jinja2's immutable sandbox
with the extras HF templates use (``raise_exception``, ``strftime_now``, ``tojson``,
loop controls).
"""
from __future__ import annotations

import datetime
import json
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

import jinja2
from jinja2.sandbox import ImmutableSandboxedEnvironment

CHATML = (
    "{% for message in messages %}{{ '<|im_start|>' + message['role'] + '\\n' + message['content'] + '<|im_end|>' + '\\n' }}"
    "{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}{% endif %}"
)

# Private-use characters bracket client text inside the rendered prompt; they are split out
# again after rendering so the tokenizer never parses control tokens inside them.
G0, G1 = "\ue000", "\ue001"


class TemplateError(ValueError):
    pass


def _raise(msg):
    raise TemplateError(str(msg))


def _env() -> ImmutableSandboxedEnvironment:
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, undefined=jinja2.StrictUndefined,
                                        extensions=["jinja2.ext.loopcontrols"])
    env.globals["raise_exception"] = _raise
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    env.filters["tojson"] = lambda v, indent=None, ensure_ascii=False: json.dumps(v, indent=indent, ensure_ascii=ensure_ascii)
    return env


class ChatTemplate:
    def __init__(self, source: Optional[str] = None, bos: str = "", eos: str = ""):
        self.source = source or CHATML
        self.bos, self.eos = bos, eos
        try:
            self.tpl = _env().from_string(self.source)
        except jinja2.TemplateSyntaxError as exc:
            raise TemplateError(f"chat template line {exc.lineno}: {exc.message}") from None

    @staticmethod
    def _guard(messages: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
        out = []
        for m in messages:
            m = dict(m)
            c = m.get("content")
            if isinstance(c, str):
                m["content"] = G0 + c + G1
            elif isinstance(c, list):          # OpenAI content parts: text parts are joined
                texts = [p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in ("text", "input_text", "output_text")]
                bad = [p.get("type") for p in c if isinstance(p, dict) and p.get("type") not in ("text", "input_text", "output_text")]
                if bad:
                    raise TemplateError(f"content part type {bad[0]!r} is not supported by this model")
                m["content"] = G0 + "".join(texts) + G1
            elif c is None:
                m["content"] = ""
            out.append(m)
        return out

    def render(self, messages: Sequence[Dict[str, Any]], tools: Optional[List[dict]] = None, add_generation_prompt: bool = True,
               **extra) -> List[Tuple[str, bool]]:
        """Render to (text, trusted) segments: template markup is trusted, client text is not."""
        try:
            s = self.tpl.render(messages=self._guard(messages), tools=tools or None, add_generation_prompt=add_generation_prompt,
                                bos_token=self.bos, eos_token=self.eos, **extra)
        except TemplateError:
            raise
        except jinja2.TemplateError as exc:
            raise TemplateError(f"chat template: {exc}") from None
        segs: List[Tuple[str, bool]] = []
        for i, part in enumerate(re.split(f"[{G0}{G1}]", s)):
            if part:
                segs.append((part, i % 2 == 0))
        return segs

    def render_text(self, messages, **kw) -> str:
        return "".join(t for t, _ in self.render(messages, **kw))


# ---------------------------------------------------------------------------------------
# reasoning split
# ---------------------------------------------------------------------------------------
def split_reasoning(text: str, open_tag: str = "<think>", close_tag: str = "</think>", started: bool = False) -> Tuple[str, str]:
    """(reasoning, content).  ``started``: the template already opened the think span."""
    if started and close_tag in text:
        r, _, c = text.partition(close_tag)
        return r.strip(), c.lstrip("\n")
    if started:
        return text.strip(), ""
    i = text.find(open_tag)
    if i < 0:
        return "", text
    j = text.find(close_tag, i)
    if j < 0:
        return text[i + len(open_tag):].strip(), text[:i]
    return text[i + len(open_tag):j].strip(), (text[:i] + text[j + len(close_tag):]).lstrip("\n")


# ---------------------------------------------------------------------------------------
# tool-call scanners
# ---------------------------------------------------------------------------------------
def _call(name: str, args: Any, idx: int) -> Dict[str, Any]:
    return {"id": f"call_{idx}", "type": "function",
            "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}}


def parse_hermes(text: str) -> Tuple[str, List[dict]]:
    """``<tool_call>{"name":..,"arguments":{..}}</tool_call>`` blocks (Hermes / Qwen2.5 / Qwen3)."""
    calls, out, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*(.*?)\s*</tool_call>", text, re.S):
        out.append(text[pos:m.start()])
        pos = m.end()
        try:
            obj = json.loads(m.group(1))
            calls.append(_call(obj["name"], obj.get("arguments", obj.get("parameters", {})), len(calls)))
        except (json.JSONDecodeError, KeyError, TypeError):
            out.append(m.group(0))
    out.append(text[pos:])
    return "".join(out).strip(), calls


def parse_qwen_xml(text: str) -> Tuple[str, List[dict]]:
    """``<tool_call><function=NAME><parameter=K>V</parameter>...</function></tool_call>`` (Qwen3-Coder)."""
    calls, out, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", text, re.S):
        out.append(text[pos:m.start()])
        pos = m.end()
        args = {}
        for p in re.finditer(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", m.group(2), re.S):
            v = p.group(2)
            try:
                args[p.group(1)] = json.loads(v)
            except json.JSONDecodeError:
                args[p.group(1)] = v
        calls.append(_call(m.group(1), args, len(calls)))
    out.append(text[pos:])
    return "".join(out).strip(), calls


def parse_glm_xml(text: str) -> Tuple[str, List[dict]]:
    """``<tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>`` (GLM-4.5+)."""
    calls, out, pos = [], [], 0
    for m in re.finditer(r"<tool_call>\s*([^\s<]+)\s*(.*?)</tool_call>", text, re.S):
        out.append(text[pos:m.start()])
        pos = m.end()
        keys = re.findall(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", m.group(2), re.S)
        args = {}
        for k, v in keys:
            try:
                args[k] = json.loads(v)
            except json.JSONDecodeError:
                args[k] = v
        calls.append(_call(m.group(1), args, len(calls)))
    out.append(text[pos:])
    return "".join(out).strip(), calls


def parse_mistral(text: str) -> Tuple[str, List[dict]]:
    """``[TOOL_CALLS][{"name":..,"arguments":..}, ...]``."""
    i = text.find("[TOOL_CALLS]")
    if i < 0:
        return text, []
    try:
        arr = json.loads(text[i + len("[TOOL_CALLS]"):].strip())
        calls = [_call(o["name"], o.get("arguments", {}), k) for k, o in enumerate(arr if isinstance(arr, list) else [arr])]
        return text[:i].strip(), calls
    except (json.JSONDecodeError, KeyError, TypeError):
        return text, []


DSML = "\uff5cDSML\uff5c"          # the marker token of the DeepSeek-V3.2 / V4 tool markup: fullwidth bars around DSML


def _dsml_tags(spaced: bool):
    """(block open, block close, invoke open prefix, invoke close, parameter open prefix, parameter close) of one
    spelling: plain ``<|DSML|tool_calls>`` or the spaced one whose tags carry a space after the marker and whose block
    is ``calls``."""
    sp = " " if spaced else ""
    block = "calls" if spaced else "tool_calls"
    return (f"<{DSML}{sp}{block}>", f"</{DSML}{sp}{block}>", f"<{DSML}{sp}invoke name=\"", f"</{DSML}{sp}invoke>",
            f"<{DSML}{sp}parameter name=\"", f"</{DSML}{sp}parameter>")


def parse_dsml(text: str, spaced: Optional[bool] = None) -> Tuple[str, List[dict]]:
    """DSML tool calls (``crates/serve/src/dsml.rs`` in the reference):

        <|DSML|tool_calls>
        <|DSML|invoke name="NAME">
        <|DSML|parameter name="KEY" string="true">RAW TEXT</|DSML|parameter>
        <|DSML|parameter name="KEY" string="false">JSON</|DSML|parameter>
        </|DSML|invoke>
        </|DSML|tool_calls>

    (bars are the fullwidth ones).  Arguments become a JSON object in parameter order; a ``string="false"`` value that
    is not valid JSON is kept as a string.  A block that does not parse, or is still open at the end, stays content as
    raw text.  ``spaced`` picks the spelling; None reads whichever the text opens with, never both."""
    if spaced is None:
        spaced = _dsml_tags(True)[0] in text and _dsml_tags(False)[0] not in text
    b_open, b_close, i_open, i_close, p_open, p_close = _dsml_tags(spaced)
    calls, out, pos = [], [], 0
    while True:
        i = text.find(b_open, pos)
        if i < 0:
            break
        j = text.find(b_close, i)
        if j < 0:
            break                                  # an open block at the end of the text is content
        body = text[i + len(b_open):j]
        got = _dsml_block(body, i_open, i_close, p_open, p_close, len(calls))
        lead = text[pos:i]
        if got is None:
            out.append(text[pos:j + len(b_close)])
        else:
            out.append(lead[:-2] if lead.endswith("\n\n") else lead)      # the template writes two newlines before a block
            calls.extend(got)
        pos = j + len(b_close)
    out.append(text[pos:])
    return "".join(out).strip(), calls


def _dsml_block(body: str, i_open, i_close, p_open, p_close, first_index: int) -> Optional[List[dict]]:
    """The calls of one block's inside, or None when it is not well-formed."""
    calls, pos = [], 0
    while True:
        rest = body[pos:]
        if not rest.strip():
            return calls if calls else None
        k = body.find(i_open, pos)
        if k < 0 or body[pos:k].strip():
            return None
        q = body.find("\">", k + len(i_open))
        e = body.find(i_close, k)
        if q < 0 or e < 0 or q > e:
            return None
        name = body[k + len(i_open):q]
        inner, ipos, args = body[q + 2:e], 0, {}
        while True:
            if not inner[ipos:].strip():
                break
            a = inner.find(p_open, ipos)
            if a < 0 or inner[ipos:a].strip():
                return None
            m = re.match(r'([^"]*)" string="(true|false)">', inner[a + len(p_open):])
            if not m:
                return None
            v0 = a + len(p_open) + m.end()
            v1 = inner.find(p_close, v0)
            if v1 < 0:
                return None
            raw = inner[v0:v1]
            if m.group(2) == "true":
                args[m.group(1)] = raw
            else:
                try:
                    args[m.group(1)] = json.loads(raw)
                except json.JSONDecodeError:
                    args[m.group(1)] = raw
            ipos = v1 + len(p_close)
        calls.append(_call(name, args, first_index + len(calls)))
        pos = e + len(i_close)


def parse_muse(text: str) -> Dict[str, Any]:
    """The recipient protocol with ATEM call markup (``crates/serve/src/museatem.rs`` in the reference): a turn is one
    or more messages `` to=<recipient><|message|>BODY`` ended by ``<|eom|>`` (more follow, each reopened by
    ``<|start|>assistant``) or ``<|eot|>``.  Recipient ``self`` is reasoning, ``commentary`` and ``user`` are content,
    any other name is a tool call whose body is

        <atem:function_calls><atem:invoke name="NAME"><atem:parameter name="KEY">VALUE</atem:parameter></atem:invoke></atem:function_calls>

    A value is JSON when it parses, else text.  Markup that does not parse, text that is no message open and a message
    the text ends inside go to their channel as raw text.  Returns reasoning_content / content / tool_calls."""
    reasoning, content, calls = [], [], []
    pos = 0
    head = re.compile(r"\s*(?:<\|start\|>assistant)?\s*to=([^\s<]+)<\|message\|>")
    while pos < len(text):
        m = head.match(text, pos)
        if not m:
            content.append(text[pos:])
            break
        ends = [(text.find(t, m.end()), t) for t in ("<|eom|>", "<|eot|>")]
        ends = [(i, t) for i, t in ends if i >= 0]
        end, tok = min(ends) if ends else (len(text), "")
        body, who = text[m.end():end], m.group(1)
        if who == "self":
            reasoning.append(body)
        elif who in ("commentary", "user"):
            content.append(body)
        else:
            got = _atem_calls(body, len(calls)) if tok else None
            if got is None:
                content.append(text[pos:end + len(tok)])
            else:
                calls.extend(got)
        pos = end + len(tok)
        if tok == "<|eot|>":
            content.append(text[pos:])
            break
    return {"reasoning_content": "\n".join(s.strip() for s in reasoning if s.strip()),
            "content": "\n".join(s.strip() for s in content if s.strip()), "tool_calls": calls}


def _atem_calls(body: str, first_index: int) -> Optional[List[dict]]:
    m = re.fullmatch(r"\s*<atem:function_calls>(.*)</atem:function_calls>\s*", body, re.S)
    if not m:
        return None
    calls, pos, inner = [], 0, m.group(1)
    for inv in re.finditer(r'\s*<atem:invoke name="([^"]*)">(.*?)</atem:invoke>', inner, re.S):
        if inv.start() != pos:
            return None
        args, ipos, params = {}, 0, inv.group(2)
        for prm in re.finditer(r'\s*<atem:parameter name="([^"]*)">(.*?)</atem:parameter>', params, re.S):
            if prm.start() != ipos:
                return None
            try:
                args[prm.group(1)] = json.loads(prm.group(2))
            except json.JSONDecodeError:
                args[prm.group(1)] = prm.group(2)
            ipos = prm.end()
        if params[ipos:].strip():
            return None
        calls.append(_call(inv.group(1), args, first_index + len(calls)))
        pos = inv.end()
    if inner[pos:].strip() or not calls:
        return None
    return calls


TOOL_PARSERS = {"hermes": parse_hermes, "qwenxml": parse_qwen_xml, "glmxml": parse_glm_xml, "mistral": parse_mistral,
                "dsml": lambda t: parse_dsml(t, False), "dsml_spaced": lambda t: parse_dsml(t, True),
                "muse": lambda t: (lambda r: (r["content"], r["tool_calls"]))(parse_muse(t))}


def cut_call(text: str, fmt: str = "hermes") -> Optional[Tuple[str, Optional[str], str]]:
    """A reply that stops inside a call: ``(content before the call, the call's name once it is whole else None, the
    arguments' text read so far)``; None when no call is open at the end.  JSON framing and the function/parameter markup
    are read; in another framing an open call is named with no name."""
    at = text.rfind("<tool_call>")
    if at < 0 or "</tool_call>" in text[at:]:
        return None
    before, inside = text[:at].rstrip(), text[at + len("<tool_call>"):]
    if fmt == "qwenxml":
        m = re.match(r"\s*<function=([^>\s]+)>", inside)
        if not m:
            return before, None, inside
        args = {}
        for p in re.finditer(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", inside[m.end():], re.S):
            try:
                args[p.group(1)] = json.loads(p.group(2))
            except json.JSONDecodeError:
                args[p.group(1)] = p.group(2)
        return before, m.group(1), json.dumps(args, ensure_ascii=False)
    m = re.match(r'\s*\{\s*"name"\s*:\s*"((?:[^"\\]|\\.)*)"\s*(?:,\s*"arguments"\s*:\s*)?', inside)
    if not m:
        return before, None, inside
    return before, json.loads('"' + m.group(1) + '"'), inside[m.end():]


def detect_tool_format(template_source: str) -> str:
    if "<atem:" in template_source:
        return "muse"
    if DSML in template_source:
        return "dsml_spaced" if f"<{DSML} " in template_source else "dsml"
    if "<function=" in template_source:
        return "qwenxml"
    if "<arg_key>" in template_source:
        return "glmxml"
    if "[TOOL_CALLS]" in template_source:
        return "mistral"
    return "hermes"


def parse_tool_calls(text: str, fmt: str = "hermes") -> Tuple[str, List[dict]]:
    content, calls = TOOL_PARSERS.get(fmt, parse_hermes)(text)
    if not calls and fmt != "hermes":
        content, calls = parse_hermes(text)
    return content, calls


class ToolCallStream:
    """Streams ``tool_calls`` deltas: text outside call blocks passes through at once, a call
    block is held until it closes, then emitted whole (chunking-invariant by construction)."""

    def __init__(self, fmt: str = "hermes", open_tag: str = "<tool_call>", close_tag: str = "</tool_call>"):
        if fmt in ("dsml", "dsml_spaced"):
            open_tag, close_tag = _dsml_tags(fmt == "dsml_spaced")[:2]
        self.fmt, self.open, self.close = fmt, open_tag, close_tag
        self.buf = ""
        self.n_calls = 0

    def push(self, piece: str) -> Tuple[str, List[dict]]:
        self.buf += piece
        text_out, calls = "", []
        while True:
            i = self.buf.find(self.open)
            if i < 0:
                # keep a tail that may be the start of an opening tag
                keep = 0
                for k in range(min(len(self.open) - 1, len(self.buf)), 0, -1):
                    if self.buf.endswith(self.open[:k]):
                        keep = k
                        break
                text_out += self.buf[:len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                return text_out, calls
            j = self.buf.find(self.close, i)
            if j < 0:
                text_out += self.buf[:i]
                self.buf = self.buf[i:]
                return text_out, calls
            text_out += self.buf[:i]
            block = self.buf[i:j + len(self.close)]
            _, got = parse_tool_calls(block, self.fmt)
            if not got:
                text_out += block              # a closed block that is no call stays text, as in the one-shot scan
            for c in got:
                c["id"] = f"call_{self.n_calls}"
                c["index"] = self.n_calls
                self.n_calls += 1
                calls.append(c)
            self.buf = self.buf[j + len(self.close):]

    def flush(self) -> str:
        s, self.buf = self.buf, ""
        return s


class ToolStreamError(ValueError):
    """Markup that stopped being a call after its name went out."""

    def __init__(self, name: str, why: str):
        super().__init__(f"the tool call {name!r} {why}")
        self.name = name


class ToolCallDeltas:
    """Streams a JSON-framed call (``<tool_call>{"name": .., "arguments": {..}}</tool_call>``) as the model writes it, in
    OpenAI's shape: the first delta of a call carries ``index``, ``id``, ``type`` and ``function.name`` with empty
    arguments, and ``function.arguments`` fragments follow as the text arrives, up to the brace that closes the
    arguments.  Text outside calls passes through at once, less a tail that could still become the opening tag.  A block
    that closes before its name is readable (another key order, no JSON) is scanned whole, as the one-shot parser would;
    markup that stops being a call after the name went out raises :class:`ToolStreamError`."""

    HEAD = re.compile(r'\s*\{\s*"name"\s*:\s*"((?:[^"\\]|\\.)*)"\s*,\s*"arguments"\s*:\s*')

    def __init__(self, open_tag: str = "<tool_call>", close_tag: str = "</tool_call>"):
        self.open, self.close = open_tag, close_tag
        self.tail = re.compile(r"\s*\}\s*" + re.escape(close_tag))
        self.buf = ""
        self.state = "text"
        self.n_calls = 0
        self.name = ""
        self.depth, self.in_str, self.esc = 0, False, False

    @property
    def open_call(self) -> Optional[str]:
        """The call the stream stands inside ('' while its name is not whole), None outside a call."""
        return None if self.state == "text" else (self.name if self.state != "head" else "")

    def push(self, piece: str) -> Tuple[str, List[dict]]:
        self.buf += piece
        text_out, deltas = "", []
        while True:
            if self.state == "text":
                i = self.buf.find(self.open)
                if i < 0:
                    keep = 0
                    for k in range(min(len(self.open) - 1, len(self.buf)), 0, -1):
                        if self.buf.endswith(self.open[:k]):
                            keep = k
                            break
                    text_out += self.buf[:len(self.buf) - keep]
                    self.buf = self.buf[len(self.buf) - keep:]
                    return text_out, deltas
                text_out += self.buf[:i]
                self.buf = self.buf[i + len(self.open):]
                self.state, self.name = "head", ""
            if self.state == "head":
                m = self.HEAD.match(self.buf)
                j = self.buf.find(self.close)
                if m and (j < 0 or m.end() <= j):
                    self.name = json.loads('"' + m.group(1) + '"')
                    deltas.append({"index": self.n_calls, "id": f"call_{self.n_calls}", "type": "function",
                                   "function": {"name": self.name, "arguments": ""}})
                    self.buf = self.buf[m.end():]
                    self.state, self.depth, self.in_str, self.esc = "args", 0, False, False
                elif j >= 0:
                    block = self.open + self.buf[:j + len(self.close)]           # closed before its name was readable
                    _, got = parse_hermes(block)
                    if not got:
                        text_out += block
                    for c in got:
                        c["id"], c["index"] = f"call_{self.n_calls}", self.n_calls
                        self.n_calls += 1
                        deltas.append(c)
                    self.buf = self.buf[j + len(self.close):]
                    self.state = "text"
                    continue
                else:
                    return text_out, deltas
            if self.state == "args":
                n, frag_end = 0, None
                for n, ch in enumerate(self.buf):
                    if self.depth == 0 and not self.in_str:
                        if ch.isspace():
                            continue
                        if ch not in "{[":
                            raise ToolStreamError(self.name, "has arguments that are not a JSON object")
                    if self.in_str:
                        if self.esc:
                            self.esc = False
                        elif ch == "\\":
                            self.esc = True
                        elif ch == '"':
                            self.in_str = False
                    elif ch == '"':
                        self.in_str = True
                    elif ch in "{[":
                        self.depth += 1
                    elif ch in "}]":
                        self.depth -= 1
                        if self.depth == 0:
                            frag_end = n + 1
                            break
                cut = frag_end if frag_end is not None else len(self.buf)
                frag = self.buf[:cut] if (self.depth > 0 or frag_end is not None) else ""
                if frag:
                    deltas.append({"index": self.n_calls, "function": {"arguments": frag}})
                self.buf = self.buf[cut:] if frag else self.buf
                if frag_end is None:
                    return text_out, deltas
                self.state = "tail"
            if self.state == "tail":
                m = self.tail.match(self.buf)
                if m:
                    self.buf = self.buf[m.end():]
                    self.n_calls += 1
                    self.state = "text"
                    continue
                squeezed = re.sub(r"\s+", "", self.buf)
                if ("}" + self.close).startswith(squeezed):
                    return text_out, deltas
                raise ToolStreamError(self.name, "is followed by text where its closing tag belongs")

    def flush(self) -> str:
        """What is left when the generation ends: text outside a call, or the unread head of a call."""
        s, self.buf = (self.open + self.buf if self.state == "head" else self.buf if self.state == "text" else ""), ""
        return s


# ---------------------------------------------------------------------------------------
# structured output: JSON (optionally against a schema subset) as a prefix validator
# ---------------------------------------------------------------------------------------
class JsonConstraint:
    """Keeps the output a prefix of one JSON value and, when a schema is given, of a value the
    schema subset accepts: ``type``, ``properties``, ``required``, ``items``, ``enum``,
    ``const``, ``additionalProperties: false``, ``minItems``/``maxItems``.  ``allowed`` is asked
    for every candidate piece before it is picked (masked pick), ``done`` when an end-of-turn
    token is a candidate."""

    def __init__(self, schema: Optional[dict] = None):
        self.schema = schema

    # -- a small incremental JSON scanner: returns (state, value-so-far validity) -----------
    @staticmethod
    def _scan(s: str):
        """Returns ("bad" | "open" | "closed", depth_stack) for the text as a JSON prefix."""
        stack: List[str] = []
        i, n = 0, len(s)
        expect = "value"            # value | key | colon | comma_or_end | end
        while i < n:
            c = s[i]
            if c in " \t\r\n":
                i += 1
                continue
            if expect == "end":
                return "bad", stack
            if expect in ("value", "key"):
                if expect == "key" and c != '"':
                    if c == "}" and stack and stack[-1] == "{0":
                        stack.pop()
                        expect = "comma_or_end" if stack else "end"
                        i += 1
                        continue
                    return "bad", stack
                if c == '"':
                    j = i + 1
                    while j < n:
                        if s[j] == "\\":
                            j += 2
                            continue
                        if s[j] == '"':
                            break
                        if ord(s[j]) < 0x20:
                            return "bad", stack
                        j += 1
                    if j >= n:
                        return "open", stack + ["str"]
                    i = j + 1
                    expect = "colon" if expect == "key" else ("comma_or_end" if stack else "end")
                    continue
                if c == "{":
                    stack.append("{0")
                    expect = "key"
                    i += 1
                    continue
                if c == "[":
                    stack.append("[0")
                    expect = "value"
                    i += 1
                    continue
                if c == "]" and stack and stack[-1] == "[0":
                    stack.pop()
                    expect = "comma_or_end" if stack else "end"
                    i += 1
                    continue
                m = re.match(r"-?(?:0|[1-9]\d*)(?:\.\d+)?(?:[eE][+-]?\d+)?", s[i:])
                if m and m.end() > 0:
                    j = i + m.end()
                    if j >= n:
                        return "open", stack + ["num"]
                    i = j
                    expect = "comma_or_end" if stack else "end"
                    continue
                if re.match(r"-?(?:\d+\.?|\d+\.\d+[eE][+-]?)?$", s[i:]) and s[i:] not in ("",):
                    return "open", stack + ["num"]
                for lit in ("true", "false", "null"):
                    if s.startswith(lit, i):
                        i += len(lit)
                        expect = "comma_or_end" if stack else "end"
                        break
                    if lit.startswith(s[i:]):
                        return "open", stack + ["lit"]
                else:
                    return "bad", stack
                continue
            if expect == "colon":
                if c != ":":
                    return "bad", stack
                expect = "value"
                i += 1
                continue
            if expect == "comma_or_end":
                top = stack[-1]
                if c == ",":
                    stack[-1] = top[0] + "1"
                    expect = "key" if top[0] == "{" else "value"
                    i += 1
                    if expect == "key":
                        stack[-1] = "{1"
                    continue
                if (c == "}" and top[0] == "{") or (c == "]" and top[0] == "["):
                    stack.pop()
                    expect = "comma_or_end" if stack else "end"
                    i += 1
                    continue
                return "bad", stack
        if expect == "end":
            return "closed", stack
        return "open", stack

    def allowed(self, text: str, piece: str) -> bool:
        state, _ = self._scan(text + piece)
        if state == "bad":
            return False
        if self.schema is not None and state == "closed":
            return self._valid((text + piece))
        if self.schema is not None and self.schema.get("type") == "object" and (text + piece).lstrip()[:1] not in ("", "{"):
            return False
        if self.schema is not None and self.schema.get("type") == "array" and (text + piece).lstrip()[:1] not in ("", "["):
            return False
        return True

    def closed(self, text: str) -> bool:
        return self._scan(text)[0] == "closed" and text.strip()[:1] in "{["

    def done(self, text: str) -> bool:
        return self._scan(text)[0] == "closed" and (self.schema is None or self._valid(text))

    def _valid(self, text: str) -> bool:
        try:
            return validate(json.loads(text), self.schema or {})
        except json.JSONDecodeError:
            return False


def validate(v: Any, schema: dict) -> bool:
    """The JSON-schema subset this server enforces."""
    if "const" in schema:
        return v == schema["const"]
    if "enum" in schema:
        return v in schema["enum"]
    if "anyOf" in schema:
        return any(validate(v, s) for s in schema["anyOf"])
    t = schema.get("type")
    if isinstance(t, list):
        return any(validate(v, {**schema, "type": x}) for x in t)
    if t == "object":
        if not isinstance(v, dict):
            return False
        props = schema.get("properties", {})
        if any(k not in v for k in schema.get("required", [])):
            return False
        if schema.get("additionalProperties") is False and any(k not in props for k in v):
            return False
        return all(validate(v[k], s) for k, s in props.items() if k in v)
    if t == "array":
        if not isinstance(v, list):
            return False
        if len(v) < schema.get("minItems", 0) or len(v) > schema.get("maxItems", 1 << 30):
            return False
        it = schema.get("items")
        return all(validate(x, it) for x in v) if isinstance(it, dict) else True
    if t == "string":
        return isinstance(v, str)
    if t == "integer":
        return isinstance(v, int) and not isinstance(v, bool)
    if t == "number":
        return isinstance(v, (int, float)) and not isinstance(v, bool)
    if t == "boolean":
        return isinstance(v, bool)
    if t == "null":
        return v is None
    return True
