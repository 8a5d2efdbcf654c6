"""HTTP API: llama-server compatible routes plus the OpenAI and Anthropic surfaces.

Routes (``crates/serve/src/api.rs:1743-1779`` in the reference): ``GET /health|/v1/health``,
``GET /v1/models|/models|/api/tags``, ``GET /v1/models/{id}``, ``POST /api/show``, ``GET /props``,
``GET /slots``, ``POST /slots/{id}?action=save|restore|erase``, ``GET /metrics``,
``POST /completion|/completions|/v1/completions``, ``POST /v1/chat/completions|/chat/completions``,
``POST /v1/messages`` (+ ``/count_tokens``), ``POST /v1/responses`` (+ ``GET/DELETE /v1/responses/{id}``),
``POST /v1/embeddings|/embeddings|/embedding``, ``POST /tokenize|/detokenize|/apply-template``,
``POST /residency/reset``, ``POST /shutdown`` (loopback only).

Start protocol (``listener.rs:1-10``, ``event.rs``): the socket is bound *before* the model
loads and answers 503 ``loading`` with the phase; ``bound``/``ready``/``error``/``stopped`` events
go to stdout as JSON lines.  Unknown request fields are ignored; a known field this build
does not serve is a 400 naming it (``docs/serving.md:62-64``).  An engine failure is fatal:
the request gets 500, ``/health`` turns 503 and the process exits 70.
"""
from __future__ import annotations

import collections
import gzip
import hmac
import ipaddress
import json
import math
import os
import queue
import re
import socket
import struct
import threading
import time
import uuid
import zlib
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Dict, List, Optional, Tuple
from urllib.parse import parse_qs, urlparse

from ..utils import events, levers
from . import chat as C
from .engine import Engine, EngineError
from .promptcache import PromptCache
from .sampler import SamplingParams
from .sched import Board, QueueFull
from .worker import Request, Worker

UNSUPPORTED_FIELDS = {"grammar": "GBNF grammars are not served; use response_format / json_schema",
                      "image_data": "this model takes text only", "lora": "LoRA adapters are not served",
                      "mirostat": None, "dynatemp_range": None, "xtc_probability": None, "dry_multiplier": None}


GENERATING_ROUTES = ("/completion", "/completions", "/v1/completions", "/v1/chat/completions", "/chat/completions", "/v1/messages",
                     "/v1/responses", "/v1/embeddings", "/embeddings", "/embedding")


from .admit import Refused  # noqa: E402


class ApiError(Exception):
    def __init__(self, status: int, message: str, kind: str = "invalid_request_error", param: Optional[str] = None):
        super().__init__(message)
        self.status, self.message, self.kind = status, message, kind
        if param is None:                        # an error about one request field names it, as OpenAI's errors do
            m = re.match(r"field '([A-Za-z_][\w.]*)'", message)
            param = m.group(1) if m else None
        self.param = param


class State:
    """Everything the handlers share."""

    def __init__(self, args: Dict[str, Any]):
        self.args = args
        self.phase = "plan"                     # plan | load | ready | failed | stopping
        self.engine: Optional[Engine] = None
        self.board: Optional[Board] = None
        self.worker: Optional[Worker] = None
        self.cache: Optional[PromptCache] = None
        self.template: Optional[C.ChatTemplate] = None
        self.tool_format = "hermes"
        self.alias = args.get("alias")
        self.api_keys, key_limits = self._load_keys(args)
        from .admit import Admission
        self.key_limits = key_limits
        self.admission = Admission(key_limits)
        self.t_start = time.time()
        self.responses: "collections.OrderedDict[str, dict]" = collections.OrderedDict()
        self.responses_bytes = 0
        self.stop_event = threading.Event()
        self.stop_cause = ""
        self.exit_code = 0
        self.inflight: Dict[str, int] = {}
        self.lock = threading.Lock()
        self.residency = None

    @staticmethod
    def _load_keys(args):
        """Keys of ``--api-key`` (no limits) and of the key file, whose lines may carry limit fields
        (``KEY inflight=2 rate=30/m burst=5``, see ``serve/admit.py``)."""
        from .admit import parse_key_line
        keys, limits = [], {}
        if args.get("api_key"):
            from ..utils.flags import split_keys
            keys += split_keys(str(args["api_key"]))
        if args.get("api_key_file"):
            with open(args["api_key_file"]) as fh:
                for ln in fh:
                    ln = ln.strip()
                    if not ln or ln.startswith("#"):
                        continue
                    key, lim = parse_key_line(ln)
                    if key in limits and not limits[key].same(lim):
                        raise ValueError(f"{args['api_key_file']}: a key is given twice with different fields")
                    keys.append(key)
                    limits[key] = lim
        return keys, limits

    @property
    def model_id(self) -> str:
        return self.alias or (self.engine.model_name if self.engine else "loading")

    def attach(self, engine: Engine, template: Optional[C.ChatTemplate], cache_bytes: int, queue_depth: int = 64) -> None:
        self.engine = engine
        self.template = template or C.ChatTemplate()
        self.tool_format = C.detect_tool_format(self.template.source)
        self.board = Board(engine.n_slots, queue_depth)
        self.cache = PromptCache(cache_bytes)
        self.worker = Worker(engine, self.board, self.cache, on_fatal=self._fatal)
        self.worker.start()
        self.phase = "ready"

    def _fatal(self, exc: BaseException) -> None:
        self.phase = "failed"
        self.exit_code = 70
        self.stop_cause = "engine"
        events.emit("error", code=70, word="engine", message=str(exc))
        self.stop_event.set()


# -------------------------------------------------------------------------------------------
# request shaping
# -------------------------------------------------------------------------------------------
SAMPLER_ORDER = ("penalties", "top_k", "top_p", "min_p", "temperature")      # the chain this server runs, in its order
I32_MAX = 2 ** 31 - 1


def sampling_from(body: Dict[str, Any], defaults: Dict[str, Any]) -> SamplingParams:
    def f(name, dflt, alt=None):
        v = body.get(name, body.get(alt) if alt else None)
        if v is None:
            return dflt
        # a sampling field of the wrong type or a non-finite value is refused by name (null is unset)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or (isinstance(v, float) and not math.isfinite(v)):
            raise ApiError(400, f"field {name!r} takes a finite number")
        return v
    seed = f("seed", defaults.get("seed", -1))
    return SamplingParams(
        temperature=float(f("temperature", defaults.get("temp", 0.8))), top_k=int(f("top_k", defaults.get("top_k", 40))),
        top_p=float(f("top_p", defaults.get("top_p", 0.95))), min_p=float(f("min_p", defaults.get("min_p", 0.05))),
        repeat_penalty=float(f("repeat_penalty", defaults.get("repeat_penalty", 1.0))),
        frequency_penalty=float(f("frequency_penalty", 0.0)), presence_penalty=float(f("presence_penalty", 0.0)),
        repeat_last_n=int(f("repeat_last_n", defaults.get("repeat_last_n", 64))),
        seed=int(seed) if seed is not None and int(seed) >= 0 else 0)


# sampler stages this server lacks: refused when a request turns one on (the value that leaves it off passes)
_OFF_VALUES = {"typical_p": (1, 1.0), "top_n_sigma": (-1, -1.0, 0, 0.0), "dry_multiplier": (0, 0.0), "xtc_probability": (0, 0.0),
               "dynatemp_range": (0, 0.0), "mirostat": (0,), "mirostat_tau": None, "mirostat_eta": None, "dry_base": None,
               "dry_allowed_length": None, "dry_penalty_last_n": None, "xtc_threshold": None, "dynatemp_exponent": None}


def logit_bias_from(body: Dict[str, Any], n_vocab: int = 0) -> Dict[int, float]:
    """OpenAI's ``logit_bias``: an object from token ids to a number in -100 to 100.  The other forms clients send (an
    array of pairs, ``false`` for "never", a token's text as the key) are refused by name rather than half-read, and so
    are a value out of range and an id named twice (``"7"`` beside ``"07"``)."""
    raw = body.get("logit_bias")
    if raw is None:
        return {}
    def bad(why: str):
        return ApiError(400, f"logit_bias: {why}", param="logit_bias")
    if not isinstance(raw, dict):
        raise bad("takes an object from token ids to numbers; an array of pairs is not read")
    out: Dict[int, float] = {}
    for k, v in raw.items():
        if not isinstance(k, str) or not k.strip().lstrip("+").isdigit():
            raise bad(f"the key {k!r} is not a token id (a token's text is not read)")
        t = int(k)
        if n_vocab and t >= n_vocab:
            raise bad(f"the id {t} is outside the vocabulary of {n_vocab}")
        if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v:
            raise bad(f"the value of {k!r} is not a number (false is not read; -100 bans an id)")
        if not -100 <= v <= 100:
            raise bad(f"the value of {k!r} is outside -100 to 100")
        if t in out:
            raise bad(f"the id {t} is named twice")
        out[t] = float(v)
    return out


def check_fields(body: Dict[str, Any], allow_n: bool = False) -> None:
    for k, why in UNSUPPORTED_FIELDS.items():
        if k in body and body[k] not in (None, "", 0, 0.0, [], False):
            raise ApiError(400, f"field {k!r} is not supported" + (f": {why}" if why else ""))
    for k, off in _OFF_VALUES.items():
        if off is not None and body.get(k) is not None and body[k] not in off:
            raise ApiError(400, f"field {k!r} turns on a sampler stage this server does not run")
    order = body.get("samplers")
    if order is not None:
        if not isinstance(order, list) or not all(isinstance(x, str) for x in order):
            raise ApiError(400, "field 'samplers' takes a list of sampler names")
        unknown = [x for x in order if x not in SAMPLER_ORDER]
        if unknown:
            raise ApiError(400, f"field 'samplers' names {unknown[0]!r}, a sampler this server lacks")
        want = [x for x in SAMPLER_ORDER if x in order]
        if list(order) != want:
            raise ApiError(400, f"field 'samplers' orders the chain as {order}; this server runs {want}")
    for k in ("n_predict", "max_tokens", "max_completion_tokens", "max_output_tokens"):
        v = body.get(k)
        if v is not None and (isinstance(v, bool) or not isinstance(v, int) or not -1 <= v <= I32_MAX):
            raise ApiError(400, f"field {k!r} takes a whole number from -1 to {I32_MAX}")
    n = body.get("n")
    if n is not None and (isinstance(n, bool) or not isinstance(n, int) or n < 1 or (n > 1 and not allow_n)):
        raise ApiError(400, "field 'n' above 1 is not served on this route" if isinstance(n, int) and not isinstance(n, bool) and n > 1
                       else "field 'n' takes a whole number from 1")


def stops_from(body) -> List[str]:
    s = body.get("stop")
    if s is None:
        return []
    if isinstance(s, str):
        return [s]
    if isinstance(s, list) and all(isinstance(x, str) for x in s):
        return [x for x in s if x]
    raise ApiError(400, "stop must be a string or a list of strings")


def constraint_from(body):
    """The structured-output constraint of a request: a segment program walked token by token when the schema compiles
    to one (``serve/constrain.py``), else the JSON prefix validator."""
    from .constrain import constraint_for
    asked = (body.get("response_format") or {}).get("type") in ("json_schema", "json_object") or bool(body.get("json_schema"))
    if asked:
        # a document that must close cannot also be told never to end, nor share the reply with a budgeted think span
        if body.get("ignore_eos"):
            raise ApiError(400, "ignore_eos beside structured output: the document ends the reply", param="ignore_eos")
        if body.get("reasoning_budget") not in (None, -1):
            raise ApiError(400, "reasoning_budget beside structured output: the think span is closed at once there",
                           param="reasoning_budget")

    def pick(schema):
        from .constrain import unserved_keyword
        bad = unserved_keyword(schema) if schema else None
        if bad is not None:
            raise ApiError(400, f"the schema keyword {bad!r} is outside the served subset", param="response_format")
        return constraint_for(schema) or C.JsonConstraint(schema)
    rf = body.get("response_format")
    if rf:
        t = rf.get("type")
        if t == "json_object":
            return pick(rf.get("schema"))
        if t == "json_schema":
            js = rf.get("json_schema") or {}
            return pick(js.get("schema", js))
        if t not in (None, "text"):
            raise ApiError(400, f"response_format.type {t!r} is not supported")
    if body.get("json_schema"):
        return pick(body["json_schema"])
    return None


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    server_version = "bloomery-b200"
    state: State = None  # set by serve()

    def log_message(self, fmt, *a):  # request lines go through records, not stderr noise
        pass

    # ---- plumbing ----------------------------------------------------------------------
    def _send(self, status: int, obj: Any, headers: Optional[Dict[str, str]] = None) -> None:
        data = obj if isinstance(obj, (bytes, bytearray)) else json.dumps(obj, ensure_ascii=False).encode()
        enc = self.headers.get("Accept-Encoding", "") if hasattr(self, "headers") and self.headers else ""
        extra = dict(headers or {})
        if "gzip" in enc and len(data) > 1024:
            data = gzip.compress(data, 5)
            extra["Content-Encoding"] = "gzip"
        self.send_response(status)
        self.send_header("Content-Type", extra.pop("Content-Type", "application/json; charset=utf-8"))
        self.send_header("Content-Length", str(len(data)))
        self.send_header("Access-Control-Allow-Origin", "*")
        for k, v in extra.items():
            self.send_header(k, v)
        self.end_headers()
        self.wfile.write(data)

    def _error(self, status: int, message: str, kind: str = "invalid_request_error", param: Optional[str] = None) -> None:
        if self.path.startswith("/v1/messages"):
            self._send(status, {"type": "error", "error": {"type": kind, "message": message}})
        else:
            err = {"code": status, "message": message, "type": kind}
            if param:
                err["param"] = param
            self._send(status, {"error": err})

    def _body(self) -> Dict[str, Any]:
        if self.headers.get("Expect", "").lower() == "100-continue":
            self.wfile.write(b"HTTP/1.1 100 Continue\r\n\r\n")
        if self.headers.get("Transfer-Encoding", "").lower() == "chunked":
            raw = bytearray()
            while True:
                line = self.rfile.readline().strip()
                n = int(line.split(b";")[0] or b"0", 16)
                if n == 0:
                    self.rfile.readline()
                    break
                raw += self.rfile.read(n)
                self.rfile.readline()
        else:
            n = int(self.headers.get("Content-Length") or 0)
            if n > 256 << 20:
                raise ApiError(413, "request body too large")
            raw = self.rfile.read(n) if n else b""
        ce = self.headers.get("Content-Encoding", "").strip().lower()
        if ce in ("gzip", "x-gzip", "deflate"):
            try:
                raw = gzip.decompress(raw) if ce != "deflate" else zlib.decompress(raw)
            except (OSError, EOFError, zlib.error) as exc:
                raise ApiError(400, f"the {ce} body does not decode: {exc}") from None
            if len(raw) > 256 << 20:
                raise ApiError(413, "request body too large")
        elif ce and ce != "identity":
            raise ApiError(415, f"Content-Encoding {ce!r} is not read; send gzip or deflate, one coding")
        if not raw:
            return {}
        try:
            body = json.loads(raw)
        except json.JSONDecodeError as exc:
            raise ApiError(400, f"request body is not JSON: {exc}") from None
        if not isinstance(body, dict):
            raise ApiError(400, "request body must be a JSON object")
        return body

    def _authorised(self) -> bool:
        keys = self.state.api_keys
        if not keys or self.path in ("/health", "/v1/health"):
            return True
        got = self.headers.get("Authorization", "")
        got = got[7:] if got.startswith("Bearer ") else self.headers.get("x-api-key", "")
        self._key = next((k for k in keys if hmac.compare_digest(got, k)), None)
        return self._key is not None

    def _loopback(self) -> bool:
        try:
            return ipaddress.ip_address(self.client_address[0]).is_loopback
        except ValueError:
            return False

    # ---- dispatch ----------------------------------------------------------------------
    def do_OPTIONS(self):
        self.send_response(204)
        self.send_header("Access-Control-Allow-Origin", "*")
        self.send_header("Access-Control-Allow-Headers", "*")
        self.send_header("Access-Control-Allow-Methods", "GET, POST, DELETE, OPTIONS")
        self.send_header("Content-Length", "0")
        self.end_headers()

    def do_GET(self):
        self._route("GET")

    def do_POST(self):
        self._route("POST")

    def do_DELETE(self):
        self._route("DELETE")

    def _route(self, method: str) -> None:
        st = self.state
        url = urlparse(self.path)
        path, q = url.path.rstrip("/") or "/", parse_qs(url.query)
        try:
            if not self._authorised():
                raise ApiError(401, "invalid API key", "authentication_error")
            lim = st.key_limits.get(getattr(self, "_key", None)) if getattr(st, "key_limits", None) else None
            if lim is not None and not lim.reaches(method, path):
                self.close_connection = True
                raise ApiError(403, "this key's scope does not reach this route", "permission_error")
            if path in ("/health", "/v1/health"):
                if st.phase == "ready":
                    return self._send(200, {"status": "ok", "slots_idle": st.engine.n_slots - st.board.busy_count(),
                                            "slots_processing": st.board.busy_count()})
                if st.phase == "failed":
                    return self._send(503, {"error": {"code": 503, "message": "engine failed", "type": "unavailable_error"}})
                return self._send(503, {"error": {"code": 503, "message": "Loading model", "type": "unavailable_error",
                                                  "phase": st.phase}})
            if st.phase != "ready":
                if st.phase == "failed":
                    raise ApiError(503, "engine failed", "unavailable_error")
                return self._send(503, {"error": {"code": 503, "message": "Loading model", "type": "unavailable_error", "phase": st.phase}})
            if method == "GET":
                if path in ("/v1/models", "/models"):
                    return self._send(200, {"object": "list", "data": [self._model_card()]})
                if path == "/api/tags":
                    return self._send(200, {"models": [{"name": st.model_id, "model": st.model_id, "details": {"format": "gguf"}}]})
                if path.startswith(("/v1/models/", "/models/")):
                    name = path.split("/models/", 1)[1]
                    if name != st.model_id:
                        raise ApiError(404, f"no model {name!r} here; this server serves {st.model_id!r}", "not_found_error")
                    return self._send(200, self._model_card())
                if path == "/props":
                    return self._send(200, self._props())
                if path == "/slots":
                    return self._send(200, st.board.snapshot())
                if path == "/metrics":
                    return self._send(200, self._metrics().encode(), {"Content-Type": "text/plain; version=0.0.4"})
                if path.startswith("/v1/responses/"):
                    r = st.responses.get(path.split("/")[3])
                    if r is None:
                        raise ApiError(404, "no such response", "not_found_error")
                    return self._send(200, self._public(r))
                raise ApiError(404, f"no route GET {path}", "not_found_error")
            if method == "DELETE":
                if path.startswith("/v1/responses/"):
                    r = st.responses.pop(path.split("/")[3], None)
                    if r is None:
                        raise ApiError(404, "no such response", "not_found_error")
                    return self._send(200, {"id": r["id"], "object": "response", "deleted": True})
                raise ApiError(404, f"no route DELETE {path}", "not_found_error")
            body = self._body()
            if path.startswith("/v1/responses/") and path.endswith("/cancel"):
                r = st.responses.get(path.split("/")[3])
                if r is None:
                    raise ApiError(404, "no such response", "not_found_error")
                req_ = r.get("_req")
                if req_ is not None and r.get("status") in ("queued", "in_progress"):
                    req_.cancelled.set()
                    r["status"] = "cancelled"
                return self._send(200, self._public(r))
            if path in GENERATING_ROUTES:
                # a generating request takes one of its key's places (in flight, and of its rate bucket) until answered
                release = st.admission.admit(getattr(self, "_key", None) or "")
                try:
                    return self._generating_route(path, body)
                finally:
                    release()
            if path in ("/completion", "/completions"):
                return self._completion(body, "llama")
            if path == "/v1/completions":
                return self._completion(body, "oai")
            if path in ("/v1/chat/completions", "/chat/completions"):
                return self._chat(body)
            if path in ("/v1/chat/completions/input_tokens", "/chat/completions/input_tokens", "/v1/messages/count_tokens", "/v1/responses/input_tokens"):
                msgs = self._anthropic_messages(body) if "messages" in path and "/v1/messages" in path else body.get("messages") or self._responses_messages(body)
                ids = self._chat_ids(msgs, body.get("tools"))
                return self._send(200, {"input_tokens": len(ids)})
            if path in ("/v1/systemone", "/systemone"):
                return self._systemone(body)
            if path == "/v1/messages":
                return self._messages(body)
            if path == "/v1/responses":
                return self._responses(body)
            if path in ("/v1/embeddings", "/embeddings", "/embedding"):
                return self._embeddings(body)
            if path == "/tokenize":
                tk = st.engine.tokenizer
                if not isinstance(body.get("content"), str):
                    raise ApiError(400, "field 'content' takes a string")
                ids = tk.encode(body["content"], parse_special=bool(body.get("parse_special", True)),
                                add_bos=bool(body.get("add_special", False)))
                if body.get("with_pieces"):
                    return self._send(200, {"tokens": [{"id": i, "piece": tk.decode([i], skip_special=False)} for i in ids]})
                return self._send(200, {"tokens": ids})
            if path == "/detokenize":
                toks = body.get("tokens")
                if not isinstance(toks, list):
                    raise ApiError(400, "tokens must be a list of ids")
                return self._send(200, {"content": st.engine.tokenizer.decode([int(t) for t in toks], skip_special=False)})
            if path == "/apply-template":
                from . import reasoning as RS
                try:
                    kwargs = RS.effort_kwargs(body.get("reasoning_effort"), body.get("chat_template_kwargs"))
                except RS.ReasoningError as exc:
                    raise ApiError(400, str(exc)) from None
                out = {"prompt": st.template.render_text(self._roles(body.get("messages") or []), tools=body.get("tools"), **kwargs)}
                if body.get("return_prompt_ids"):
                    # the guarded tokenization chat uses: client text never yields control tokens
                    out["prompt_ids"] = self._chat_ids(body.get("messages"), body.get("tools"), **kwargs)
                return self._send(200, out)
            if path == "/api/show":
                name = body.get("model") or body.get("name")
                if name is not None and name != st.model_id:
                    raise ApiError(404, f"no model {name!r} here; this server serves {st.model_id!r}", "not_found_error")
                info = dict(self._props()["model"])
                arch = str(info.get("arch") or "model")
                info[f"{arch}.context_length"] = st.engine.slot_ctx          # the served context, as Ollama clients read it
                caps = ["completion"] + (["tools"] if st.template is not None else [])
                return self._send(200, {"model_info": info, "details": {"format": "gguf", "family": arch}, "template": st.template.source,
                                        "capabilities": caps})
            if path.startswith("/slots/"):
                return self._slot_action(int(path.split("/")[2]), (q.get("action") or [""])[0], body)
            if path == "/residency/reset":
                if st.residency is not None:
                    st.worker.run_on_engine_thread(st.residency.reset)
                return self._send(200, {"ok": True})
            if path == "/shutdown":
                if not self._loopback():
                    raise ApiError(403, "shutdown is honoured from the loopback interface only", "permission_error")
                st.stop_cause = "shutdown"
                self._send(200, {"ok": True})
                st.stop_event.set()
                return None
            raise ApiError(404, f"no route POST {path}", "not_found_error")
        except ApiError as e:
            headers_415 = e.status == 415
            if headers_415:
                self._send(415, {"error": {"code": 415, "message": e.message, "type": e.kind}}, {"Accept-Encoding": "gzip, deflate"})
            else:
                self._error(e.status, e.message, e.kind, e.param)
        except C.TemplateError as e:
            self._error(400, str(e))
        except Refused as e:
            self._send(429, {"error": {"code": 429, "message": str(e), "type": "rate_limit_error"}}, {"Retry-After": str(e.retry_after)})
        except QueueFull as e:
            self._send(503, {"error": {"code": 503, "message": str(e), "type": "unavailable_error"}}, {"Retry-After": "1"})
        except (BrokenPipeError, ConnectionResetError):
            pass
        except Exception as e:  # noqa: BLE001 - the handler must answer
            try:
                self._error(500, f"{type(e).__name__}: {e}", "server_error")
            except Exception:  # noqa: BLE001
                pass

    def _generating_route(self, path: str, body):
        if path in ("/completion", "/completions"):
            return self._completion(body, "llama")
        if path == "/v1/completions":
            return self._completion(body, "oai")
        if path in ("/v1/chat/completions", "/chat/completions"):
            return self._chat(body)
        if path == "/v1/messages":
            return self._messages(body)
        if path == "/v1/responses":
            return self._responses(body)
        return self._embeddings(body)

    # ---- small surfaces ------------------------------------------------------------------
    def _model_card(self):
        st = self.state
        return {"id": st.model_id, "object": "model", "created": int(st.t_start), "owned_by": "bloomery_b200",
                "meta": {"n_vocab": st.engine.n_vocab, "n_ctx_train": st.engine.slot_ctx}}

    def _props(self):
        st = self.state
        a = st.args
        return {"default_generation_settings": {"n_ctx": st.engine.slot_ctx, "params": {
                    "temperature": a.get("temp", 0.8), "top_k": a.get("top_k", 40), "top_p": a.get("top_p", 0.95),
                    "min_p": a.get("min_p", 0.05), "repeat_penalty": a.get("repeat_penalty", 1.0),
                    "repeat_last_n": a.get("repeat_last_n", 64), "n_predict": a.get("n_predict", -1), "cache_prompt": True}},
                "total_slots": st.engine.n_slots, "model_path": a.get("model") or "", "model_alias": st.model_id,
                "chat_template": st.template.source, "bos_token": st.template.bos, "eos_token": st.template.eos,
                "model": st.engine.props(), "build_info": "bloomery_b200", "prompt_cache": st.cache.stats(),
                "placement": a.get("_place_word", ""), "modalities": {"vision": False, "audio": False},
                "thinking_off": self._thinking_off(), "tool_format": st.tool_format,
                "engine": {"draft": {"kind": {"NgramDraft": "lookup", "MtpDraft": "mtp", "NoneType": "off"}.get(
                                         type(getattr(st.worker, "draft", None)).__name__, type(getattr(st.worker, "draft", None)).__name__),
                                     "max_width": int(getattr(getattr(st.worker, "width", None), "max_width", 0) or 0)}}}

    def _metrics(self) -> str:
        st = self.state
        m = st.worker.metrics
        busy = st.board.busy_count()
        lines = []

        def g(name, help_, val, typ="counter"):
            lines.append(f"# HELP llamacpp:{name} {help_}\n# TYPE llamacpp:{name} {typ}\nllamacpp:{name} {val}")
        g("prompt_tokens_total", "Number of prompt tokens processed.", m.get("prompt_tokens_total"))
        g("prompt_seconds_total", "Prompt process time", m.get("prompt_seconds_total"))
        g("tokens_predicted_total", "Number of generation tokens processed.", m.get("tokens_predicted_total"))
        g("tokens_predicted_seconds_total", "Predict process time", m.get("tokens_predicted_seconds_total"))
        g("n_decode_total", "Total number of decode rounds", m.get("n_decode_total"))
        g("n_busy_slots_per_decode", "Average number of busy slots per decode round",
          m.get("n_busy_slots_per_decode") / max(1.0, m.get("n_decode_total")), "gauge")
        ps, ts = m.get("prompt_seconds_total"), m.get("tokens_predicted_seconds_total")
        g("prompt_tokens_seconds", "Average prompt throughput in tokens/s.", m.get("prompt_tokens_total") / ps if ps else 0, "gauge")
        g("predicted_tokens_seconds", "Average generation throughput in tokens/s.", m.get("tokens_predicted_total") / ts if ts else 0, "gauge")
        g("requests_processing", "Number of requests processing.", busy, "gauge")
        g("requests_deferred", "Number of requests deferred.", len(st.board.queue), "gauge")
        g("round_seconds_total", "Seconds spent in engine rounds", m.get("round_seconds_total"))
        g("prompt_cache_seconds_total", "Seconds spent in the host prompt cache", st.cache.seconds)
        g("prompt_cache_hits_total", "Prompt cache hits", m.get("prompt_cache_hits_total"))
        g("draft_tokens_total", "Speculative tokens drafted", m.get("draft_tokens_total"))
        g("draft_accepted_total", "Speculative tokens accepted", m.get("draft_accepted_total"))
        for w, n in sorted(st.worker.rounds_by_width.items()):
            lines.append(f'llamacpp:rounds_total{{width="{w}"}} {n}')
        for w, sec in sorted(st.worker.round_seconds_by_width.items()):
            lines.append(f'llamacpp:round_seconds_by_width_total{{width="{w}"}} {sec:.6f}')
        for w, sec in sorted(st.worker.round_card_wait_by_width.items()):
            lines.append(f'llamacpp:round_card_wait_seconds_total{{width="{w}"}} {sec:.6f}')
        g("card_wait_seconds_total", "Seconds the engine's host thread waited for the card", f"{float(m.get('card_wait_seconds_total') or 0.0):.6f}")
        source = {"NgramDraft": "ngram", "MtpDraft": "mtp"}.get(type(st.worker.draft).__name__, "none")
        for depth, n in sorted(st.worker.draft_by_depth.items()):
            lines.append(f'llamacpp:spec_decode_num_draft_tokens_by_depth_total{{source="{source}",depth="{depth}"}} {n}')
            lines.append(f'llamacpp:spec_decode_num_accepted_tokens_by_depth_total{{source="{source}",depth="{depth}"}} '
                         f'{st.worker.accepted_by_depth.get(depth, 0)}')
        dec = getattr(st.engine, "dec", None)
        if dec is not None and hasattr(dec, "waits"):
            for name, val in sorted(dec.waits.metrics().items()):
                g(name, "Engine-thread waits by kind", val)
            wd = getattr(dec, "watchdog", None)
            g("engine_wedged", "1 while a bounded engine wait has outlived its bound", int(bool(wd and wd.is_wedged())), "gauge")
        return "\n".join(lines) + "\n"

    def _slot_action(self, slot_id: int, action: str, body) -> None:
        st = self.state
        if not 0 <= slot_id < st.engine.n_slots:
            raise ApiError(404, f"no slot {slot_id}", "not_found_error")
        slot = st.board.slots[slot_id]
        base = st.args.get("slot_save_path")
        if action == "erase":
            def erase():
                if slot.busy:
                    raise ApiError(409, f"slot {slot_id} is busy")
                st.engine.reset(slot_id)
                n = len(slot.ids)
                slot.ids = []
                return n
            return self._send(200, {"id_slot": slot_id, "n_erased": st.worker.run_on_engine_thread(erase)})
        if action in ("save", "restore"):
            if not base:
                raise ApiError(400, "start the server with --slot-save-path to save or restore slots")
            name = os.path.basename(str(body.get("filename", "")))
            if not name:
                raise ApiError(400, "filename is required")
            path = os.path.join(base, name)
            from .slotfile import read_slot_file, write_slot_file
            t0 = time.time()
            if action == "save":
                def save():
                    saved = st.engine.snapshot(slot_id, slot.ids)
                    return write_slot_file(path, st.engine.n_vocab, slot.ids, saved)
                nbytes = st.worker.run_on_engine_thread(save)
                return self._send(200, {"id_slot": slot_id, "filename": name, "n_saved": len(slot.ids), "n_written": nbytes,
                                        "timings": {"save_ms": (time.time() - t0) * 1e3}})
            def restore():
                if slot.busy:
                    raise ApiError(409, f"slot {slot_id} is busy")
                ids, saved = read_slot_file(path, st.engine.n_vocab)
                n = st.engine.restore(slot_id, saved, len(ids))
                slot.ids = list(ids[:n])
                return n
            n = st.worker.run_on_engine_thread(restore)
            return self._send(200, {"id_slot": slot_id, "filename": name, "n_restored": n,
                                    "timings": {"restore_ms": (time.time() - t0) * 1e3}})
        raise ApiError(400, f"action {action!r}: expected save, restore or erase")

    def _embeddings(self, body) -> None:
        st = self.state
        inp = body.get("input", body.get("content"))
        if inp is None:
            raise ApiError(400, "input is required")
        items = inp if isinstance(inp, list) else [inp]
        data = []
        for i, text in enumerate(items):
            ids = st.engine.tokenizer.encode(str(text))
            if len(ids) + 1 > st.engine.slot_ctx:
                raise ApiError(400, f"input {i} has {len(ids)} tokens, more than the slot context of {st.engine.slot_ctx}")
            # on the engine thread, between rounds: the engine's buffers belong to that thread
            vec = st.worker.run_on_engine_thread(lambda ids=ids: st.engine.embed(ids)) if st.worker else st.engine.embed(ids)
            if vec is None:
                raise ApiError(501, "this model has no embedding head", "not_supported_error")
            data.append({"object": "embedding", "index": i, "embedding": [float(x) for x in vec]})
        self._send(200, {"object": "list", "data": data, "model": st.model_id,
                         "usage": {"prompt_tokens": sum(len(st.engine.tokenizer.encode(str(t))) for t in items), "total_tokens": 0}})

    # ---- generation ----------------------------------------------------------------------
    def _choices(self, body, prompt_ids: List[int]) -> List[Request]:
        """The requests of an ``n``-choice call: choice i samples with the request's seed plus i, so choice 0 is the
        answer ``n`` = 1 gives.  They queue together, so n is at most the slots plus the queue depth; streamed choices
        are not served."""
        st = self.state
        n = int(body.get("n") or 1)
        if n > 1 and body.get("stream"):
            raise ApiError(400, "field 'n' above 1 beside 'stream' is not served")
        if n > st.engine.n_slots + st.board.queue_depth:
            raise ApiError(400, f"field 'n' = {n} is above the slots plus the queue depth ({st.engine.n_slots} + {st.board.queue_depth})")
        seed = body.get("seed")
        base = int(seed) if isinstance(seed, int) and not isinstance(seed, bool) and seed >= 0 else 0
        return [self._make_request(dict(body, seed=base + i) if n > 1 else body, list(prompt_ids), allow_n=True) for i in range(n)]

    def _collect_all(self, reqs: List[Request]) -> List[dict]:
        """Submit every choice, then wait for each: they run side by side in the engine's rounds."""
        from .sched import QueueFull
        sent = []
        try:
            for r in reqs:
                self.state.board.submit(r)
                sent.append(r)
        except QueueFull as exc:
            for r in sent:
                r.cancelled.set()
            raise ApiError(503, str(exc), "unavailable_error") from None
        out = []
        for r in reqs:
            while True:
                ev = r.events.get()
                if ev[0] == "done":
                    out.append(ev[1])
                    break
                if ev[0] == "error":
                    for o in reqs:
                        o.cancelled.set()
                    raise ApiError(ev[1], ev[2], "server_error" if ev[1] >= 500 else "invalid_request_error")
        return out

    def _make_request(self, body, prompt_ids: List[int], n_predict_key=("n_predict", "max_tokens", "max_completion_tokens", "max_output_tokens"),
                      allow_n: bool = False) -> Request:
        st = self.state
        check_fields(body, allow_n)
        n_predict = -1
        for k in n_predict_key:
            if body.get(k) is not None:
                n_predict = int(body[k])
                break
        if n_predict < 0 and st.args.get("n_predict", -1) >= 0:
            n_predict = int(st.args["n_predict"])
        lb = logit_bias_from(body, int(getattr(st.engine, "n_vocab", 0) or 0))
        n_probs = int(body.get("n_probs") or 0)
        if body.get("logprobs") is True:
            n_probs = max(n_probs, int(body.get("top_logprobs") or 1))
        elif isinstance(body.get("logprobs"), int) and not isinstance(body.get("logprobs"), bool):
            n_probs = max(n_probs, int(body["logprobs"]))
        if not prompt_ids:
            tk = st.engine.tokenizer
            prompt_ids = [tk.bos_id] if tk.bos_id >= 0 else [0]
        constraint = constraint_from(body)
        # structured output decodes greedily unless the request names a temperature itself
        defaults = dict(st.args, temp=0.0) if constraint is not None else st.args
        return Request(prompt_ids=prompt_ids, sampling=sampling_from(body, defaults), n_predict=n_predict, stop=stops_from(body),
                       stream=bool(body.get("stream", False)), cache_prompt=bool(body.get("cache_prompt", True)),
                       n_probs=n_probs, ignore_eos=bool(body.get("ignore_eos", False)),
                       id_slot=(int(body["id_slot"]) if body.get("id_slot", -1) not in (None, -1) else None),
                       constraint=constraint, logit_bias=lb,
                       t_max_predict_ms=float(body.get("t_max_predict_ms") or 0),
                       endpoint=(urlparse(self.path).path.rstrip("/") or "/"), **self._reasoning_fields(body))

    @staticmethod
    def _reasoning_fields(body) -> Dict[str, Any]:
        from . import reasoning as RS
        choice = body.get("tool_choice")
        try:
            return {"reasoning_budget": RS.budget_from(body, forced_tool=choice == "required" or isinstance(choice, dict)),
                    "reasoning_loop": RS.loop_flag(body)}
        except RS.ReasoningError as exc:
            raise ApiError(400, str(exc)) from None

    def _prompt_ids(self, prompt) -> List[int]:
        tk = self.state.engine.tokenizer
        if isinstance(prompt, str):
            return tk.encode(prompt, parse_special=True)
        if isinstance(prompt, list):
            if all(isinstance(x, int) and not isinstance(x, bool) for x in prompt):
                bad = [x for x in prompt if not 0 <= x < self.state.engine.n_vocab]
                if bad:
                    raise ApiError(400, f"token id {bad[0]} is outside the vocabulary")
                return list(prompt)
            ids: List[int] = []
            for part in prompt:
                if isinstance(part, str):
                    ids += tk.encode(part, parse_special=True, add_bos=False)
                elif isinstance(part, int):
                    ids.append(part)
                else:
                    raise ApiError(400, "a mixed prompt may hold strings and token ids only")
            return ids
        raise ApiError(400, "prompt must be a string, a list of token ids, or a mix of both")

    def _collect(self, req: Request):
        """Block until the request ends; returns its final record."""
        self.state.board.submit(req)
        while True:
            ev = req.events.get()
            if ev[0] == "done":
                return ev[1]
            if ev[0] == "error":
                raise ApiError(ev[1], ev[2], "server_error" if ev[1] >= 500 else "invalid_request_error")

    def _sse_begin(self) -> None:
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Connection", "keep-alive")
        self.send_header("Access-Control-Allow-Origin", "*")
        self.send_header("Transfer-Encoding", "chunked")
        self.end_headers()

    def _sse(self, obj, event: Optional[str] = None) -> None:
        data = (f"event: {event}\n" if event else "") + "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n"
        raw = data.encode()
        self.wfile.write(f"{len(raw):x}\r\n".encode() + raw + b"\r\n")
        self.wfile.flush()

    def _sse_end(self) -> None:
        self.wfile.write(b"0\r\n\r\n")
        self.wfile.flush()

    def _stream(self, req: Request, on_text, on_done) -> None:
        """Drive an SSE response from the request's events; a dropped client cancels the request."""
        self.state.board.submit(req)
        self._sse_begin()
        try:
            while True:
                ev = req.events.get()
                if ev[0] == "text":
                    on_text(ev[1])
                elif ev[0] == "done":
                    on_done(ev[1])
                    break
                elif ev[0] == "error":
                    self._sse({"error": {"code": ev[1], "message": ev[2]}})
                    break
            self._sse_end()
        except (BrokenPipeError, ConnectionResetError):
            req.cancelled.set()
            self.close_connection = True

    def _completion(self, body, shape: str) -> None:
        st = self.state
        if "prompt" not in body:
            raise ApiError(400, "prompt is required")
        if shape != "llama":
            pr = body["prompt"]
            if isinstance(pr, list) and pr and all(isinstance(x, (str, list)) for x in pr) and len(pr) > 1:
                raise ApiError(400, "field 'prompt' holds several prompts; this route takes one a request")
            for k, bad in (("echo", bool(body.get("echo"))), ("suffix", bool(body.get("suffix"))),
                           ("best_of", isinstance(body.get("best_of"), int) and body["best_of"] > 1),
                           ("logprobs", body.get("logprobs") not in (None, False, 0))):
                if bad:
                    raise ApiError(400, f"field {k!r} is not served on /v1/completions")
        many = self._choices(body, self._prompt_ids(body["prompt"])) if shape != "llama" else None
        req = many[0] if many else self._make_request(body, self._prompt_ids(body["prompt"]))
        rid = f"cmpl-{uuid.uuid4().hex[:24]}"
        if shape == "llama":
            def final(d, content):
                return {"content": content, "stop": True, "model": st.model_id, "tokens_predicted": d["tokens_predicted"],
                        "tokens_evaluated": d["tokens_evaluated"], "tokens_cached": d["tokens_cached"], "id_slot": d["id_slot"],
                        "stop_type": d["stop_type"] if d["stop_type"] != "cancelled" else "none", "stopping_word": d["stopping_word"],
                        "timings": d["timings"], "truncated": False, "tokens": d["tokens"] if body.get("return_tokens") else [],
                        **({"completion_probabilities": d["probs"]} if req.n_probs else {}),
                        "generation_settings": {"n_predict": req.n_predict, "temperature": req.sampling.temperature,
                                                "top_k": req.sampling.top_k, "top_p": req.sampling.top_p, "min_p": req.sampling.min_p,
                                                "seed": req.sampling.seed, "stop": req.stop}}
            if req.stream:
                return self._stream(req, lambda t: self._sse({"content": t, "stop": False}), lambda d: self._sse(final(d, "")))
            d = self._collect(req)
            return self._send(200, final(d, d["text"]))
        finish = {"eos": "stop", "word": "stop", "limit": "length", "cancelled": "stop"}

        def chunk(text, fr=None):
            return {"id": rid, "object": "text_completion", "created": int(time.time()), "model": st.model_id,
                    "choices": [{"index": 0, "text": text, "finish_reason": fr, "logprobs": None}]}
        if req.stream:
            def done(d):
                self._sse(chunk("", finish.get(d["stop_type"], "stop")))
                self._sse("[DONE]")
            return self._stream(req, lambda t: self._sse(chunk(t)), done)
        ds = self._collect_all(many)
        d = ds[0]
        out = chunk(d["text"], finish.get(d["stop_type"], "stop"))
        out["choices"] = [{"index": i, "text": di["text"], "finish_reason": finish.get(di["stop_type"], "stop"),
                           "logprobs": {"content": di["probs"]} if req.n_probs else None} for i, di in enumerate(ds)]
        done_n = sum(di["tokens_predicted"] for di in ds)
        out["usage"] = {"prompt_tokens": d["tokens_evaluated"], "completion_tokens": done_n,
                        "total_tokens": d["tokens_evaluated"] + done_n}            # the prompt counts once
        out["timings"] = d["timings"]
        self._send(200, out)

    def _chat_ids(self, messages, tools=None, **extra) -> List[int]:
        st = self.state
        if not isinstance(messages, list) or not messages:
            raise ApiError(400, "messages must be a non-empty list")
        for m in messages:
            if not isinstance(m, dict) or "role" not in m:
                raise ApiError(400, "every message needs a role")
        # a developer message reaches the template as system (the mapping llama-server makes), except on a template that
        # names the developer role itself (GPT-OSS's)
        messages = self._roles(messages)
        segs = st.template.render(messages, tools=tools, add_generation_prompt=True, **extra)
        return st.engine.tokenizer.encode_marked(segs)

    def _roles(self, messages):
        if isinstance(messages, list) and "developer" not in self.state.template.source \
                and any(isinstance(m, dict) and m.get("role") == "developer" for m in messages):
            return [dict(m, role="system") if isinstance(m, dict) and m.get("role") == "developer" else m for m in messages]
        return messages

    def _thinking_off(self) -> str:
        """How this template turns thinking off: ``switch`` (it reads ``enable_thinking``), ``low_effort`` (no switch but
        an effort header), ``off_word`` (its own word for no thinking, ``no_think``) or ``neither``."""
        src = self.state.template.source
        if "enable_thinking" in src:
            return "switch"
        if "no_think" in src:
            return "off_word"
        if "reasoning_effort" in src:
            return "low_effort"
        return "neither"

    def _template_opened_think(self, ids: List[int]) -> bool:
        """Whether the rendered prompt ends inside a think span the template opened itself."""
        tail = self.state.engine.tokenizer.decode(list(ids[-16:]), skip_special=False)
        return tail.rstrip().endswith("<think>")

    @staticmethod
    def _forced_name(choice) -> Optional[str]:
        """``"required"`` or the function a ``tool_choice`` names, in OpenAI's, the Responses API's or Anthropic's shape;
        None when the choice forces nothing."""
        if choice in (None, "auto", "none"):
            return None
        if choice == "required":
            return "required"
        if isinstance(choice, dict):
            t = choice.get("type")
            if t in ("auto", "none"):
                return None
            if t == "any":
                return "required"
            name = (choice.get("function") or {}).get("name") if isinstance(choice.get("function"), dict) else choice.get("name")
            if t in ("function", "tool") and isinstance(name, str) and name:
                return name
        raise ApiError(400, f"tool_choice {choice!r} is not supported", param="tool_choice")

    def _force_call(self, reqs: List[Request], body, tools, ids: List[int]) -> None:
        """Hold each of ``reqs`` to one tool call when the request's ``tool_choice`` forces one: the call is written in
        the framing the template renders calls in, its arguments follow the tool's schema, and a think span the template
        opened stays free until the model closes it."""
        forced = self._forced_name(body.get("tool_choice"))
        from .constrain import ForcedCall, Unsupported, forced_call_program, watched_calls
        if forced is None:
            choice = body.get("tool_choice")
            off = choice == "none" or (isinstance(choice, dict) and choice.get("type") == "none")
            if tools and not off and str(levers.get("BLOOMERY_WATCH_CALLS")) != "off":
                for t in tools:                                    # an invalid tool is a 400; one outside the subset is unwatched
                    fn = t.get("function", t) if isinstance(t, dict) else None
                    if not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
                        raise ApiError(400, "tools: each tool needs a function with a name", param="tools")
                    if fn.get("parameters") is not None and not isinstance(fn["parameters"], dict):
                        raise ApiError(400, f"tools: the parameters of {fn['name']!r} are not a schema object", param="tools")
                for r_ in reqs:
                    if r_.constraint is None:
                        r_.constraint = watched_calls(tools, self.state.tool_format)
            return
        rf = body.get("response_format") or {}
        if rf.get("type") in ("json_schema", "json_object") or body.get("json_schema"):
            raise ApiError(400, "a JSON response_format beside a forced tool_choice: the reply is the call", param="response_format")
        try:
            program = forced_call_program(tools, forced, self.state.tool_format)
        except Unsupported as exc:
            raise ApiError(400, f"tool_choice: {exc}", param="tool_choice") from None
        open_think = self._template_opened_think(ids)
        for r_ in reqs:
            r_.constraint = ForcedCall(program, think_open=open_think)
            if body.get("temperature") is None:                      # a forced call decodes greedily unless the request says
                import dataclasses
                r_.sampling = dataclasses.replace(r_.sampling, temperature=0.0)

    def _chat(self, body) -> None:
        st = self.state
        tools = body.get("tools")
        self._forced_name(body.get("tool_choice"))
        from . import reasoning as RS
        try:
            kwargs = RS.effort_kwargs(body.get("reasoning_effort"), body.get("chat_template_kwargs"))
        except RS.ReasoningError as exc:
            raise ApiError(400, str(exc)) from None
        ids = self._chat_ids(body.get("messages"), tools if body.get("tool_choice") != "none" else None, **kwargs)
        many = self._choices(body, ids)
        req = many[0]
        for r_ in many:
            r_.think_started = self._template_opened_think(ids)
        if many[0].think_started:
            # a JSON response_format closes the span the template opened at once and writes the document after it
            from .constrain import AfterThink
            for r_ in many:
                if r_.constraint is not None:
                    r_.constraint, r_.reasoning_budget = AfterThink(r_.constraint), 0
        self._force_call(many, body, tools, ids)
        rid = f"chatcmpl-{uuid.uuid4().hex[:24]}"
        finish = {"eos": "stop", "word": "stop", "limit": "length", "cancelled": "stop", "reasoning_loop": "reasoning_loop"}
        want_reasoning = body.get("reasoning_format", "auto") != "none"

        def usage(d):
            return {"prompt_tokens": d["tokens_evaluated"], "completion_tokens": d["tokens_predicted"],
                    "total_tokens": d["tokens_evaluated"] + d["tokens_predicted"],
                    "prompt_tokens_details": {"cached_tokens": d["tokens_cached"]}}
        if req.stream:
            # a JSON-framed call streams as the model writes it (name first, argument fragments after); the other
            # framings send a call when it closes
            tcs = (C.ToolCallDeltas() if st.tool_format == "hermes" else C.ToolCallStream(st.tool_format)) if tools else None
            saw_call = [False]
            broke = [False]

            def delta(dl, fr=None):
                return {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": st.model_id,
                        "choices": [{"index": 0, "delta": dl, "finish_reason": fr}]}

            def on_text(t):
                if tcs is None:
                    return self._sse(delta({"content": t}))
                if broke[0]:
                    return
                try:
                    text, calls = tcs.push(t)
                except C.ToolStreamError as exc:
                    # markup that stopped being a call after its name went out: the stream ends with an error naming it
                    broke[0] = True
                    req.cancelled.set()
                    return self._sse({"error": {"code": 500, "message": str(exc), "type": "server_error"}})
                if text:
                    self._sse(delta({"content": text}))
                for c in calls:
                    saw_call[0] = True
                    self._sse(delta({"tool_calls": [c]}))

            def on_done(d):
                if broke[0]:
                    return self._sse("[DONE]")
                inside = getattr(tcs, "open_call", None) if tcs is not None else None
                if tcs is not None:
                    rest = tcs.flush()
                    if rest:
                        self._sse(delta({"content": rest}))
                if inside is not None and d["stop_type"] != "limit":
                    self._sse({"error": {"code": 500, "message": f"the generation ended inside the tool call {inside or '(unnamed)'!r}",
                                         "type": "server_error"}})
                    return self._sse("[DONE]")
                fin = delta({}, "length" if inside is not None else "tool_calls" if saw_call[0] else finish.get(d["stop_type"], "stop"))
                if (body.get("stream_options") or {}).get("include_usage"):
                    fin["usage"] = usage(d)
                fin["timings"] = d["timings"]
                self._sse(fin)
                self._sse("[DONE]")
            self._sse_role = True
            self.state.board  # noqa: B018 - keep the attribute access explicit for readers
            def first_then(t, _f=[True]):
                if _f[0]:
                    _f[0] = False
                    self._sse(delta({"role": "assistant", "content": ""}))
                on_text(t)
            return self._stream(req, first_then, on_done)
        ds = self._collect_all(many)
        choices = []
        for i, di in enumerate(ds):
            reasoning, content = C.split_reasoning(di["text"], started=req.think_started) if want_reasoning else ("", di["text"])
            calls: List[dict] = []
            cut_short = False
            if tools:
                content, calls = C.parse_tool_calls(content, st.tool_format)
                cut = C.cut_call(content, st.tool_format)
                if cut is not None:
                    # the reply stops inside a call: cut by the token limit it answers 200 with finish_reason length (the
                    # call with the arguments read so far once its name is whole, its text as content before that); a
                    # generation that ends on its own there has written no call a client can run
                    if di["stop_type"] != "limit":
                        raise ApiError(500, f"the generation ended inside the tool call {cut[1] or '(unnamed)'!r}", "server_error")
                    cut_short = True
                    if cut[1] is not None:
                        content = cut[0]
                        calls = calls + [{"id": f"call_{len(calls)}", "type": "function", "function": {"name": cut[1], "arguments": cut[2]}}]
            msg: Dict[str, Any] = {"role": "assistant", "content": content if (content or not calls) else None}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                msg["tool_calls"] = calls
            choices.append({"index": i, "message": msg,
                            "finish_reason": "length" if cut_short else "tool_calls" if calls else finish.get(di["stop_type"], "stop"),
                            "logprobs": {"content": di["probs"]} if req.n_probs else None})
        d = ds[0]
        use = usage(d)
        use["completion_tokens"] = sum(di["tokens_predicted"] for di in ds)            # the prompt counts once
        use["total_tokens"] = use["prompt_tokens"] + use["completion_tokens"]
        out = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": st.model_id,
               "choices": choices, "usage": use, "timings": d["timings"]}
        self._send(200, out)

    # ---- the decision models' request on a generative model ----------------------------------
    def _systemone(self, body) -> None:
        """``POST /v1/systemone``: the schema text goes in the system message and the state in the user message, the
        reply is held to a JSON object by the structured-output path, and each question's scores are the logits of the
        tokens its options start with, read where the model picks (``serve/systemone.py``)."""
        from . import systemone as S1
        from .constrain import AfterThink
        st = self.state
        tk = st.engine.tokenizer
        encode = lambda text: tk.encode(text, parse_special=False, add_bos=False)      # noqa: E731
        try:
            state, questions = S1.read_request(body)
            schema = S1.plan(questions, encode)
        except S1.SystemOneError as exc:
            raise ApiError(exc.status, str(exc), "not_supported_error" if exc.status == 501 else "invalid_request_error") from None
        cache = body.get("cache_prompt", True)
        if not isinstance(cache, bool):
            raise ApiError(400, "cache_prompt takes true or false", param="cache_prompt")
        msgs = [{"role": "system", "content": S1.schema_text(questions)}, {"role": "user", "content": state}]
        ids = self._chat_ids(msgs)
        room = st.engine.slot_ctx - len(ids) - 1
        if room < 16:
            raise ApiError(400, f"the request of {len(ids)} ids leaves no room for the answers in a context of {st.engine.slot_ctx}",
                           "exceed_context_size_error")
        req = self._make_request({"response_format": {"type": "json_schema", "json_schema": {"schema": schema}}, "temperature": 0,
                                  "cache_prompt": cache, "max_tokens": min(room, 64 + 48 * len(questions))}, ids)
        if req.constraint is None or not hasattr(req.constraint, "forced_text"):
            raise ApiError(400, "the questions' ids do not write out to a schema this server walks")
        req.think_started = self._template_opened_think(ids)
        if req.think_started:
            req.constraint, req.reasoning_budget = AfterThink(req.constraint), 0
        req.pick_rows = []
        d = self._collect(req)
        text = d["text"]
        if req.think_started and "</think>" in text:
            text = text[text.index("</think>") + len("</think>"):]
        document = text.lstrip("\n")
        lead = len(d["text"]) - len(document)
        try:
            got = S1.answers(questions, document, [(n - lead, row) for n, row in req.pick_rows], encode)
        except S1.SystemOneError as exc:
            raise ApiError(exc.status, str(exc), "server_error" if exc.status >= 500 else "invalid_request_error") from None
        t = d["timings"]
        self._send(200, {"model": st.model_id, "answers": got,
                         "usage": {"input_tokens": d["tokens_evaluated"], "output_tokens": d["tokens_predicted"]},
                         "timings": {"prompt_n": t.get("prompt_n", d["tokens_evaluated"] - d["tokens_cached"]),
                                     "prompt_ms": t.get("prompt_ms", 0.0), "head_ms": t.get("predicted_ms", 0.0),
                                     "cache_n": d["tokens_cached"]}})

    # ---- Anthropic Messages ----------------------------------------------------------------
    def _anthropic_messages(self, body) -> List[dict]:
        msgs: List[dict] = []
        sysm = body.get("system")
        if isinstance(sysm, list):
            sysm = "".join(p.get("text", "") for p in sysm if isinstance(p, dict))
        if sysm:
            msgs.append({"role": "system", "content": sysm})
        for m in body.get("messages") or []:
            c = m.get("content")
            if isinstance(c, list):
                parts, calls = [], []
                for p in c:
                    t = p.get("type")
                    if t == "text":
                        parts.append(p.get("text", ""))
                    elif t == "tool_use":
                        calls.append({"id": p.get("id"), "type": "function", "function": {"name": p.get("name"), "arguments": json.dumps(p.get("input", {}))}})
                    elif t == "tool_result":
                        rc = p.get("content")
                        if isinstance(rc, list):
                            rc = "".join(x.get("text", "") for x in rc if isinstance(x, dict))
                        msgs.append({"role": "tool", "tool_call_id": p.get("tool_use_id"), "content": rc or ""})
                    else:
                        raise ApiError(400, f"content block type {t!r} is not supported")
                if parts or calls:
                    mm = {"role": m.get("role"), "content": "".join(parts)}
                    if calls:
                        mm["tool_calls"] = calls
                    msgs.append(mm)
            else:
                msgs.append({"role": m.get("role"), "content": c or ""})
        return msgs

    def _messages(self, body) -> None:
        st = self.state
        if body.get("max_tokens") is None:
            raise ApiError(400, "max_tokens is required")
        tools = None
        if body.get("tools"):
            tools = [{"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                       "parameters": t.get("input_schema", {})}} for t in body["tools"]]
        ids = self._chat_ids(self._anthropic_messages(body), tools)
        b2 = dict(body)
        b2["stop"] = body.get("stop_sequences")
        req = self._make_request(b2, ids)
        req.think_started = self._template_opened_think(ids)
        self._force_call([req], body, tools, ids)
        mid = f"msg_{uuid.uuid4().hex[:24]}"
        reason = {"eos": "end_turn", "word": "stop_sequence", "limit": "max_tokens", "cancelled": "end_turn",
                  "reasoning_loop": "reasoning_loop"}
        if req.stream:
            def start():
                self._sse({"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "content": [],
                           "model": st.model_id, "stop_reason": None, "usage": {"input_tokens": len(ids), "output_tokens": 0}}}, "message_start")
                self._sse({"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}}, "content_block_start")
            started = [False]

            def on_text(t):
                if not started[0]:
                    started[0] = True
                    start()
                self._sse({"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": t}}, "content_block_delta")

            def on_done(d):
                if not started[0]:
                    start()
                self._sse({"type": "content_block_stop", "index": 0}, "content_block_stop")
                self._sse({"type": "message_delta", "delta": {"stop_reason": reason.get(d["stop_type"], "end_turn"),
                           "stop_sequence": d["stopping_word"] or None}, "usage": {"output_tokens": d["tokens_predicted"]}}, "message_delta")
                self._sse({"type": "message_stop"}, "message_stop")
            return self._stream(req, on_text, on_done)
        d = self._collect(req)
        reasoning, content = C.split_reasoning(d["text"], started=req.think_started)
        blocks: List[dict] = []
        calls: List[dict] = []
        if tools:
            content, calls = C.parse_tool_calls(content, st.tool_format)
        if reasoning:
            blocks.append({"type": "thinking", "thinking": reasoning})
        if content or not calls:
            blocks.append({"type": "text", "text": content})
        for c in calls:
            blocks.append({"type": "tool_use", "id": c["id"].replace("call_", "toolu_"), "name": c["function"]["name"],
                           "input": json.loads(c["function"]["arguments"] or "{}")})
        self._send(200, {"id": mid, "type": "message", "role": "assistant", "model": st.model_id, "content": blocks,
                         "stop_reason": "tool_use" if calls else reason.get(d["stop_type"], "end_turn"),
                         "stop_sequence": d["stopping_word"] or None,
                         "usage": {"input_tokens": d["tokens_evaluated"], "output_tokens": d["tokens_predicted"],
                                   "cache_read_input_tokens": d["tokens_cached"]}})

    # ---- OpenAI Responses ------------------------------------------------------------------
    def _responses_messages(self, body) -> List[dict]:
        msgs: List[dict] = []
        if body.get("instructions"):
            msgs.append({"role": "system", "content": body["instructions"]})
        prev = body.get("previous_response_id")
        if prev:
            old = self.state.responses.get(prev)
            if old is None:
                raise ApiError(404, f"previous_response_id {prev!r} is not in the store", "not_found_error")
            msgs += old.get("_messages", [])
        inp = body.get("input")
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        elif isinstance(inp, list):
            for it in inp:
                t = it.get("type", "message")
                if t == "message":
                    c = it.get("content")
                    if isinstance(c, list):
                        c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
                    msgs.append({"role": it.get("role", "user"), "content": c or ""})
                elif t == "function_call_output":
                    msgs.append({"role": "tool", "tool_call_id": it.get("call_id"), "content": str(it.get("output", ""))})
                elif t == "function_call":
                    msgs.append({"role": "assistant", "content": "", "tool_calls": [{"id": it.get("call_id"), "type": "function",
                                 "function": {"name": it.get("name"), "arguments": it.get("arguments", "{}")}}]})
                elif t == "item_reference":
                    raise ApiError(400, "an item_reference input item is not served: send the item itself", param="input")
                else:
                    raise ApiError(400, f"input item type {t!r} is not supported", param="input")
        elif inp is not None:
            raise ApiError(400, "input must be a string or a list of items")
        return msgs

    def _responses(self, body) -> None:
        st = self.state
        msgs = self._responses_messages(body)
        tools = None
        spaces: Dict[str, str] = {}                     # a flattened function's bare name -> the namespace it came in
        if body.get("tools"):
            def fn(t):
                return {"type": "function", "function": {"name": t.get("name"), "description": t.get("description", ""),
                                                         "parameters": t.get("parameters", {})}}
            tools = []
            for t in body["tools"]:
                if not isinstance(t, dict):
                    raise ApiError(400, "tools: each tool is an object", param="tools")
                if t.get("type") == "function":
                    tools.append(fn(t))
                elif t.get("type") == "namespace":
                    # a namespace tool is flattened: each function inside serves under its bare name, and a call of it
                    # carries the namespace in its item
                    for inner in t.get("tools") or []:
                        if isinstance(inner, dict) and inner.get("type", "function") == "function" and inner.get("name"):
                            if inner["name"] in spaces or any(x["function"]["name"] == inner["name"] for x in tools):
                                raise ApiError(400, f"tools: the function {inner['name']!r} is named twice once namespaces are flattened",
                                               param="tools")
                            spaces[inner["name"]] = str(t.get("name") or "")
                            tools.append(fn(inner))
            tools = tools or None
        from . import reasoning as RS
        try:
            kwargs = RS.effort_kwargs((body.get("reasoning") or {}).get("effort") if isinstance(body.get("reasoning"), dict) else None, None)
        except RS.ReasoningError as exc:
            raise ApiError(400, str(exc)) from None
        ids = self._chat_ids(msgs, tools, **kwargs)
        b2 = dict(body)
        fmt = (body.get("text") or {}).get("format")
        if fmt and fmt.get("type") in ("json_schema", "json_object"):
            b2["response_format"] = {"type": fmt["type"], "json_schema": {"schema": fmt.get("schema")}} if fmt["type"] == "json_schema" else {"type": "json_object"}
        if body.get("conversation") is not None:
            raise ApiError(400, "field 'conversation' is not served; continue with previous_response_id")
        background = body.get("background") is True
        if background and (body.get("store") is False or body.get("stream")):
            raise ApiError(400, "field 'background' beside store: false or stream: true is not served")
        req = self._make_request(b2, ids)
        req.think_started = self._template_opened_think(ids)
        if req.think_started and req.constraint is not None:
            from .constrain import AfterThink
            req.constraint, req.reasoning_budget = AfterThink(req.constraint), 0
        self._force_call([req], b2, tools, ids)
        rid = f"resp_{uuid.uuid4().hex[:24]}"

        def build(d):
            reasoning, content = C.split_reasoning(d["text"], started=req.think_started)
            calls: List[dict] = []
            if tools:
                content, calls = C.parse_tool_calls(content, st.tool_format)
            output: List[dict] = []
            if reasoning:
                output.append({"type": "reasoning", "id": f"rs_{uuid.uuid4().hex[:16]}", "summary": [{"type": "summary_text", "text": reasoning}]})
            if content or not calls:
                output.append({"type": "message", "id": f"msg_{uuid.uuid4().hex[:16]}", "role": "assistant", "status": "completed",
                               "content": [{"type": "output_text", "text": content, "annotations": []}]})
            for c in calls:
                output.append({"type": "function_call", "id": f"fc_{uuid.uuid4().hex[:16]}", "call_id": c["id"],
                               "name": c["function"]["name"], "arguments": c["function"]["arguments"], "status": "completed"})
                if c["function"]["name"] in spaces:
                    output[-1]["namespace"] = spaces[c["function"]["name"]]
            resp = {"id": rid, "object": "response", "created_at": int(time.time()), "status": "completed" if d["stop_type"] not in ("limit", "reasoning_loop") else "incomplete",
                    "model": st.model_id, "output": output, "output_text": content,
                    "usage": {"input_tokens": d["tokens_evaluated"], "output_tokens": d["tokens_predicted"],
                              "total_tokens": d["tokens_evaluated"] + d["tokens_predicted"],
                              "input_tokens_details": {"cached_tokens": d["tokens_cached"]}}}
            if body.get("store", True):
                keep = dict(resp)
                # a later previous_response_id continues the input and the output, not the instructions
                convo = msgs[1:] if body.get("instructions") and msgs and msgs[0].get("role") == "system" else msgs
                keep["_messages"] = convo + [{"role": "assistant", "content": content}]
                self._store(keep)
            return resp
        if background:
            # answered `queued` at once; the generation runs behind it and the stored response turns completed,
            # incomplete, cancelled or failed; a full store refuses new background work until finished ones leave
            with st.lock:
                running = sum(1 for r_ in st.responses.values() if r_.get("status") in ("queued", "in_progress"))
            if running >= 1024:
                raise ApiError(503, "the response store is full of running responses", "unavailable_error")
            queued = {"id": rid, "object": "response", "created_at": int(time.time()), "status": "queued", "model": st.model_id,
                      "output": [], "background": True, "_req": req, "_messages": msgs}
            self._store(queued)

            def work():
                try:
                    d = self._collect(req)
                    cancelled = queued.get("status") == "cancelled" or d["stop_type"] == "cancelled"
                    done = build(d)                      # stores the finished response under the same id
                    if cancelled:
                        st.responses[rid]["status"] = "cancelled"
                except Exception as exc:             # noqa: BLE001 - the poller reads the failure
                    queued.update(status="failed", error={"message": str(exc)})
            threading.Thread(target=work, name=f"response-{rid}", daemon=True).start()
            return self._send(200, self._public(queued))
        if req.stream:
            seq = [0]

            def ev(name, payload):
                payload["type"] = name
                payload["sequence_number"] = seq[0]
                seq[0] += 1
                self._sse(payload, name)
            started = [False]

            def start():
                started[0] = True
                ev("response.created", {"response": {"id": rid, "object": "response", "status": "in_progress", "model": st.model_id, "output": []}})
                ev("response.output_item.added", {"output_index": 0, "item": {"type": "message", "role": "assistant", "content": []}})

            def on_text(t):
                if not started[0]:
                    start()
                ev("response.output_text.delta", {"output_index": 0, "content_index": 0, "delta": t})

            def on_done(d):
                if not started[0]:
                    start()
                resp = build(d)
                ev("response.output_text.done", {"output_index": 0, "content_index": 0, "text": resp["output_text"]})
                ev("response.completed", {"response": resp})
            return self._stream(req, on_text, on_done)
        self._send(200, build(self._collect(req)))

    @staticmethod
    def _public(resp: dict) -> dict:
        """A stored response without the server's own fields."""
        return {k: v for k, v in resp.items() if not k.startswith("_")}

    def _store(self, resp: dict) -> None:
        """Bounded response store: 1,024 responses / 256 MiB (``response_store.rs``)."""
        st = self.state
        size = len(json.dumps(self._public(resp), default=str)) + len(json.dumps(resp.get("_messages", []), default=str))
        with st.lock:
            old = st.responses.get(resp["id"])
            if old is not None:                      # a background response finishing under its own id
                st.responses_bytes -= old.get("_size", 0)
            st.responses[resp["id"]] = resp
            st.responses_bytes += size
            resp["_size"] = size
            while len(st.responses) > 1024 or st.responses_bytes > (256 << 20):
                _, old = st.responses.popitem(last=False)
                st.responses_bytes -= old.get("_size", 0)


class Server:
    """Binds first, answers ``loading`` while the model loads, then serves."""

    def __init__(self, args: Dict[str, Any]):
        self.state = State(args)
        handler = type("BoundHandler", (Handler,), {"state": self.state})
        ThreadingHTTPServer.allow_reuse_address = True
        ThreadingHTTPServer.daemon_threads = True
        self.httpd = ThreadingHTTPServer((args.get("host", "127.0.0.1"), int(args.get("port", 8080))), handler)
        self.host, self.port = self.httpd.server_address[:2]
        self.thread = threading.Thread(target=self.httpd.serve_forever, name="http", daemon=True)

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def start(self) -> None:
        self.thread.start()
        events.emit("bound", url=self.url, host=self.host, port=self.port)

    def ready(self, engine: Engine, template=None, cache_bytes: int = 0, queue_depth: int = 64) -> None:
        self.state.attach(engine, template, cache_bytes, queue_depth)
        events.emit("ready", url=self.url, model=self.state.model_id, ctx=engine.slot_ctx, slots=engine.n_slots,
                    place=self.state.args.get("_place_word", ""))

    def wait(self) -> int:
        self.state.stop_event.wait()
        return self.stop()

    def stop(self) -> int:
        st = self.state
        if st.phase != "failed":
            st.phase = "stopping"
        if st.worker:
            st.worker.shutdown()
        self.httpd.shutdown()
        self.httpd.server_close()
        if st.engine:
            st.engine.close()
        events.emit("stopped", cause=st.stop_cause or "signal", code=st.exit_code)
        return st.exit_code
