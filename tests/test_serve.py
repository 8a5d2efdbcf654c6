"""HTTP contract on the mock engine (no model, no card), as the reference tests its server
(``crates/serve/tests/*.rs`` on ``MockEngine``)."""
import json
import threading
import time
import urllib.error
import urllib.request

import pytest

from bloomery_b200.serve.api import Server
from bloomery_b200.serve.chat import ChatTemplate
from bloomery_b200.serve.engine import MockEngine
from bloomery_b200.utils import flags


@pytest.fixture()
def server(tmp_path):
    opts = flags.parse(["--port", "0", "--mock", "--slot-save-path", str(tmp_path)])
    s = Server(opts)
    s.start()
    s.ready(MockEngine(n_slots=2, slot_ctx=512), ChatTemplate(), 1 << 20)
    yield s
    s.state.stop_event.set()
    s.stop()


def call(s, path, body=None, method=None, headers=None):
    data = json.dumps(body).encode() if body is not None else None
    req = urllib.request.Request(s.url + path, data=data, method=method or ("POST" if data is not None else "GET"),
                                 headers={"Content-Type": "application/json", **(headers or {})})
    try:
        r = urllib.request.urlopen(req)
        raw = r.read()
        return r.status, (json.loads(raw) if raw[:1] in (b"{", b"[") else raw.decode())
    except urllib.error.HTTPError as e:
        raw = e.read()
        return e.code, (json.loads(raw) if raw[:1] == b"{" else raw.decode())


def test_loading_then_ready():
    opts = flags.parse(["--port", "0", "--mock"])
    s = Server(opts)
    s.start()
    code, body = call(s, "/health")
    assert code == 503 and body["error"]["message"] == "Loading model" and body["error"]["phase"] == "plan"
    code, body = call(s, "/completion", {"prompt": "x"})
    assert code == 503
    s.ready(MockEngine(), ChatTemplate(), 0)
    assert call(s, "/health")[0] == 200
    s.state.stop_event.set()
    assert s.stop() == 0


def test_completion_echo_and_cache(server):
    code, r = call(server, "/completion", {"prompt": "hello world", "n_predict": 64, "temperature": 0})
    assert code == 200 and r["content"] == "hello world" and r["stop_type"] == "eos"
    assert r["tokens_evaluated"] == 11 and r["tokens_cached"] == 0 and r["timings"]["predicted_n"] == 11
    code, r = call(server, "/completion", {"prompt": "hello world, again", "n_predict": 3, "temperature": 0})
    assert r["tokens_cached"] >= 11 and r["stop_type"] == "limit" and r["content"] == "hel"
    code, r = call(server, "/completion", {"prompt": "hello world, again", "n_predict": 3, "cache_prompt": False})
    assert r["tokens_cached"] == 0


def test_stop_strings_and_token_prompt(server):
    code, r = call(server, "/completion", {"prompt": "abcdefgh", "stop": ["de"], "temperature": 0})
    assert r["content"] == "abc" and r["stop_type"] == "word" and r["stopping_word"] == "de"
    code, r = call(server, "/completion", {"prompt": [104, 105], "n_predict": 8, "temperature": 0})
    assert r["content"] == "hi"
    code, r = call(server, "/completion", {"prompt": [70000]})
    assert code == 400 and "vocabulary" in r["error"]["message"]


def test_unknown_field_ignored_unsupported_refused(server):
    code, r = call(server, "/completion", {"prompt": "ab", "n_predict": 2, "some_future_field": 1})
    assert code == 200
    code, r = call(server, "/completion", {"prompt": "ab", "grammar": "root ::= x"})
    assert code == 400 and "grammar" in r["error"]["message"]


def test_openai_completion_and_chat(server):
    code, r = call(server, "/v1/completions", {"prompt": "xyz", "max_tokens": 2, "temperature": 0})
    assert r["object"] == "text_completion" and r["choices"][0]["text"] == "xy" and r["choices"][0]["finish_reason"] == "length"
    assert r["usage"]["completion_tokens"] == 2
    code, r = call(server, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5})
    assert r["object"] == "chat.completion" and r["choices"][0]["message"]["role"] == "assistant"
    assert r["usage"]["prompt_tokens"] > 10
    code, r = call(server, "/v1/chat/completions", {"messages": []})
    assert code == 400


def test_chat_stream_sse(server):
    req = urllib.request.Request(server.url + "/v1/chat/completions", data=json.dumps(
        {"messages": [{"role": "user", "content": "stream"}], "max_tokens": 4, "stream": True,
         "stream_options": {"include_usage": True}}).encode())
    raw = urllib.request.urlopen(req).read().decode()
    events = [json.loads(l[6:]) for l in raw.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
    assert raw.rstrip().endswith("data: [DONE]")
    assert events[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(e["choices"][0]["delta"].get("content") or "" for e in events)
    assert len(text) == 4 and events[-1]["choices"][0]["finish_reason"] == "length" and events[-1]["usage"]["completion_tokens"] == 4


def test_chat_stream_sends_a_call_as_it_is_written(server):
    """A streamed chat reply sends a call in OpenAI's shape: a first delta with index, id, type and the name, then
    argument fragments; a call the token limit cuts ends with finish_reason length."""
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
                 "type": "object", "properties": {"unit": {"enum": ["c", "f"]}, "days": {"type": "integer"}}, "required": ["unit", "days"]}}}]
    body = {"messages": [{"role": "user", "content": "weather"}], "tools": tools, "stream": True, "max_tokens": 128,
            "tool_choice": {"type": "function", "function": {"name": "get_weather"}}}

    def events_of(b):
        req = urllib.request.Request(server.url + "/v1/chat/completions", data=json.dumps(b).encode())
        raw = urllib.request.urlopen(req).read().decode()
        assert raw.rstrip().endswith("data: [DONE]")
        return [json.loads(l[6:]) for l in raw.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
    ev = events_of(body)
    deltas = [c for e in ev if "choices" in e for c in (e["choices"][0]["delta"].get("tool_calls") or [])]
    assert deltas[0]["index"] == 0 and deltas[0]["type"] == "function" and deltas[0]["id"] and deltas[0]["function"] == {
        "name": "get_weather", "arguments": ""}
    assert len(deltas) > 3 and all("name" not in d["function"] for d in deltas[1:])
    args = json.loads("".join(d["function"]["arguments"] for d in deltas))
    assert args["unit"] in ("c", "f") and isinstance(args["days"], int)
    assert ev[-1]["choices"][0]["finish_reason"] == "tool_calls"
    assert not "".join(e["choices"][0]["delta"].get("content") or "" for e in ev if "choices" in e).strip()
    cut = events_of(dict(body, max_tokens=60))
    assert cut[-1]["choices"][0]["finish_reason"] == "length"
    assert any(e["choices"][0]["delta"].get("tool_calls") for e in cut if "choices" in e)


def test_systemone_on_a_generative_model():
    """The decision models' request answered by the served model: every question is one pick of the walk, the scores are
    the logits of the tokens the options start with, and the body follows the decision models' formulas."""
    body = {"state": "User: what is the weather in Seoul tomorrow?", "questions": {
        "tool": {"type": "choice", "instructions": "Which tool next?", "criteria": {"web_search": "Look it up", "calculator": "Arithmetic", "none": "Answer"}},
        "urgency": {"type": "score", "criteria": ["Can wait", "This week", "Today"]},
        "outage": {"type": "noul"},
        "twin": {"type": "choice", "criteria": {"ab": "first", "ac": "second"}}}}      # told apart after the shared "a
    server = Server(flags.parse(["--port", "0", "--mock"]))
    server.start()
    server.ready(MockEngine(n_slots=1, slot_ctx=4096), ChatTemplate(), 1 << 20)
    code, r = call(server, "/v1/systemone", body)
    assert code == 200, r
    assert list(r) == ["model", "answers", "usage", "timings"] and list(r["answers"]) == ["tool", "urgency", "outage", "twin"]
    tool, urg, out, twin = (r["answers"][k] for k in ("tool", "urgency", "outage", "twin"))
    assert tool["type"] == "choice" and tool["choice"] in body["questions"]["tool"]["criteria"]
    assert list(tool["probabilities"]) == ["web_search", "calculator", "none"] and abs(sum(tool["probabilities"].values()) - 1) < 1e-3
    assert tool["probabilities"][tool["choice"]] == max(tool["probabilities"].values())
    u = 1 / 3
    assert abs(tool["confidence"] - max(0.0, (max(tool["probabilities"].values()) - u) / (1 - u))) < 2e-3
    assert urg["type"] == "score" and urg["legend"] == {"0": "Can wait", "1": "This week", "2": "Today"}
    assert abs(urg["score"] - sum(i * urg["probabilities"][str(i)] for i in range(3))) < 2e-3 and 0 <= urg["confidence"] <= 1
    assert out["type"] == "noul" and 0 <= out["noul"] <= 1
    assert twin["choice"] in ("ab", "ac") and list(twin["probabilities"]) == ["ab", "ac"]
    assert r["usage"]["input_tokens"] > 0 and r["usage"]["output_tokens"] > 0 and r["timings"]["cache_n"] >= 0
    # the same request again restores its prompt from the cache
    assert call(server, "/v1/systemone", body)[1]["timings"]["cache_n"] > 0
    for bad, status in (({"questions": {"q": {"type": "noul"}}}, 400), ({"state": "s", "questions": {}}, 400),
                        ({"state": "s", "questions": {"q": {"type": "rank"}}}, 400),
                        ({"state": "s", "questions": {"q": {"type": "choice", "criteria": ["a"]}}}, 400),
                        ({"state": "s", "questions": {"q": {"type": "score", "criteria": ["only"]}}}, 400),
                        ({"state": "s", "questions": {"q": {"type": "noul"}}, "videos": ["x"]}, 501),
                        ({"state": "s", "questions": {"q": {"type": "noul"}}, "images": ["data:image/png;base64,AA=="]}, 501),
                        ({"state": "s", "questions": {"q": {"type": "noul"}}, "cache_prompt": "yes"}, 400)):
        assert call(server, "/v1/systemone", bad)[0] == status, bad
    server.state.stop_event.set()
    server.stop()


def test_anthropic_and_responses(server):
    code, r = call(server, "/v1/messages", {"messages": [{"role": "user", "content": "yo"}], "max_tokens": 3, "system": "be brief"})
    assert r["type"] == "message" and r["stop_reason"] == "max_tokens" and r["content"][0]["type"] == "text"
    code, r = call(server, "/v1/messages", {"messages": [{"role": "user", "content": "yo"}]})
    assert code == 400 and r["type"] == "error"
    code, r = call(server, "/v1/messages/count_tokens", {"messages": [{"role": "user", "content": "yo"}]})
    assert r["input_tokens"] > 0
    code, r = call(server, "/v1/responses", {"input": "abc", "max_output_tokens": 3})
    assert r["object"] == "response" and r["status"] == "incomplete" and len(r["output_text"]) == 3
    rid = r["id"]
    assert call(server, f"/v1/responses/{rid}")[1]["id"] == rid
    code, r2 = call(server, "/v1/responses", {"input": "more", "previous_response_id": rid, "max_output_tokens": 2})
    assert code == 200 and r2["usage"]["input_tokens"] > r["usage"]["input_tokens"]
    assert call(server, f"/v1/responses/{rid}", method="DELETE")[1]["deleted"] is True
    assert call(server, f"/v1/responses/{rid}")[0] == 404


def test_tokenize_props_slots_metrics_models(server):
    assert call(server, "/tokenize", {"content": "ab"})[1] == {"tokens": [97, 98]}
    assert call(server, "/detokenize", {"tokens": [97, 98]})[1] == {"content": "ab"}
    assert "<|im_start|>user" in call(server, "/apply-template", {"messages": [{"role": "user", "content": "q"}]})[1]["prompt"]
    p = call(server, "/props")[1]
    assert p["total_slots"] == 2 and p["default_generation_settings"]["params"]["top_k"] == 40
    assert len(call(server, "/slots")[1]) == 2
    assert "llamacpp:prompt_tokens_total" in call(server, "/metrics")[1]
    assert call(server, "/v1/models")[1]["data"][0]["id"] == "mock-echo"
    assert call(server, "/api/tags")[1]["models"][0]["name"] == "mock-echo"
    assert call(server, "/nope")[0] == 404


def test_slot_save_restore_erase(server):
    call(server, "/completion", {"prompt": "remember me", "n_predict": 2, "id_slot": 0})
    code, r = call(server, "/slots/0?action=save", {"filename": "s.bin"})
    assert code == 200 and r["n_saved"] > 0
    code, r = call(server, "/slots/0?action=erase", {})
    assert r["n_erased"] > 0
    code, r = call(server, "/slots/0?action=restore", {"filename": "s.bin"})
    assert code == 200 and r["n_restored"] > 0
    assert call(server, "/slots/0?action=bogus", {})[0] == 400
    assert call(server, "/slots/9?action=erase", {})[0] == 404


def test_two_concurrent_requests_share_rounds():
    opts = flags.parse(["--port", "0", "--mock"])
    server = Server(opts)
    server.start()
    server.ready(MockEngine(n_slots=2, slot_ctx=512, step_delay=0.003), ChatTemplate(), 0)
    out = [None, None]

    def go(i):
        out[i] = call(server, "/completion", {"prompt": "abcdefghijklmnopqrstuvwxyz" * 2 + str(i), "temperature": 0})[1]
    ts = [threading.Thread(target=go, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out[0]["content"].endswith("0") and out[1]["content"].endswith("1")
    assert 2 in server.state.worker.rounds_by_width          # one decode round served both slots
    server.state.stop_event.set()
    server.stop()


def test_json_mode(server):
    code, r = call(server, "/completion", {"prompt": '{"a": [1, 2, {"b": null}]} trailing', "temperature": 0,
                                            "response_format": {"type": "json_object"}})
    assert json.loads(r["content"]) == {"a": [1, 2, {"b": None}]}


def test_schema_program_forces_keys_without_sampling(server):
    """A schema that compiles to a segment program: the echo engine wants to write spaces and other keys, the program
    keeps the canonical object, and its literal text is taken through the jump arm."""
    schema = {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "boolean"}}, "required": ["a", "b"]}
    code, r = call(server, "/completion", {"prompt": '{"a":   41, "zzz": 1, "b": true} trailing', "temperature": 0, "n_predict": 64,
                                            "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}})
    assert code == 200
    got = json.loads(r["content"])
    assert list(got) == ["a", "b"] and isinstance(got["a"], int) and isinstance(got["b"], bool)
    assert r["content"].startswith('{"a": ') and getattr(server.state.worker, "jumped", 0) >= 3


def test_structured_output_samples_from_the_masked_row(server):
    """Unset, a structured-output request decodes greedily; a positive temperature draws with the request's sampler among
    the ids the schema allows, so every draw is a valid document and the seed picks among the options."""
    schema = {"type": "object", "properties": {"pick": {"enum": ["alpha", "beta", "gamma", "delta"]}}, "required": ["pick"]}
    body = {"prompt": "choose", "n_predict": 48, "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}}
    greedy = {call(server, "/completion", dict(body, seed=s))[1]["content"] for s in range(3)}
    assert len(greedy) == 1 and json.loads(greedy.pop())["pick"] in schema["properties"]["pick"]["enum"]
    seen = set()
    for s in range(12):
        code, r = call(server, "/completion", dict(body, seed=s, temperature=3.0, top_k=0, top_p=1.0, min_p=0.0))
        assert code == 200
        seen.add(json.loads(r["content"])["pick"])
    assert seen <= set(schema["properties"]["pick"]["enum"]) and len(seen) >= 2
    same = [call(server, "/completion", dict(body, seed=5, temperature=3.0, top_k=0, top_p=1.0, min_p=0.0))[1]["content"] for _ in range(2)]
    assert same[0] == same[1]


def test_open_think_span_json_document_and_forced_call():
    """On a template that opens the think span itself, a JSON response_format closes the span at once and writes the
    document after it; a forced call leaves the span to the model and starts after its close."""
    from bloomery_b200.serve.chat import CHATML
    s = Server(flags.parse(["--port", "0", "--mock"]))
    s.start()
    s.ready(MockEngine(n_slots=1, slot_ctx=1024), ChatTemplate(CHATML.rstrip() + "<think>\n"), 0)
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}
    msgs = [{"role": "user", "content": "answer"}]
    code, r = call(s, "/v1/chat/completions", {"messages": msgs, "max_tokens": 64, "reasoning_format": "none",
                                                "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}})
    assert code == 200, r
    text = r["choices"][0]["message"]["content"]
    assert text.startswith("</think>") and isinstance(json.loads(text[len("</think>"):])["ok"], bool)
    code, r = call(s, "/v1/chat/completions", {"messages": msgs, "max_tokens": 64,
                                                "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}})
    assert code == 200 and isinstance(json.loads(r["choices"][0]["message"]["content"])["ok"], bool)
    s.state.stop_event.set()
    s.stop()


def test_forced_tool_choice_writes_one_call(server):
    """``tool_choice`` ``required`` or a named function holds the reply to one call in the template's framing, on the
    chat, Messages and Responses routes; what cannot be forced is a 400 naming the field."""
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
                 "type": "object", "properties": {"unit": {"enum": ["c", "f"]}, "days": {"type": "integer"}}, "required": ["unit", "days"]}}},
             {"type": "function", "function": {"name": "now"}}]
    msgs = [{"role": "user", "content": "weather for 3 days"}]
    code, r = call(server, "/v1/chat/completions", {"messages": msgs, "tools": tools, "max_tokens": 96,
                                                    "tool_choice": {"type": "function", "function": {"name": "get_weather"}}})
    assert code == 200, r
    calls = r["choices"][0]["message"]["tool_calls"]
    assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
    args = json.loads(calls[0]["function"]["arguments"])
    assert args["unit"] in ("c", "f") and isinstance(args["days"], int)
    assert r["choices"][0]["finish_reason"] == "tool_calls"
    code, r = call(server, "/v1/chat/completions", {"messages": msgs, "tools": tools[1:], "max_tokens": 64, "tool_choice": "required"})
    assert code == 200 and r["choices"][0]["message"]["tool_calls"][0]["function"]["name"] == "now"
    # a call the token limit cuts: finish_reason length; the call with what was read once its name is whole, its text before
    forced = {"messages": msgs, "tools": tools, "tool_choice": {"type": "function", "function": {"name": "get_weather"}}}
    code, r = call(server, "/v1/chat/completions", dict(forced, max_tokens=60))
    ch = r["choices"][0]
    assert code == 200 and ch["finish_reason"] == "length" and ch["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert ch["message"]["tool_calls"][0]["function"]["arguments"].startswith('{"unit": ')
    code, r = call(server, "/v1/chat/completions", dict(forced, max_tokens=20))
    ch = r["choices"][0]
    assert code == 200 and ch["finish_reason"] == "length" and "tool_calls" not in ch["message"] and "<tool_call>" in ch["message"]["content"]
    # Anthropic's any / tool and the Responses API's shapes force the same way
    atools = [{"name": "now", "input_schema": {"type": "object", "properties": {}}}]
    code, r = call(server, "/v1/messages", {"messages": msgs, "tools": atools, "max_tokens": 64, "tool_choice": {"type": "any"}})
    assert code == 200 and [b["name"] for b in r["content"] if b["type"] == "tool_use"] == ["now"]
    code, r = call(server, "/v1/responses", {"input": "time?", "tools": [{"type": "function", "name": "now"}], "max_output_tokens": 64,
                                             "tool_choice": {"type": "function", "name": "now"}, "store": False})
    assert code == 200 and [o["name"] for o in r["output"] if o["type"] == "function_call"] == ["now"]
    # a namespace tool is flattened: its functions serve under their bare names and a call carries the namespace
    ns = [{"type": "namespace", "name": "multi_agent_v1", "tools": [{"type": "function", "name": "spawn"}]}]
    code, r = call(server, "/v1/responses", {"input": "go", "tools": ns, "max_output_tokens": 64, "store": False,
                                             "tool_choice": {"type": "function", "name": "spawn"}})
    item = [o for o in r["output"] if o["type"] == "function_call"][0]
    assert code == 200 and item["name"] == "spawn" and item["namespace"] == "multi_agent_v1"
    code, r = call(server, "/v1/responses", {"input": [{"type": "item_reference", "id": "msg_1"}]})
    assert code == 400 and "item_reference" in r["error"]["message"]
    # refusals name the field
    for body, param in (({"tool_choice": {"type": "function", "function": {"name": "absent"}}}, "tool_choice"),
                        ({"tool_choice": "required", "response_format": {"type": "json_object"}}, "response_format"),
                        ({"tool_choice": "sometimes"}, "tool_choice"),
                        ({"tool_choice": "required", "tools": [{"type": "function", "function": {"name": "f", "parameters": {"anyOf": [{"type": "object"}]}}}]}, "tool_choice")):
        code, r = call(server, "/v1/chat/completions", dict({"messages": msgs, "tools": tools}, **body))
        assert code == 400 and r["error"]["param"] == param, (body, r)
    for kw in ({"type": "string", "pattern": "x+"}, {"type": "object", "properties": {"a": {"type": "integer", "minimum": 3}}},
               {"allOf": [{"type": "string"}]}, {"type": "array", "items": {"type": "string", "minLength": 2}}):
        code, r = call(server, "/completion", {"prompt": "x", "response_format": {"type": "json_schema", "json_schema": {"schema": kw}}})
        assert code == 400 and "outside the served subset" in r["error"]["message"], kw
    for body, param in (({"ignore_eos": True}, "ignore_eos"), ({"reasoning_budget": 8}, "reasoning_budget")):
        code, r = call(server, "/completion", dict({"prompt": "x", "response_format": {"type": "json_object"}}, **body))
        assert code == 400 and r["error"]["param"] == param


def test_key_file_limits_answer_429(tmp_path):
    kf = tmp_path / "keys.txt"
    kf.write_text("# keys\nslow rate=1/m burst=1\nfree\n")
    opts = flags.parse(["--port", "0", "--mock", "--api-key-file", str(kf)])
    s = Server(opts)
    s.start()
    s.ready(MockEngine(), ChatTemplate(), 0)
    slow, free = {"Authorization": "Bearer slow"}, {"Authorization": "Bearer free"}
    assert call(s, "/completion", {"prompt": "ab", "n_predict": 2}, headers=slow)[0] == 200
    code, r = call(s, "/completion", {"prompt": "ab", "n_predict": 2}, headers=slow)
    assert code == 429 and r["error"]["type"] == "rate_limit_error"
    assert call(s, "/tokenize", {"content": "ab"}, headers=slow)[0] == 200          # not a generating route: no place taken
    for _ in range(3):
        assert call(s, "/completion", {"prompt": "ab", "n_predict": 2}, headers=free)[0] == 200
    assert call(s, "/completion", {"prompt": "ab"}, headers={"Authorization": "Bearer nope"})[0] == 401
    s.state.stop_event.set()
    s.stop()


def test_key_scopes_answer_403_outside_their_routes(tmp_path):
    kf = tmp_path / "keys.txt"
    kf.write_text("app scope=inference\nwatch scope=read\nroot\n")
    s = Server(flags.parse(["--port", "0", "--mock", "--api-key-file", str(kf), "--slot-save-path", str(tmp_path)]))
    s.start()
    s.ready(MockEngine(), ChatTemplate(), 0)
    app, watch, root = ({"Authorization": f"Bearer {k}"} for k in ("app", "watch", "root"))
    assert call(s, "/completion", {"prompt": "ab", "n_predict": 2}, headers=app)[0] == 200
    code, r = call(s, "/props", headers=app)
    assert code == 403 and r["error"]["type"] == "permission_error"
    assert call(s, "/props", headers=watch)[0] == 200 and call(s, "/metrics", headers=watch)[0] == 200
    assert call(s, "/completion", {"prompt": "ab"}, headers=watch)[0] == 403
    assert call(s, "/v1/models", headers=app)[0] == 200 and call(s, "/v1/models", headers=watch)[0] == 200
    assert call(s, "/slots/0?action=erase", {}, headers=app)[0] == 403
    assert call(s, "/slots/0?action=erase", {}, headers=root)[0] == 200
    assert call(s, "/health")[0] == 200
    s.state.stop_event.set()
    s.stop()
    kf.write_text("app scope=inference\napp scope=read\n")
    with pytest.raises(ValueError, match="given twice"):
        Server(flags.parse(["--port", "0", "--mock", "--api-key-file", str(kf)]))


def test_api_key_and_shutdown():
    opts = flags.parse(["--port", "0", "--mock", "--api-key", "sekret"])
    s = Server(opts)
    s.start()
    s.ready(MockEngine(), ChatTemplate(), 0)
    assert call(s, "/props")[0] == 401
    assert call(s, "/props", headers={"Authorization": "Bearer sekret"})[0] == 200
    assert call(s, "/health")[0] == 200
    assert call(s, "/shutdown", {}, headers={"Authorization": "Bearer sekret"})[0] == 200
    assert s.state.stop_event.wait(2)
    assert s.stop() == 0


def test_engine_failure_is_fatal():
    opts = flags.parse(["--port", "0", "--mock"])
    s = Server(opts)
    s.start()
    s.ready(MockEngine(fail_at=3), ChatTemplate(), 0)
    code, r = call(s, "/completion", {"prompt": "abcdef", "temperature": 0})
    assert code == 500 and "engine failure" in r["error"]["message"]
    assert s.state.stop_event.wait(2)
    assert call(s, "/health")[0] == 503
    assert s.stop() == 70


def test_speculative_drafts_change_passes_not_tokens():
    """With the n-gram draft on, the echo engine's text is unchanged and several tokens settle per round."""
    from bloomery_b200.runtime.speculative import NgramDraft, WidthChooser
    outs = []
    for drafting in (False, True):
        s = Server(flags.parse(["--port", "0", "--mock"]))
        s.start()
        s.ready(MockEngine(n_slots=1, slot_ctx=512), ChatTemplate(), 0)
        if drafting:
            s.state.worker.enable_drafting(NgramDraft(), WidthChooser(max_width=7))
        code, r = call(s, "/completion", {"prompt": "abcabcabcabc xyz abcabcabcabc xyz", "temperature": 0, "n_predict": 40})
        outs.append((r["content"], r["timings"]["draft_n"], r["timings"]["draft_n_accepted"], s.state.worker.metrics.get("n_decode_total")))
        if drafting:
            text = call(s, "/metrics")[1]
            by_depth = [ln for ln in text.splitlines() if ln.startswith("llamacpp:spec_decode_num_draft_tokens_by_depth_total")]
            assert by_depth and 'source="ngram",depth="0"' in by_depth[0]
            assert sum(int(ln.rsplit(" ", 1)[1]) for ln in by_depth) == r["timings"]["draft_n"]          # the depths sum to the total
            acc = [ln for ln in text.splitlines() if ln.startswith("llamacpp:spec_decode_num_accepted_tokens_by_depth_total")]
            assert sum(int(ln.rsplit(" ", 1)[1]) for ln in acc) == r["timings"]["draft_n_accepted"]
            assert "llamacpp:round_seconds_by_width_total{width=" in text
        s.state.stop_event.set()
        s.stop()
    assert outs[0][0] == outs[1][0]                      # same text
    assert outs[0][1] == 0 and outs[1][1] > 0 and outs[1][2] > 0
    assert outs[1][3] < outs[0][3]                       # fewer decode rounds for the same tokens


def test_sampled_and_structured_requests_draft_to_the_same_ids():
    """A sampled request (seeded), one with a logit bias and one asking for probabilities take the same ids with the
    n-gram draft on as without it: every kept id is the request's own pick from its verified row."""
    from bloomery_b200.runtime.speculative import NgramDraft, WidthChooser
    bodies = [{"prompt": "abcabcabcabc xyz abcabcabcabc xyz", "temperature": 0.9, "seed": 11, "n_predict": 40, "top_k": 2},
              {"prompt": "abcabcabcabc xyz abcabcabcabc xyz", "temperature": 0, "n_predict": 30, "logit_bias": {"98": 5.0}},
              {"prompt": "abcabcabcabc xyz abcabcabcabc xyz", "temperature": 0, "n_predict": 20, "n_probs": 2}]
    outs = []
    for drafting in (False, True):
        s = Server(flags.parse(["--port", "0", "--mock"]))
        s.start()
        s.ready(MockEngine(n_slots=1, slot_ctx=512), ChatTemplate(), 0)
        if drafting:
            s.state.worker.enable_drafting(NgramDraft(), WidthChooser(max_width=7))
        got = []
        for b in bodies:
            code, r = call(s, "/completion", dict(b))
            assert code == 200
            got.append((r["content"], r["tokens_predicted"], [p["id"] for p in r.get("completion_probabilities", [])] if "n_probs" in b else None))
        outs.append((got, s.state.worker.metrics.get("draft_accepted_total")))
        s.state.stop_event.set()
        s.stop()
    assert outs[0][0] == outs[1][0]
    assert outs[0][1] == 0 and outs[1][1] > 0


@pytest.mark.parametrize("native", ["0", "1"])
def test_cpu_engine_serves_a_gguf_file(tmp_path, native):
    """``-dev none``: the process opens a GGUF file, plans, loads the CPU engine and answers greedy text equal
    to the oracle's continuation; a second request reuses the cached prefix; a third runs with n-gram drafting.  The
    native host step (the default) and the plain PyTorch model both serve it."""
    import os
    import subprocess
    import sys
    import torch
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.cpu_ref import CpuModel
    from bloomery_b200.models.spec import tiny_qwen3moe
    spec = tiny_qwen3moe()
    spec.vocab, spec.n_layer = 512, 2
    path = str(tmp_path / "tiny.gguf")
    items = list(W.synth_tensors(spec, "cpu", seed=9))
    W.write_gguf(spec, iter(items), path)
    import socket
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    env = dict(os.environ, BLOOMERY_DRAFT="ngram", BLOOMERY_HOST_NATIVE=native)
    proc = subprocess.Popen([sys.executable, "-m", "bloomery_b200.serve", "-m", path, "-dev", "none", "--port", str(port),
                             "-c", "4096", "-np", "2", "--no-warmup"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE)

    class S:
        url = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            try:
                if call(S, "/health")[0] == 200:
                    break
            except Exception:
                pass
            time.sleep(0.1)
        else:
            raise AssertionError("server did not become ready: " + proc.stderr.read().decode()[-2000:])
        prompt = [3, 77, 200, 411, 9, 3, 77, 200]
        code, r = call(S, "/completion", {"prompt": prompt, "n_predict": 6, "temperature": 0, "return_tokens": True})
        assert code == 200, r
        want = CpuModel(W.Weights.from_items(spec, iter(items), "cpu")).generate(prompt, 6)
        if native == "0":
            assert r["tokens"] == want, (r["tokens"], want)
        else:
            # the native step sums in another order: on flat random-init logits a near tie may pick another id
            assert len(r["tokens"]) == 6 and r["tokens"][0] == want[0], (r["tokens"], want)
            want = r["tokens"]
        code, r2 = call(S, "/completion", {"prompt": prompt + want[:2], "n_predict": 4, "temperature": 0, "return_tokens": True})
        assert code == 200 and r2["tokens"] == want[2:6] and r2["tokens_cached"] >= len(prompt)
        code, props = call(S, "/props")
        assert code == 200 and props["model"]["engine"] == ("cpu-native" if native == "1" else "cpu")
        code, emb = call(S, "/v1/embeddings", {"input": ["abc", "abd"]})
        assert code == 200 and len(emb["data"]) == 2 and len(emb["data"][0]["embedding"]) == spec.hidden
        v0, v1 = (torch.tensor(d["embedding"]) for d in emb["data"])
        assert abs(float(v0.norm()) - 1.0) < 1e-4 and 0.2 < float(v0 @ v1) < 0.99999
    finally:
        proc.terminate()
        proc.wait(timeout=20)


def test_worker_hands_sampling_to_an_engine_that_samples_itself():
    """An engine with ``device_sampling`` gets the request's chain, draw number and recent window with the rows and
    returns the sampled id; the host sampler is not consulted and no logits are asked for.  Requests that need the
    logits on the host (logit_bias, n_probs, constraints) stay on the host chain."""
    from bloomery_b200.serve.sampler import Sampler

    class SelfSampling(MockEngine):
        device_sampling = True

        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            self.seen = []

        def step(self, rows, want_logits=True, sampling=None):
            res = super().step(rows, want_logits=True)
            out = []
            for i, (tok, lg) in enumerate(res):
                sp = sampling[i] if sampling is not None else None
                if sp is not None:
                    params, n_drawn, recent = sp
                    self.seen.append((n_drawn, list(recent), want_logits))
                    s = Sampler(params)
                    for _ in range(n_drawn):                 # replay the stream up to this draw
                        s.rng.next_f64()
                    used = [0]
                    real = s.rng.next_f64
                    s.rng.next_f64 = lambda: (used.__setitem__(0, used[0] + 1), real())[1]
                    out.append((s.sample(lg, recent), None))
                    sp[1] = n_drawn + used[0]                # a token with one surviving candidate draws nothing
                else:
                    out.append((tok, lg if want_logits else None))
            return out

    def run(engine, body):
        s = Server(flags.parse(["--port", "0", "--mock"]))
        s.start()
        s.ready(engine, ChatTemplate(), 0)
        code, r = call(s, "/completion", body)
        s.state.stop_event.set()
        s.stop()
        assert code == 200, r
        return r

    body = {"prompt": "hello hello hello", "temperature": 0.9, "top_k": 20, "seed": 7, "n_predict": 12, "repeat_penalty": 1.2,
            "repeat_last_n": 8}
    eng = SelfSampling(n_slots=1, slot_ctx=512)
    on_card = run(eng, body)
    on_host = run(MockEngine(n_slots=1, slot_ctx=512), body)
    assert on_card["content"] == on_host["content"]                       # same chain, same seed, same draws
    ds = [d for d, _, _ in eng.seen]
    assert ds == sorted(ds) and ds[0] == 0 and len(ds) >= 1
    assert all(len(r) <= 8 for _, r, _ in eng.seen) and not any(w for _, _, w in eng.seen)
    eng2 = SelfSampling(n_slots=1, slot_ctx=512)
    run(eng2, dict(body, n_probs=2))
    assert eng2.seen == []                                                # top-probabilities need the host's logits


def test_one_stderr_line_a_request(server, capfd):
    capfd.readouterr()
    code, r = call(server, "/completion", {"prompt": "hello there", "n_predict": 3, "temperature": 0})
    assert code == 200
    err = capfd.readouterr().err
    line = next(ln for ln in err.splitlines() if ln.startswith("bloomery-serve: request "))
    assert " /completion: prompt " in line and " ids/s; generated 3 ids in " in line and line.endswith("/512")
    assert "stop length; ctx " in line


def test_long_generation_says_it_is_still_generating(capfd):
    s = Server(flags.parse(["--port", "0", "--mock"]))
    s.start()
    s.ready(MockEngine(n_slots=1, slot_ctx=512, step_delay=0.01), ChatTemplate(), 0)
    s.state.worker.generating_every = 0.05
    capfd.readouterr()
    assert call(s, "/completion", {"prompt": "abcdefghijklmnopqrstuvwxyz", "n_predict": 24, "temperature": 0})[0] == 200
    err = capfd.readouterr().err
    assert sum(1 for ln in err.splitlines() if ": generating, " in ln) >= 2
    # the rounds' card wait is counted by width beside their whole time, and never passes it
    text = call(s, "/metrics")[1]
    val = lambda name: float(next(ln for ln in text.splitlines() if ln.startswith(name)).split()[-1])       # noqa: E731
    assert 0 < val('llamacpp:round_card_wait_seconds_total{width="1"}') <= val('llamacpp:round_seconds_by_width_total{width="1"}')
    assert val("llamacpp:card_wait_seconds_total") > 0
    s.state.stop_event.set()
    s.stop()


def test_reasoning_budget_loop_and_refused_fields(server):
    # the budget writes the closing tag for the model once the span has used its ids
    code, r = call(server, "/completion", {"prompt": "<think>abcdefgh</think>done", "temperature": 0, "n_predict": 24,
                                           "reasoning_budget": 4})
    assert code == 200 and r["content"].startswith("<think>abc</think>")
    # a span that repeats itself ends with its own stop type
    big = Server(flags.parse(["--port", "0", "--mock"]))
    big.start()
    big.ready(MockEngine(n_slots=1, slot_ctx=2048), ChatTemplate(), 0)
    code, r = call(big, "/completion", {"prompt": "<think>" + "a" * 400, "temperature": 0, "n_predict": 390, "reasoning_loop": True})
    assert code == 200 and r["stop_type"] == "reasoning_loop" and 256 < r["tokens_predicted"] < 330
    code, r = call(big, "/completion", {"prompt": "<think>" + "a" * 400, "temperature": 0, "n_predict": 390})
    assert r["stop_type"] == "limit"                                   # off unless asked
    big.state.stop_event.set()
    big.stop()
    for body, word in (({"reasoning_budget": -3}, "reasoning_budget"), ({"reasoning_loop": "yes"}, "reasoning_loop"),
                       ({"temperature": "hot"}, "temperature"), ({"top_p": float("nan")}, "top_p"), ({"typical_p": 0.5}, "typical_p"),
                       ({"mirostat": 2}, "mirostat"), ({"samplers": ["top_p", "top_k"]}, "samplers"),
                       ({"samplers": ["top_k", "tail_free"]}, "tail_free"), ({"n_predict": -5}, "n_predict"), ({"n": 3}, "'n'")):
        code, r = call(server, "/completion", {"prompt": "ab", **body})
        assert code == 400 and word in r["error"]["message"], (body, r)
    assert call(server, "/completion", {"prompt": "ab", "n_predict": 2, "typical_p": 1.0, "mirostat": 0, "samplers": ["top_k", "temperature"],
                                        "temperature": None})[0] == 200
    code, r = call(server, "/tokenize", {"content": 5})
    assert code == 400 and "content" in r["error"]["message"]
    code, r = call(server, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "reasoning_effort": "loud"})
    assert code == 400 and "reasoning_effort" in r["error"]["message"]
    code, r = call(server, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "reasoning_effort": "none",
                                                    "chat_template_kwargs": {"enable_thinking": True}, "max_tokens": 2})
    assert code == 400 and "opposite" in r["error"]["message"]
    assert call(server, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "reasoning_effort": "low",
                                                 "max_tokens": 2})[0] == 200


def test_several_choices_of_one_prompt():
    """``n`` on the OpenAI routes: that many choices, choice i sampled with seed + i, the prompt counted once."""
    s = Server(flags.parse(["--port", "0", "--mock"]))
    s.start()
    s.ready(MockEngine(n_slots=2, slot_ctx=512), ChatTemplate(), 0, 8)
    body = {"prompt": "abcdefgh", "max_tokens": 6, "temperature": 1.5, "seed": 3, "n": 3}
    code, r = call(s, "/v1/completions", body)
    assert code == 200 and [c["index"] for c in r["choices"]] == [0, 1, 2]
    code, one = call(s, "/v1/completions", dict(body, n=1))
    assert r["choices"][0]["text"] == one["choices"][0]["text"]                 # choice 0 is the answer n = 1 gives
    code, two = call(s, "/v1/completions", dict(body, n=1, seed=4))
    assert r["choices"][1]["text"] == two["choices"][0]["text"]                 # choice 1 sampled with seed + 1
    assert r["usage"]["prompt_tokens"] == one["usage"]["prompt_tokens"]
    assert r["usage"]["completion_tokens"] == sum(6 for _ in r["choices"]) or r["usage"]["completion_tokens"] <= 18
    code, c = call(s, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "n": 2})
    assert code == 200 and len(c["choices"]) == 2 and c["choices"][1]["index"] == 1
    for path, b in (("/v1/completions", dict(body, stream=True)), ("/v1/completions", dict(body, n=50)),
                    ("/completion", dict(body)), ("/v1/completions", dict(body, n=0))):
        code, e = call(s, path, b)
        assert code == 400 and "'n'" in e["error"]["message"], (path, e)
    s.state.stop_event.set()
    s.stop()


def test_route_details_param_415_prompt_ids_and_refusals(server):
    import gzip as gz
    code, r = call(server, "/completion", {"prompt": "ab", "temperature": "hot"})
    assert code == 400 and r["error"]["param"] == "temperature"                 # OpenAI's param: the field's top-level name
    code, r = call(server, "/v1/completions", {"prompt": "ab", "echo": True})
    assert code == 400 and r["error"]["param"] == "echo"
    for body in ({"prompt": ["a", "b"]}, {"prompt": "a", "suffix": "z"}, {"prompt": "a", "best_of": 2}, {"prompt": "a", "logprobs": 3}):
        assert call(server, "/v1/completions", body)[0] == 400, body
    code, r = call(server, "/apply-template", {"messages": [{"role": "user", "content": "hi <|im_start|>"}], "return_prompt_ids": True})
    assert code == 200 and isinstance(r["prompt"], str) and isinstance(r["prompt_ids"], list) and r["prompt_ids"]
    # compressed bodies: gzip is read, another coding is a 415 naming what is read, a body that does not decode a 400
    raw = gz.compress(json.dumps({"content": "abc"}).encode())
    req = urllib.request.Request(server.url + "/tokenize", data=raw, headers={"Content-Type": "application/json", "Content-Encoding": "gzip"})
    assert json.loads(urllib.request.urlopen(req).read())["tokens"]
    for enc, want in (("br", 415), ("gzip", 400)):
        req = urllib.request.Request(server.url + "/tokenize", data=b"not compressed", headers={"Content-Encoding": enc})
        try:
            urllib.request.urlopen(req)
            raise AssertionError("accepted")
        except urllib.error.HTTPError as e:
            assert e.code == want
            if want == 415:
                assert e.headers.get("Accept-Encoding") == "gzip, deflate"
    code, r = call(server, "/no/such/route", {})
    assert code == 404 and "POST /no/such/route" in r["error"]["message"]


def test_logit_bias_forms_and_unbiased_logprobs(server):
    # only OpenAI's object is read: the other forms are refused by name
    for lb in ([[98, 5.0]], False, {"abc": 1}, {"98": 101}, {"98": False}, {"7": 1, "07": 2}, {"999999": 1}):
        code, r = call(server, "/completion", {"prompt": "ab", "n_predict": 2, "logit_bias": lb})
        assert code == 400 and r["error"]["param"] == "logit_bias", lb
    # the bias moves the pick; the probabilities reported stay the model's own
    base = call(server, "/completion", {"prompt": "abcabc", "temperature": 0, "n_predict": 1, "n_probs": 3})[1]
    first = base["completion_probabilities"][0]
    other = first["top_logprobs"][1]
    code, r = call(server, "/completion", {"prompt": "abcabc", "temperature": 0, "n_predict": 1, "n_probs": 3,
                                           "logit_bias": {str(first["id"]): -100, str(other["id"]): 100}})
    assert code == 200
    got = r["completion_probabilities"][0]
    assert got["id"] == other["id"]
    assert abs(got["logprob"] - other["logprob"]) < 1e-4
    assert [t["id"] for t in got["top_logprobs"]] == [t["id"] for t in first["top_logprobs"]]
    code, r = call(server, "/chat/completions/input_tokens", {"messages": [{"role": "user", "content": "hi"}]})
    assert code == 200 and r["input_tokens"] > 0
    # a developer message is the system message of the same text; /props names the template's thinking switch and the draft
    as_dev = call(server, "/apply-template", {"messages": [{"role": "developer", "content": "be brief"}, {"role": "user", "content": "hi"}]})[1]
    as_sys = call(server, "/apply-template", {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]})[1]
    assert as_dev["prompt"] == as_sys["prompt"] and "developer" not in as_dev["prompt"]
    props = call(server, "/props")[1]
    assert props["thinking_off"] in ("switch", "low_effort", "off_word", "neither") and props["engine"]["draft"]["kind"] == "off"


def test_background_responses_poll_cancel_and_refusals():
    s = Server(flags.parse(["--port", "0", "--mock"]))
    s.start()
    s.ready(MockEngine(n_slots=1, slot_ctx=512, step_delay=0.01), ChatTemplate(), 0)
    code, r = call(s, "/v1/responses", {"input": "abcdefghij", "max_output_tokens": 8, "background": True})
    assert code == 200 and r["status"] == "queued" and "_req" not in r and "_messages" not in r
    rid = r["id"]
    for _ in range(200):
        code, got = call(s, f"/v1/responses/{rid}")
        if got["status"] not in ("queued", "in_progress"):
            break
        time.sleep(0.02)
    assert got["status"] in ("completed", "incomplete") and got["output"]
    # a running one can be cancelled
    code, r2 = call(s, "/v1/responses", {"input": "abcdefghijklmnopqrstuvwxyz" * 3, "max_output_tokens": 200, "background": True})
    code, c = call(s, f"/v1/responses/{r2['id']}/cancel", {})
    assert code == 200 and c["status"] == "cancelled"
    for _ in range(200):
        if call(s, f"/v1/responses/{r2['id']}")[1]["status"] == "cancelled" and s.state.board.busy_count() == 0:
            break
        time.sleep(0.02)
    assert s.state.board.busy_count() == 0 and call(s, f"/v1/responses/{r2['id']}")[1]["status"] == "cancelled"
    assert call(s, "/v1/responses/resp_missing/cancel", {})[0] == 404
    for body in ({"input": "a", "background": True, "stream": True}, {"input": "a", "background": True, "store": False},
                 {"input": "a", "conversation": "conv_1"}):
        assert call(s, "/v1/responses", body)[0] == 400, body
    # previous_response_id continues the conversation without the old instructions
    code, first = call(s, "/v1/responses", {"input": "hello", "instructions": "be brief", "max_output_tokens": 4})
    kept = s.state.responses[first["id"]]["_messages"]
    assert kept[0]["role"] == "user" and all(m.get("content") != "be brief" for m in kept)
    assert call(s, "/v1/responses", {"input": "more", "previous_response_id": first["id"], "max_output_tokens": 4})[0] == 200
    s.state.stop_event.set()
    s.stop()


def test_model_lookup_and_ollama_shapes(server):
    assert call(server, "/v1/models/mock-echo")[0] == 200 and call(server, "/models/mock-echo")[0] == 200
    code, r = call(server, "/v1/models/other")
    assert code == 404 and "mock-echo" in r["error"]["message"]               # names what the server does serve
    code, tags = call(server, "/api/tags")
    assert code == 200 and tags["models"][0]["name"] == "mock-echo"
    code, show = call(server, "/api/show", {"model": "mock-echo"})
    assert code == 200 and "completion" in show["capabilities"] and show["template"]
    assert any(k.endswith(".context_length") and v == 512 for k, v in show["model_info"].items())
    assert call(server, "/api/show", {"model": "other"})[0] == 404
