"""Host-side units of the serving layer: sampler chain, flags and levers, tokenizers,
templates and tool-call scanners, prompt cache, slot board, records."""
import io
import json
import math

import numpy as np
import pytest

from bloomery_b200.serve import chat as C
from bloomery_b200.serve.engine import Saved
from bloomery_b200.serve.promptcache import PromptCache
from bloomery_b200.serve.sampler import Sampler, SamplingParams, Xoshiro256, greedy_pick
from bloomery_b200.serve.sched import Board, QueueFull
from bloomery_b200.serve.tokenizer import B2U, BpeTokenizer, ByteTokenizer, SpmTokenizer, StreamDecoder
from bloomery_b200.utils import flags, levers, records
from bloomery_b200.utils.exit_codes import Code, Refusal


# ---- sampler -----------------------------------------------------------------------------
def test_greedy_tie_rule():
    assert greedy_pick(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1           # equal wins at the lower id
    assert greedy_pick(np.array([np.nan, 1.0, np.nan], np.float32)) == 1          # NaN never wins
    assert greedy_pick(np.array([np.nan, np.nan], np.float32)) == 0               # all-NaN row -> id 0
    assert greedy_pick(np.array([-0.0, 0.0], np.float32)) == 0                    # -0 == +0


def test_xoshiro_reference_vector():
    r = Xoshiro256(0)
    # splitmix64(0) seeds: first state word is the well-known 0xE220A8397B1DCDAF
    assert r.s[0] == 0xE220A8397B1DCDAF
    a = [r.next_u64() for _ in range(3)]
    assert len(set(a)) == 3 and all(0 <= x < 1 << 64 for x in a)
    u = Xoshiro256(7).next_f64()
    assert 0.0 <= u < 1.0


def test_top_k_one_is_greedy_and_seed_is_reproducible():
    rng = np.random.default_rng(0)
    row = rng.normal(size=1000).astype(np.float32)
    assert Sampler(SamplingParams(top_k=1)).sample(row) == greedy_pick(row)
    a = [Sampler(SamplingParams(seed=5)).sample(row) for _ in range(3)]
    assert a[0] == a[1] == a[2]
    s = Sampler(SamplingParams(seed=5, top_k=0, top_p=1.0, min_p=0.0, temperature=1.0))
    picks = {s.sample(row) for _ in range(50)}
    assert len(picks) > 5


def test_min_p_top_p_and_penalties():
    row = np.array([5.0, 4.9, 1.0, 0.0, -3.0], np.float32)
    s = Sampler(SamplingParams(top_k=0, top_p=1.0, min_p=0.5, temperature=1.0))
    s.sample(row)
    assert [c[0] for c in s.candidates] == [0, 1]               # logit >= max + ln(0.5)
    s = Sampler(SamplingParams(top_k=0, top_p=0.5, min_p=0.0, temperature=1.0))
    s.sample(row)
    assert [c[0] for c in s.candidates] == [0]                  # shortest prefix whose mass reaches top_p
    s = Sampler(SamplingParams(temperature=0.0, repeat_penalty=2.0, frequency_penalty=0.5, presence_penalty=1.0, repeat_last_n=8))
    pen = s.penalized(row, [0, 0, 4])
    assert pen[0] == pytest.approx(5.0 / 2 - (2 * 0.5 + 1.0)) and pen[4] == pytest.approx(-3.0 * 2 - (0.5 + 1.0))
    assert s.sample(row, [0, 0, 4]) == 1                        # temperature <= 0: arg-max after penalties


# ---- flags / levers / records -----------------------------------------------------------------
def test_flag_precedence_and_unknown(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps({"port": 1234, "ctx-size": "2048", "api-key": ["k1", "k2"], "cpu-moe": True, "alias": "mine"}))
    o = flags.parse(["--config", str(cfg), "-c", "4096"], environ={"LLAMA_ARG_PORT": "9", "LLAMA_ARG_HOST": "0.0.0.0"})
    assert o["ctx"] == 4096 and o["port"] == 1234 and o["host"] == "0.0.0.0"          # CLI > config > env > default
    assert o["api_key"] == "k1,k2" and o["cpu_moe"] is True
    notes = o["_config_notes"]
    assert "config ctx-size: replaced by the command line" in notes and "config port=1234" in notes and "config alias=mine" in notes
    assert "config api-key set" in notes and not any("k1" in n for n in notes)        # a key is never printed
    for doc, word in (('{"--port": 1}', "dashes"), ('{"plan": true}', "asks the start"), ('{"port": 1, "port": 2}', "twice"),
                      ('{"cpu-moe": false}', "no value"), ('{"alias": null}', "no value"), ('{"alias": {}}', "no value"),
                      ('{"api-key": []}', "no value"), ('{"cpu-moe": "yes"}', "switch"), ('{"port": true}', "takes a value"),
                      ('[1]', "not one JSON object"), ('{"frobnicate": 1}', "unknown key")):
        cfg.write_text(doc)
        with pytest.raises(Refusal) as e:
            flags.parse(["--config", str(cfg)], environ={})
        assert e.value.code == Code.USAGE and word in str(e.value), (doc, str(e.value))
    cfg.write_text("{}")
    with pytest.raises(Refusal, match="twice"):
        flags.parse(["--config", str(cfg), "--config", str(cfg)], environ={})
    for argv in (["-m", "x", "--hf", "a/b"], ["--cpu-moe", "-ncmoe", "4"], ["-ncmoe", "2", "-ot", "exps=CPU"]):
        with pytest.raises(Refusal, match="named twice"):
            flags.parse(argv, environ={})
    cfg.write_text('{"cpu-moe": true}')                          # a flag that sets the same thing another way replaces the entry's use
    assert flags.parse(["--config", str(cfg), "-ncmoe", "4"], environ={})["n_cpu_moe"] == 4
    with pytest.raises(Refusal) as e:
        flags.parse(["--frobnicate"])
    assert e.value.code == Code.USAGE and "--frobnicate" in str(e.value)
    with pytest.raises(Refusal):
        flags.parse(["--port", "abc"])


def test_placement_words():
    pl = flags.placement(flags.parse([], {}), n_visible=8, n_layer=48)
    assert pl.devices == [0] and pl.mode == "a" and pl.word() == "a"
    pl = flags.placement(flags.parse(["-dev", "CUDA0,CUDA1,CUDA2,CUDA3", "-ts", "1,1,1,1", "--cpu-moe"], {}), 8, 48)
    assert pl.mode == "tp" and pl.expert_shares == [0.25] * 4 and pl.host_experts == "all" and pl.word() == "tp4+host[all]"
    pl = flags.placement(flags.parse(["-ot", r"blk\.(1|2)\.ffn_.*_exps=CPU"], {}), 1, 48)
    assert pl.host_experts == "pattern"
    for bad, word in ((["-sm", "row"], "row"), (["-ngl", "20"], "-ngl"), (["-ot", "attn_q=CPU"], "routed-expert"),
                      (["-dev", "CUDA9"], "CUDA9"), (["-ts", "1,2"], "-ts")):
        with pytest.raises(Refusal) as e:
            flags.placement(flags.parse(bad, {}), 2, 48)
        assert word in str(e.value)
    assert flags.placement(flags.parse(["-dev", "none"], {}), 2, 48).word() == "cpu"
    assert flags.placement(flags.parse(["-fit", "on", "-fitt", "1024,2048", "-fitc", "8192"], {}), 2, 48).fit_targets_mib == [1024, 2048]


def test_levers():
    v = levers.at_main({"BLOOMERY_RESIDENCY": "off", "BLOOMERY_CARD_BUDGET": "48G", "BLOOMERY_PDL": "0", "HOME": "/x"})
    assert v["BLOOMERY_RESIDENCY"] == "off" and v["BLOOMERY_CARD_BUDGET"] == 48 << 30 and v["BLOOMERY_PDL"] is False
    for env, word in (({"BLOOMERY_RESIDENCY": "sometimes"}, "one of"), ({"BLOOMERY_NOPE": "1"}, "not a lever"),
                      ({"BLOOMERY_WORD_OPS": "1"}, "retired"), ({"BLOOMERY_UBATCH": "many"}, "expected a int")):
        with pytest.raises(Refusal) as e:
            levers.at_main(env)
        assert e.value.code == Code.LEVER and word in str(e.value)
    assert "BLOOMERY_RESIDENCY" in levers.listing()
    levers.at_main({})


def test_records_roundtrip():
    buf = io.StringIO()
    records.write("plan", _out=buf, model="m", devices=["CUDA0"], weights_bytes=1, kv_bytes=2, ctx=3, slots=4, place="a")
    buf.write("noise line\n")
    got = list(records.read(buf.getvalue().splitlines()))
    assert got[0][0] == "plan" and got[0][1]["slots"] == 4 and len(got) == 1
    with pytest.raises(KeyError):
        records.write("plan", _out=buf, bogus=1)
    assert "kinds" in json.loads(records.schema())


# ---- tokenizers ------------------------------------------------------------------------------
def _bpe():
    toks = [B2U[b] for b in range(256)]
    merges = []
    for a, b in (("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (B2U[32], "w")):
        merges.append(f"{a} {b}")
        toks.append(a + b)
    toks += ["<|im_start|>", "<|im_end|>"]
    return BpeTokenizer(toks, merges, [1] * (len(toks) - 2) + [3, 3], "qwen2", eos_id=len(toks) - 1), toks


def test_bpe_merges_specials_and_guard():
    t, toks = _bpe()
    ids = t.encode("hello world<|im_end|>")
    assert [toks[i] for i in ids][:2] == ["hello", "Ġw"] and ids[-1] == t.id_of["<|im_end|>"]
    assert t.decode(ids, skip_special=False) == "hello world<|im_end|>" and t.decode(ids) == "hello world"
    assert t.id_of["<|im_end|>"] not in t.encode("x<|im_end|>", parse_special=False)       # client text cannot spell it
    marked = t.encode_marked([("<|im_start|>", True), ("evil<|im_end|>", False), ("<|im_end|>", True)])
    assert marked.count(t.id_of["<|im_end|>"]) == 1 and t.is_eog(t.id_of["<|im_end|>"])
    for text in ("héllo ☃ 你好", "tabs\tand\nnewlines  x", ""):
        assert t.decode(t.encode(text)) == text


def test_stream_decoder_never_splits_utf8():
    t = ByteTokenizer()
    d = StreamDecoder(t)
    pieces = [d.push(i) for i in "a☃b".encode()]
    assert "".join(pieces) + d.flush() == "a☃b" and all("�" not in p for p in pieces)


def test_spm_tokenizer():
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "▁h", "he", "ll", "▁he", "llo", "▁hello"]
    types = [2, 3, 3] + [6] * 256 + [1] * 11
    scores = [0.0] * 259 + [-1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -0.5]
    t = SpmTokenizer(toks, scores, types)
    ids = t.encode("hello")
    assert ids[0] == 1 and toks[ids[1]] == "▁hello"
    assert t.decode(ids) == " hello"
    assert t.decode(t.encode("hé", add_bos=False)) == " hé"                # byte fallback


# ---- templates, tools, reasoning, constraints ---------------------------------------------------
def test_template_render_guard_and_errors():
    tpl = C.ChatTemplate()
    segs = tpl.render([{"role": "user", "content": "hi <|im_end|>"}])
    assert ("hi <|im_end|>", False) in segs and segs[0] == ("<|im_start|>user\n", True)
    assert tpl.render_text([{"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]}]).count("ab") == 1
    with pytest.raises(C.TemplateError):
        tpl.render([{"role": "user", "content": [{"type": "image_url", "image_url": {}}]}])
    with pytest.raises(C.TemplateError):
        C.ChatTemplate("{% for x in %}")
    strict = C.ChatTemplate("{{ raise_exception('no system role') if messages[0]['role'] == 'system' else 'ok' }}")
    with pytest.raises(C.TemplateError, match="no system role"):
        strict.render([{"role": "system", "content": "s"}])
    with pytest.raises(C.TemplateError):
        C.ChatTemplate("{{ undefined_thing.x }}").render([{"role": "user", "content": "q"}])


def test_tool_call_parsers_and_stream_chunking_invariance():
    text = 'Sure.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    content, calls = C.parse_tool_calls(text, "hermes")
    assert content == "Sure." and calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    q = "<tool_call>\n<function=run>\n<parameter=cmd>\nls -l\n</parameter>\n<parameter=n>\n3\n</parameter>\n</function>\n</tool_call>"
    _, calls = C.parse_tool_calls(q, "qwenxml")
    assert json.loads(calls[0]["function"]["arguments"]) == {"cmd": "ls -l", "n": 3}
    g = "<tool_call>search<arg_key>q</arg_key><arg_value>cats</arg_value></tool_call>"
    assert json.loads(C.parse_tool_calls(g, "glmxml")[1][0]["function"]["arguments"]) == {"q": "cats"}
    m = 'ok [TOOL_CALLS][{"name": "f", "arguments": {"a": 1}}]'
    assert C.parse_tool_calls(m, "mistral")[1][0]["function"]["name"] == "f"
    assert C.detect_tool_format("... <function= ...") == "qwenxml" and C.detect_tool_format("plain") == "hermes"
    # the streamed scanner gives the same calls and text however the text is chunked
    for step in (1, 3, 7, len(text)):
        s = C.ToolCallStream("hermes")
        out, got = "", []
        for i in range(0, len(text), step):
            t, c = s.push(text[i:i + step])
            out += t
            got += c
        out += s.flush()
        assert out == "Sure." and len(got) == 1 and got[0]["function"]["name"] == "get_weather"


def test_dsml_tool_calls_both_spellings_and_streaming():
    D = C.DSML
    plain = (f'On it.\n\n<{D}tool_calls>\n<{D}invoke name="get_weather">\n'
             f'<{D}parameter name="city" string="true">Paris, "FR"</{D}parameter>\n'
             f'<{D}parameter name="days" string="false">3</{D}parameter>\n'
             f'<{D}parameter name="opts" string="false">{{"units": "c"}}</{D}parameter>\n'
             f'<{D}parameter name="odd" string="false">not json</{D}parameter>\n'
             f'</{D}invoke>\n<{D}invoke name="ping">\n</{D}invoke>\n</{D}tool_calls>')
    content, calls = C.parse_tool_calls(plain, "dsml")
    assert content == "On it." and [c["function"]["name"] for c in calls] == ["get_weather", "ping"]
    args = json.loads(calls[0]["function"]["arguments"])
    assert args == {"city": 'Paris, "FR"', "days": 3, "opts": {"units": "c"}, "odd": "not json"}
    assert list(args) == ["city", "days", "opts", "odd"]                       # parameter order is kept
    assert json.loads(calls[1]["function"]["arguments"]) == {}
    spaced = (f'<{D} calls>\n<{D} invoke name="f">\n<{D} parameter name="x" string="false">1</{D} parameter>\n'
              f'</{D} invoke>\n</{D} calls>')
    assert json.loads(C.parse_tool_calls(spaced, "dsml_spaced")[1][0]["function"]["arguments"]) == {"x": 1}
    assert C.parse_tool_calls(spaced, "dsml")[1] == []                          # a scan reads the one spelling it is given
    assert C.detect_tool_format(f"... <{D} calls> ...") == "dsml_spaced" and C.detect_tool_format(f"<{D}tool_calls>") == "dsml"
    # markup that does not parse, and a block still open at the end, stay content
    broken = f'<{D}tool_calls>\n<{D}invoke name="f">\n<{D}parameter name="x">1</{D}parameter>\n</{D}invoke>\n</{D}tool_calls>'
    assert C.parse_tool_calls(broken, "dsml") == (broken, [])
    open_end = f'hello <{D}tool_calls>\n<{D}invoke name="f">'
    assert C.parse_tool_calls(open_end, "dsml") == (open_end, [])
    for step in (1, 2, 5, 11, len(plain)):                                      # chunking never changes the result
        s = C.ToolCallStream("dsml")
        out, got = "", []
        for i in range(0, len(plain), step):
            t, c = s.push(plain[i:i + step])
            out += t
            got += c
        out += s.flush()
        assert out.strip() == "On it." and [c["function"]["arguments"] for c in got] == [c["function"]["arguments"] for c in calls]


def test_muse_recipient_protocol_and_atem_calls():
    text = (' to=self<|message|>think first<|eom|>\n<|start|>assistant to=commentary<|message|>working on it<|eom|>\n'
            '<|start|>assistant to=get_weather<|message|><atem:function_calls>\n<atem:invoke name="get_weather">\n'
            '<atem:parameter name="city">Paris</atem:parameter>\n<atem:parameter name="days">3</atem:parameter>\n'
            '</atem:invoke>\n</atem:function_calls><|eom|>\n<|start|>assistant to=user<|message|>done<|eot|>')
    r = C.parse_muse(text)
    assert r["reasoning_content"] == "think first" and r["content"] == "working on it\ndone"
    assert r["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(r["tool_calls"][0]["function"]["arguments"]) == {"city": "Paris", "days": 3}
    assert C.parse_tool_calls(text, "muse")[1][0]["function"]["name"] == "get_weather"
    broken = ' to=lookup<|message|><atem:function_calls><atem:invoke name="x">oops</atem:invoke></atem:function_calls><|eot|>'
    rb = C.parse_muse(broken)
    assert rb["tool_calls"] == [] and "oops" in rb["content"]                    # markup that does not parse stays content
    assert C.parse_muse("plain text")["content"] == "plain text"
    assert C.parse_muse(" to=user<|message|>cut off mid")["content"] == "cut off mid"
    assert C.detect_tool_format("... <atem:invoke ...") == "muse"


def test_preflight_verdicts():
    from bloomery_b200.serve import preflight as P
    assert P.cpu_gate(["sse4_2", "avx2", "fma", "f16c", "bmi2"]) is None
    msg = P.cpu_gate(["sse4_2", "avx", "fma"])
    assert "avx2" in msg and "f16c" in msg and "fma" not in msg.split(":")[0]
    assert P.cpu_gate([], machine="aarch64") is None
    assert P.parse_driver("NVRM version: NVIDIA UNIX Open Kernel Module for x86_64  580.159.01  Release") == (580, 159)
    assert P.driver_gate("580.159") is None and P.driver_gate(None) is None and P.driver_gate("garbage") is None
    assert "535.183" in P.driver_gate("535.183.01") and "R570" in P.driver_gate("535.183.01")
    assert P.no_card(1, []) is None
    assert "no CUDA device on this machine" in P.no_card(0, []) and "-dev none" in P.no_card(0, [])
    assert "lists 2" in P.no_card(0, ["NVIDIA B200", "NVIDIA B200"])
    assert P.run(0, "none") is None                                                # the CPU engine needs no card


def test_per_key_limits():
    from bloomery_b200.serve.admit import Admission, LimitError, Limits, Refused, parse_key_line
    key, lim = parse_key_line("sk-one inflight=2 rate=30/m burst=3")
    assert key == "sk-one" and lim.inflight == 2 and lim.rate == (30, True) and lim.burst == 3 and lim.interval == 2.0
    assert parse_key_line("sk-two")[1].inflight is None
    for bad in ("k rate=5", "k rate=5/h", "k inflight=0", "k burst=2", "k colour=red", "k inflight"):
        with pytest.raises(LimitError) as e:
            parse_key_line(bad)
        assert "k " not in str(e.value)                                           # the key is never in the message
    now = [100.0]
    adm = Admission({"a": Limits(inflight=2), "b": Limits(rate=(2, False), burst=2), "c": Limits()}, clock=lambda: now[0])
    r1, r2 = adm.admit("a"), adm.admit("a")
    with pytest.raises(Refused) as e:
        adm.admit("a")
    assert e.value.retry_after >= 1
    r1(); r1()                                                                     # releasing twice frees one place
    r3 = adm.admit("a")
    with pytest.raises(Refused):
        adm.admit("a")
    r2(); r3()
    adm.admit("b")(); adm.admit("b")()                                            # the burst
    with pytest.raises(Refused):
        adm.admit("b")                                                             # bucket empty: a request every 0.5 s
    now[0] += 0.5
    adm.admit("b")()
    with pytest.raises(Refused):
        adm.admit("b")
    for _ in range(50):
        adm.admit("c")                                                             # no limits, and keys count apart
        adm.admit("unknown")
    # scopes: which routes a key reaches
    from bloomery_b200.serve.admit import route_scope
    inf, rd, adm_ = parse_key_line("k scope=inference")[1], parse_key_line("k scope=read")[1], parse_key_line("k")[1]
    both = parse_key_line("k scope=inference,read inflight=1")[1]
    assert adm_.scopes == {"admin"} and both.scopes == {"inference", "read"} and both.inflight == 1
    table = [("POST", "/v1/chat/completions", "inference"), ("POST", "/tokenize", "inference"), ("GET", "/v1/responses/resp_1", "inference"),
             ("POST", "/v1/messages/count_tokens", "inference"), ("POST", "/v1/embeddings", "inference"), ("GET", "/props", "read"),
             ("GET", "/slots", "read"), ("GET", "/metrics", "read"), ("GET", "/v1/models", "lookup"), ("GET", "/v1/models/m", "lookup"),
             ("POST", "/api/show", "lookup"), ("POST", "/slots/0", "admin"), ("POST", "/residency/reset", "admin"),
             ("POST", "/shutdown", "admin"), ("GET", "/health", "public"), ("POST", "/props", "admin")]
    for method, path, want in table:
        assert route_scope(method, path) == want, (method, path)
        assert adm_.reaches(method, path)
        assert inf.reaches(method, path) == (want in ("inference", "lookup", "public"))
        assert rd.reaches(method, path) == (want in ("read", "lookup", "public"))
        assert both.reaches(method, path) == (want != "admin")
    for bad in ("k scope=", "k scope=root", "k scope=read scope=admin", "k inflight=1 inflight=2"):
        with pytest.raises(LimitError):
            parse_key_line(bad)


def test_reasoning_split():
    assert C.split_reasoning("<think>plan</think>\nanswer") == ("plan", "answer")
    assert C.split_reasoning("plan</think>answer", started=True) == ("plan", "answer")
    assert C.split_reasoning("no thinking") == ("", "no thinking")
    assert C.split_reasoning("<think>unfinished") == ("unfinished", "")


def test_json_constraint_prefixes_and_schema():
    c = C.JsonConstraint()
    assert c.allowed("", '{"a"') and c.allowed('{"a"', ": [1, 2") and not c.allowed('{"a"', " 1") and not c.allowed("", "}")
    assert c.done('{"a": [1, 2.5e3, true, null]}') and not c.done('{"a": [1,') and not c.allowed('{"a": 1}', "x")
    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "t": {"enum": ["x", "y"]}}, "required": ["n"],
              "additionalProperties": False}
    s = C.JsonConstraint(schema)
    assert s.done('{"n": 3, "t": "x"}') and not s.done('{"t": "x"}') and not s.done('{"n": 3, "z": 1}') and not s.done('{"n": "3"}')
    assert not s.allowed("", "[") and s.allowed("", "{")
    assert C.validate([1, 2], {"type": "array", "items": {"type": "number"}, "minItems": 2}) and not C.validate([1], {"type": "array", "minItems": 2})


# ---- prompt cache and board -------------------------------------------------------------------------
def test_constraint_program_walk_and_jump_arm():
    from bloomery_b200.serve.constrain import ProgramConstraint, Unsupported, Walk, compile_schema, constraint_for
    schema = {"type": "object", "properties": {
        "name": {"type": "string", "maxLength": 8}, "age": {"type": "integer"}, "ok": {"type": "boolean"},
        "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "minItems": 1, "maxItems": 2},
        "pos": {"type": "object", "properties": {"x": {"type": "number"}}, "required": ["x"]}, "kind": {"const": "v1"}},
        "required": ["name", "age", "ok", "tags", "pos", "kind"]}
    pc = ProgramConstraint(schema)
    assert pc.forced_text("") == '{"name": '                                      # keys and punctuation are never sampled
    good = '{"name": "Al\\"x", "age": -12, "ok": true, "tags": ["a", "b"], "pos": {"x": 1.5e3}, "kind": "v1"}'
    w = Walk(pc.program)
    for ch in good:
        assert w.accepts(ch), ch
        w.take(ch)
    assert w.spent and not w.accepts(" ") and json.loads(good)["tags"] == ["a", "b"]
    # pieces of several characters, as tokens are
    assert pc.allowed('{"name": ', '"Bo') and pc.allowed('{"name": "Bo', '", "age": ') and not pc.allowed('{"name": "Bo', '", "ok"')
    assert not pc.allowed('{"name": "12345678', "9") and pc.allowed('{"name": "12345678', '"')     # maxLength
    assert pc.forced_text('{"name": "Bo"') == ', "age": ' and pc.forced_text('{"name": "Bo", "age": ') == ""
    assert pc.allowed('{"name": "Bo", "age": ', "4") and not pc.allowed('{"name": "Bo", "age": ', "4.") and not pc.allowed('{"name": "Bo", "age": ', "04")
    assert pc.allowed('{"name": "Bo", "age": 4', ', "ok": ')                     # a whole number hands the next character on
    t = '{"name": "Bo", "age": 4, "ok": '
    assert pc.forced_text(t) == "" and pc.allowed(t, "tr") and pc.allowed(t, "false") and not pc.allowed(t, "maybe")
    t += 'false, "tags": ['
    assert pc.forced_text(t) == '"' and not pc.allowed(t, "]")                   # minItems 1: the array may not close yet
    t += '"a"'
    assert pc.allowed(t, "]") and pc.allowed(t, ', "b"') and not pc.allowed(t, ', "c"')
    t += ', "b"'
    assert pc.forced_text(t) == '], "pos": {"x": ' and not pc.allowed(t, ', "a"')   # maxItems 2: only the close is left
    t += '], "pos": {"x": 2'
    assert not pc.done(t) and pc.allowed(t, '}, "kind": "v1"}')
    t += '}, "kind": "v1"}'
    assert pc.done(t) and pc.closed(t) and not pc.allowed(t, "x")
    assert ProgramConstraint({"type": "number"}).done("3.25") and not ProgramConstraint({"type": "number"}).done("3.")
    assert ProgramConstraint({"anyOf": [{"type": "null"}, {"type": "integer"}]}).allowed("", "nu")
    with pytest.raises(Unsupported):
        compile_schema({"type": "object"})                                        # no property list: not a program
    assert constraint_for({"type": "object"}) is None and constraint_for(None) is None
    # required members in order, then each optional one in order, each of which may be left out
    opt = ProgramConstraint({"type": "object", "required": ["id"], "properties": {
        "note": {"type": "string"}, "id": {"type": "integer"}, "flag": {"type": "boolean"}}})
    assert opt.forced_text("") == '{"id": '
    for doc in ('{"id": 7}', '{"id": 7, "note": "x"}', '{"id": 7, "flag": true}', '{"id": 7, "note": "x", "flag": false}'):
        assert opt.allowed("", doc) and opt.done(doc), doc
    assert not opt.allowed("", '{"id": 7, "flag": true, "note": "x"}') and not opt.allowed("", '{"note": "x"')       # order; id first
    free = ProgramConstraint({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "integer"}}})
    for doc in ("{}", '{"a": 1}', '{"b": 2}', '{"a": 1, "b": 2}'):
        assert free.allowed("", doc) and free.done(doc), doc
    assert not free.allowed("", '{, "b"') and not free.allowed("", '{"b": 2, "a"')
    # a $ref into the schema itself; recursion and pointers outside it are not a program
    refd = ProgramConstraint({"type": "object", "required": ["p", "q"], "properties": {"p": {"$ref": "#/$defs/pt"}, "q": {"$ref": "#/$defs/pt"}},
                              "$defs": {"pt": {"type": "object", "required": ["x"], "properties": {"x": {"type": "number"}}}}})
    assert refd.allowed("", '{"p": {"x": 1}, "q": {"x": 2.5}}')
    for bad in ({"$ref": "other.json#/a"}, {"$ref": "#/$defs/missing", "$defs": {}},
                {"$ref": "#/$defs/n", "$defs": {"n": {"type": "array", "items": {"$ref": "#/$defs/n"}}}},
                {"type": "string", "pattern": "^a"}, {"type": "string", "minLength": 2}, {"type": "integer", "minimum": 0},
                {"allOf": [{"type": "integer"}]}, {"type": "object", "properties": {}, "minProperties": 1},
                {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["b"]},
                {"type": "object", "properties": {}, "additionalProperties": True}):
        with pytest.raises(Unsupported):
            compile_schema(bad)
        assert constraint_for(bad) is None
    deep = {"type": "integer"}
    for _ in range(140):
        deep = {"type": "array", "items": deep}
    with pytest.raises(Unsupported, match="nested levels"):
        compile_schema(deep)


def test_prompt_cache_rules():
    pc = PromptCache(100)
    s = lambda ids, n: Saved(tuple(ids), None, n)
    assert pc.put(s([1, 2, 3], 40)) and pc.put(s([9, 9], 40))
    got, n = pc.lookup([1, 2, 3, 4, 5])
    assert got.ids == (1, 2, 3) and n == 3
    assert pc.put(s([1, 2, 3, 4], 40))                      # covers [1,2,3] wholly -> that one is evicted first
    assert (1, 2, 3) not in pc._items and len(pc) == 2
    assert pc.put(s([7], 40))                               # over budget: least recently used goes
    assert pc.used <= 100 and (9, 9) not in pc._items
    assert pc.lookup([5, 5])[0] is None and not pc.put(s([1], 1000))
    pc2 = PromptCache(50)
    pc2.put(s([1], 40), pending=True)
    pc2.put(s([2], 40))
    assert (1,) in pc2._items                               # a pending copy is pinned
    pc2.settle([1])
    assert pc2.used <= 50


def test_board_slot_choice_and_queue():
    class R:
        def __init__(self, ids, i):
            self.prompt_ids, self.id = ids, i
    b = Board(3, queue_depth=2)
    b.slots[0].ids = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    b.slots[1].ids = [1, 2, 3]
    slot, shared = b.pick_slot([1, 2, 3, 4, 5, 99])
    assert slot.id == 0 and shared == 5                     # longest common prefix wins
    slot, shared = b.pick_slot([50] * 40)
    assert slot.id == 2 and shared == 0                     # nothing shared: the empty slot is preferred
    slot, shared = b.pick_slot([1] + [77] * 30)
    assert shared == 0                                      # below the 0.1 similarity floor
    b.submit(R([1], 1)); b.submit(R([2], 2))
    with pytest.raises(QueueFull):
        b.submit(R([3], 3))
    req, slot, _ = b.next_request()
    assert req.id == 1 and slot.busy                        # oldest first
    b.release(slot)
    assert not slot.busy


def test_ngram_draft_and_width_chooser():
    from bloomery_b200.runtime.speculative import NgramDraft, WidthChooser, accept_prefix
    d = NgramDraft(max_n=3)
    assert d.propose([1, 2, 3, 4, 9, 1, 2, 3], 3) == [4, 9, 1]
    assert d.propose([5, 6, 7], 4) == []
    assert accept_prefix([4, 9, 1], [4, 9, 7, 3]) == 2 and accept_prefix([4], [5, 0]) == 0
    w = WidthChooser(max_width=4)
    for _ in range(30):
        w.observe_pass(1, 1.0); w.observe_pass(5, 1.1)
        w.observe_accept(4, 4)
    assert w.choose(4) == 4                              # high acceptance, cheap rows: draft wide
    w2 = WidthChooser(max_width=4)
    for _ in range(30):
        w2.observe_pass(1, 1.0); w2.observe_pass(2, 1.9); w2.observe_pass(5, 4.5)
        w2.observe_accept(4, 0)
    assert w2.choose(4) == 0                             # nothing is ever accepted: plain steps


def test_fit_on_keeps_what_fits_on_the_card():
    """``-fit on`` on a card too small for the model: the plan keeps a multiple of four expert slots per layer on the
    card and the rest on the host; without it the same ask is refused; a trunk that does not fit is refused either way."""
    from bloomery_b200.models.spec import qwen3_30b_a3b
    from bloomery_b200.serve.cli import plan_for
    from bloomery_b200.utils.exit_codes import Refusal
    spec = qwen3_30b_a3b()
    opts = flags.parse(["-m", "x", "-fit", "on", "-np", "1", "-c", "8192"], {})
    opts["_expert_bytes"] = 16_000_000_000
    plan = plan_for(opts, spec, 17_500_000_000, 1, [12 << 30])
    word = plan["placement"].host_experts
    assert word.startswith("fit:") and 0 < int(word.split(":")[1]) < spec.n_expert and int(word.split(":")[1]) % 4 == 0
    assert plan["slot_ctx"] == 8192
    with pytest.raises(Refusal):
        plan_for(flags.parse(["-m", "x", "-np", "1", "-c", "8192"], {}), spec, 17_500_000_000, 1, [12 << 30])
    opts2 = flags.parse(["-m", "x", "-fit", "on", "-np", "1"], {})
    opts2["_expert_bytes"] = 16_000_000_000
    with pytest.raises(Refusal):
        plan_for(opts2, spec, 17_500_000_000, 1, [3 << 30])
    # -fitt: what stays free per device; a larger target leaves fewer resident experts, a list names every device
    def resident(*extra):
        o = flags.parse(["-m", "x", "-fit", "on", "-np", "1", "-c", "8192", *extra], {})
        o["_expert_bytes"] = 16_000_000_000
        return int(plan_for(o, spec, 17_500_000_000, 1, [12 << 30])["placement"].host_experts.split(":")[1])
    assert resident("-fitt", "3072") < resident("-fitt", "512")
    two = flags.parse(["-m", "x", "-dev", "CUDA0,CUDA1", "--place", "tp", "-np", "1", "-c", "8192", "-fitt", "1024,78000"], {})
    with pytest.raises(Refusal):                               # the second device keeps 78,000 MiB of its 81,920 free: nothing fits there
        plan_for(two, spec, 17_500_000_000, 2, [80 << 30, 80 << 30])
    two = flags.parse(["-m", "x", "-dev", "CUDA0,CUDA1", "--place", "tp", "-np", "1", "-c", "8192", "-fitt", "1024,2048"], {})
    assert plan_for(two, spec, 17_500_000_000, 2, [80 << 30, 80 << 30])["slot_ctx"] == 8192
    bad = flags.parse(["-m", "x", "-dev", "CUDA0,CUDA1", "--place", "tp", "-fitt", "1,2,3"], {})
    with pytest.raises(Refusal):
        plan_for(bad, spec, 17_500_000_000, 2, [80 << 30, 80 << 30])


def test_reference_sets_carry_the_model_identity(tmp_path):
    from bloomery_b200.models import weights as W
    from bloomery_b200.models.spec import tiny_qwen3moe
    from bloomery_b200.utils import refset as R
    spec = tiny_qwen3moe()
    spec.vocab, spec.n_layer = 256, 1
    a, b = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    W.write_gguf(spec, W.synth_tensors(spec, "cpu", seed=1), a)
    W.write_gguf(spec, W.synth_tensors(spec, "cpu", seed=2), b)
    out = str(tmp_path / "set.json")
    assert R.main(["make", a, out, "--cases", "2", "--prompt-len", "6", "--new", "4"]) == 0
    doc = R.read(out)
    assert len(doc["cases"]) == 2 and len(doc["cases"][0]["greedy"]) == 4 and doc["arch"] == "qwen3moe"
    assert R.main(["check", a, out, "--min-agree", "1.0"]) == 0
    assert R.main(["check", b, out]) == 1                      # another model file: refused before any token is compared
    agree, total = R.check(doc, a, lambda p, n: [doc["cases"][0]["greedy"][0]] + [0] * (n - 1), min_agree=0.0)
    assert total == 8 and agree <= 5
    open(out, "w").write("{}")
    with pytest.raises(R.RefsetError):
        R.read(out)
    # the logits kind: KL divergence over the oracle's top ids, and the flip rule for a different arg-max
    lset = str(tmp_path / "lset.json")
    assert R.main(["make", a, lset, "--cases", "2", "--prompt-len", "6", "--logits"]) == 0
    assert R.main(["check", a, lset]) == 0                     # the same model: zero divergence, no flips
    assert R.main(["check", b, lset]) == 1
    ldoc = json.load(open(lset))
    _, fn = R._logits_fn(a, "cpu")
    same = R.check_logits(ldoc, a, fn)
    assert same["mean_kld"] < 1e-9 and same["flips"] == same["misses"] == 0 and same["positions"] == 12
    import torch

    def nudged(ids):                                           # the runner-up of position 0 takes the lead by a hair
        lg = fn(ids).clone()
        top = lg[0].topk(2)
        lg[0, top.indices[1]] = top.values[0] + 1e-3
        return lg
    lead = ldoc["cases"][0]["top_logp"][0][0] - ldoc["cases"][0]["top_logp"][0][1]
    out_n = R.check_logits(ldoc, a, nudged, max_mean_kld=1.0, flip_margin=lead + 1.0)
    assert out_n["flips"] == 2 and out_n["misses"] == 0        # once per case: the same nudge on both prompts' first row
    with pytest.raises(R.RefsetError, match="pick another id"):
        R.check_logits(ldoc, a, nudged, max_mean_kld=1.0, flip_margin=0.0)
    with pytest.raises(R.RefsetError, match="KL divergence"):
        R.check_logits(ldoc, a, lambda ids: fn(ids) * 0.0, max_mean_kld=1e-7, flip_margin=100.0)


def test_need_record_and_broker_hook(tmp_path, monkeypatch):
    """The placed load states what it asks of the machine, and a hook may let it go on (0), queue it (75) or stop it."""
    import stat
    from bloomery_b200.models.spec import qwen3_30b_a3b
    from bloomery_b200.serve import cli
    from bloomery_b200.utils import levers as LV
    spec = qwen3_30b_a3b()
    opts = flags.parse(["-m", "x", "-fit", "on", "-np", "1", "-c", "8192", "-cram", "512"], {})
    opts["_expert_bytes"] = 16_000_000_000
    plan = cli.plan_for(opts, spec, 17_500_000_000, 1, [12 << 30])
    need = cli.need_record(opts, spec, 17_500_000_000, plan)
    resident = int(plan["placement"].host_experts.split(":")[1])
    assert need["pinned"] == (512 << 20) + 16_000_000_000 - 16_000_000_000 // 128 * resident
    assert need["cache_ram"] == 512 << 20 and need["cards"][0].startswith("CUDA0:") and need["threads"] >= 1 and need["allowed"]
    records.write("need", _out=io.StringIO(), **need)                 # every field is one the record kind knows

    def hook(body):
        p = tmp_path / "hook.sh"
        p.write_text("#!/bin/sh\n" + body + "\n")
        p.chmod(p.stat().st_mode | stat.S_IXUSR)
        return str(p)
    log = tmp_path / "need.log"
    for body, want in ((f"cat >> {log}", None), ("echo busy until noon; exit 75", Code.RETRY), ("echo no; exit 3", Code.REFUSED)):
        monkeypatch.setitem(LV._values, "BLOOMERY_NEED_HOOK", hook(body))
        if want is None:
            cli.ask_need_hook(need)
            assert log.read_text().startswith("need weights_bytes=17500000000 ")
        else:
            with pytest.raises(Refusal) as e:
                cli.ask_need_hook(need)
            assert e.value.code == want and ("busy until noon" in str(e.value) or "exited 3: no" in str(e.value))
    monkeypatch.setitem(LV._values, "BLOOMERY_NEED_HOOK", "relative/hook")
    with pytest.raises(Refusal):
        cli.ask_need_hook(need)
    monkeypatch.setitem(LV._values, "BLOOMERY_NEED_HOOK", "")
    cli.ask_need_hook(need)


def test_slot_count_and_context_rules():
    """One slot unless asked; ``auto`` counts from memory up to 8; a set context is never cut; the flags that contradict
    each other are refused by name."""
    from bloomery_b200.models.spec import qwen3_30b_a3b
    from bloomery_b200.serve.cli import plan_for
    spec = qwen3_30b_a3b()

    def plan(argv, free=170 << 30):
        return plan_for(flags.parse(["-m", "x", *argv], {}), spec, 17_500_000_000, 1, [free])
    p = plan([])
    assert (p["n_slots"], p["slot_ctx"], p["ctx_rule"], p["slots_from"]) == (1, spec.ctx_train // 64 * 64, "target", "flag")
    p = plan(["-np", "auto"])
    assert (p["n_slots"], p["ctx_rule"], p["slots_from"]) == (8, "target", "auto")
    p = plan(["-np", "auto", "--slot-ctx", "32768"])
    assert (p["n_slots"], p["slot_ctx"], p["ctx_rule"]) == (8, 32768, "set")
    tight = plan(["-np", "auto"], free=22 << 30)                     # one slot already has to fit under the model's limit
    assert tight["n_slots"] == 1 and tight["ctx_rule"] == "fitted" and 4096 <= tight["slot_ctx"] < spec.ctx_train
    some = plan(["-np", "auto", "--slot-ctx", "16384"], free=27 << 30)
    assert 1 <= some["n_slots"] < 8 and some["slot_ctx"] == 16384
    assert plan(["-np", "2", "-c", "16384"])["slot_ctx"] == 8192      # a set total is shared
    assert plan(["-np", "4", "--slot-ctx", "8192"])["ctx_total"] == 32768
    for bad in (["-np", "auto", "-c", "8192"], ["--slot-ctx", "4096", "-c", "8192"], ["-np", "0"], ["-np", "many"]):
        with pytest.raises(Refusal) as e:
            plan(bad)
        assert e.value.code == Code.USAGE
    with pytest.raises(Refusal) as e:
        plan(["-np", "4", "--slot-ctx", "40960"], free=26 << 30)
    assert e.value.code == Code.NO_FIT and "largest slot context" in str(e.value)


def test_reasoning_rules():
    from bloomery_b200.serve import reasoning as RS
    assert RS.effort_kwargs(None, {"a": 1}) == {"a": 1}
    assert RS.effort_kwargs("none", None) == {"enable_thinking": False, "reasoning_effort": "none"}
    assert RS.effort_kwargs("high", {"enable_thinking": True})["enable_thinking"] is True
    for effort, kw in (("loud", None), (3, None), ("none", {"enable_thinking": True}), ("low", {"enable_thinking": False})):
        with pytest.raises(RS.ReasoningError):
            RS.effort_kwargs(effort, kw)
    assert RS.budget_from({}) == -1 and RS.budget_from({"reasoning_budget": 0}) == 0
    for bad in ({"reasoning_budget": -2}, {"reasoning_budget": 1.5}, {"reasoning_budget": True}):
        with pytest.raises(RS.ReasoningError):
            RS.budget_from(bad)
    with pytest.raises(RS.ReasoningError):
        RS.budget_from({"reasoning_budget": 10}, forced_tool=True)
    assert RS.loop_flag({"reasoning_loop": True}) and not RS.loop_flag({"reasoning_loop": None})
    with pytest.raises(RS.ReasoningError):
        RS.loop_flag({"reasoning_loop": "yes"})
    # the loop check: a cycle of up to 1,024 ids over at least 256 ids and one whole cycle
    rng = np.random.default_rng(0)
    free = rng.integers(0, 1000, 3000).tolist()
    assert RS.find_loop(free) == 0
    cyc = rng.integers(0, 1000, 7).tolist()
    assert RS.find_loop(free[:100] + cyc * 36) == 0                    # 252 repeated ids: under the 256 + one cycle
    assert RS.find_loop(free[:100] + cyc * 38) == 7
    long_cycle = rng.integers(0, 1000, 600).tolist()
    assert RS.find_loop(free[:50] + long_cycle * 2) == 600 and RS.find_loop(free[:50] + long_cycle + long_cycle[:500]) == 0
    assert RS.find_loop([5] * 300) == 1
    # the span: budget and forced close
    sp = RS.ThinkSpan(budget=3)
    text = ""
    closes = []
    for i, piece in enumerate(["<think>", "a", "b", "c", "d"]):
        text += piece
        sp.note(text, i + 1)
        closes.append(sp.force_close(text))
    assert closes == [False, False, True, False, False]                # once, when the span has used its three ids
    sp0 = RS.ThinkSpan(started=True, budget=0)
    assert sp0.force_close("") and not sp0.force_close("")
    done = RS.ThinkSpan(started=True, budget=5)
    done.note("x</think>", 1)
    assert not done.inside("x</think> answer") and not done.force_close("x</think> answer")


def test_llama_server_variables():
    """A variable is its flag with that value; the command line wins and a line says so; keys add; a switch takes eight
    words; a variable nobody reads gets a line; a refusal names the variable."""
    from bloomery_b200.utils import flags, levers
    from bloomery_b200.utils.exit_codes import Refusal
    o = flags.parse(["-c", "4096"], {"LLAMA_ARG_CTX_SIZE": "8192", "LLAMA_ARG_UBATCH": "512", "LLAMA_ARG_FLASH_ATTN": "1",
                                     "LLAMA_ARG_FIT": "on", "LLAMA_ARG_CPU_MOE": "enabled"})
    assert o["ctx"] == 4096 and o["ubatch"] == 512 and o["fit"] == "on" and o["cpu_moe"] is True
    notes = "\n".join(o["_config_notes"])
    assert "LLAMA_ARG_CTX_SIZE: replaced by the command line" in notes
    assert "LLAMA_ARG_FLASH_ATTN is set: not a variable this server reads" in notes
    assert o["_from_env"]["ubatch"] == "LLAMA_ARG_UBATCH"
    assert flags.parse([], {"LLAMA_ARG_CPU_MOE": "disabled"})["cpu_moe"] is False
    with pytest.raises(Refusal, match="LLAMA_ARG_CPU_MOE"):
        flags.parse([], {"LLAMA_ARG_CPU_MOE": "maybe"})
    with pytest.raises(Refusal, match="LLAMA_ARG_CTX_SIZE"):
        flags.parse([], {"LLAMA_ARG_CTX_SIZE": "lots"})
    # keys add, an empty one ends the start, and no note prints a key
    o = flags.parse(["--api-key", "k1"], {"LLAMA_API_KEY": "k2,k3"})
    assert o["api_key"] == "k1,k2,k3" and not any("k2" in n for n in o["_config_notes"])
    assert flags.parse([], {"LLAMA_API_KEY": "k9"})["api_key"] == "k9"
    o = flags.parse(["--api-key", '"a,b",c'], {"LLAMA_API_KEY": "d"})
    assert flags.split_keys(o["api_key"]) == ["a,b", "c", "d"]
    with pytest.raises(Refusal, match="LLAMA_API_KEY names no key"):
        flags.parse([], {"LLAMA_API_KEY": ""})
    with pytest.raises(Refusal, match="--api-key names no key"):
        flags.parse(["--api-key", ""], {})
    # the model: both variables set is refused; a model on the command line replaces both
    with pytest.raises(Refusal, match="LLAMA_ARG_MODEL beside LLAMA_ARG_HF_REPO"):
        flags.parse([], {"LLAMA_ARG_MODEL": "a.gguf", "LLAMA_ARG_HF_REPO": "x/y"})
    o = flags.parse(["-m", "b.gguf"], {"LLAMA_ARG_MODEL": "a.gguf", "LLAMA_ARG_HF_REPO": "x/y"})
    assert o["model"] == "b.gguf" and o["hf"] is None
    # --place replaces the variables that name cards
    o = flags.parse(["--place", "tp"], {"LLAMA_ARG_DEVICE": "CUDA3", "LLAMA_ARG_SPLIT_MODE": "row", "LLAMA_ARG_MAIN_GPU": "2"})
    assert o["dev"] is None and o["split_mode"] == "layer" and o["main_gpu"] == 0
    assert "LLAMA_ARG_SPLIT_MODE: replaced by --place" in "\n".join(o["_config_notes"])
    # a variable whose flag would be refused ends the start under the variable's name
    o = flags.parse([], {"LLAMA_ARG_SPLIT_MODE": "row"})
    with pytest.raises(Refusal, match="LLAMA_ARG_SPLIT_MODE row is not served"):
        flags.placement(o, 2)
    with pytest.raises(Refusal, match="-sm row is not served"):
        flags.placement(flags.parse(["-sm", "row"], {}), 2)
    with pytest.raises(Refusal, match="LLAMA_ARG_DEVICE names CUDA5"):
        flags.placement(flags.parse([], {"LLAMA_ARG_DEVICE": "CUDA5"}), 2)
    # llama-server's "no limit" prompt cache is refused wherever it is named; unset keeps the default rule
    for argv, env_ in ((["--cache-ram", "-1"], {}), ([], {"LLAMA_ARG_CACHE_RAM": "-1"})):
        with pytest.raises(Refusal, match="always has a budget"):
            flags.parse(argv, env_)
    assert flags.parse([], {})["cache_ram"] == -1 and flags.parse(["-cram", "0"], {})["cache_ram"] == 0
    # the driver's launch-queue variable: unset becomes 2x, NVIDIA's other values stay, anything else stops the start
    env = {}
    levers.at_main(env)
    assert env["CUDA_SCALE_LAUNCH_QUEUES"] == "2x"
    env = {"CUDA_SCALE_LAUNCH_QUEUES": "4x"}
    levers.at_main(env)
    assert env["CUDA_SCALE_LAUNCH_QUEUES"] == "4x"
    with pytest.raises(Refusal, match="CUDA_SCALE_LAUNCH_QUEUES"):
        levers.at_main({"CUDA_SCALE_LAUNCH_QUEUES": "8x"})
    levers.at_main({})


def test_forced_call_programs_both_framings_and_open_think():
    from bloomery_b200.serve import chat as C, constrain as K
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
                 "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}},
             {"type": "function", "function": {"name": "now"}}]
    texts = {"hermes": '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo", "days": 3}}\n</tool_call>',
             "qwenxml": "<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n<parameter=days>\n3\n</parameter>\n"
                        "</function>\n</tool_call>"}
    texts["glmxml"] = ("<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Oslo</arg_value>\n<arg_key>days</arg_key>\n"
                       "<arg_value>3</arg_value>\n</tool_call>")
    D = C.DSML
    for framing, sp, blk in (("dsml", "", "tool_calls"), ("dsml_spaced", " ", "calls")):
        texts[framing] = (f'<{D}{sp}{blk}>\n<{D}{sp}invoke name="get_weather">\n<{D}{sp}parameter name="city" string="true">Oslo</{D}{sp}parameter>\n'
                          f'<{D}{sp}parameter name="days" string="false">3</{D}{sp}parameter>\n</{D}{sp}invoke>\n</{D}{sp}{blk}>')
    for framing, text in texts.items():
        c = K.ForcedCall(K.forced_call_program(tools, "required", framing))
        assert c.forced_text("").startswith(K.call_opener(framing))
        for i in range(1, len(text)):
            assert c.allowed(text[:i], text[i]), (framing, text[:i + 1])
        assert c.done(text) and c.closed(text) and not c.allowed(text, "x")
        parse = {"hermes": C.parse_hermes, "qwenxml": C.parse_qwen_xml, "glmxml": C.parse_glm_xml, "dsml": C.parse_dsml,
                 "dsml_spaced": C.parse_dsml}[framing]
        assert json.loads(parse(text)[1][0]["function"]["arguments"]) == {"city": "Oslo", "days": 3}
        # the optional member may be left out; a raw string takes no "<" and no line break
        short = text.replace(', "days": 3', "").replace("<parameter=days>\n3\n</parameter>\n", "").replace(
            "<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n", "")
        for sp in ("", " "):
            short = short.replace(f'<{D}{sp}parameter name="days" string="false">3</{D}{sp}parameter>\n', "")
        assert K.ForcedCall(K.forced_call_program(tools, "get_weather", framing)).done(short)
        # a think span the template opened stays free until its close; the reply cannot end inside it
        t = K.ForcedCall(K.forced_call_program(tools, "get_weather", framing), think_open=True)
        assert t.allowed("so", " anything <tool_call> at all") and not t.done("so") and t.forced_text("so") == ""
        assert t.allowed("so", "</think>") and t.allowed("so", "</think>\n\n" + K.call_opener(framing)[:5]) and not t.allowed("so", "</think>hello")
        assert t.done("so</think>\n\n" + text) and t.done("so</think>" + text)
    # inside a JSON-framed call a free string takes no "<" and fixed text writes it as its escape, so the scan for tags
    # never meets one the model wrote
    lt = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {
        "a<b": {"type": "string"}, "k": {"enum": ["x<y", "z"]}, "l": {"type": "array", "items": {"type": "string"}}}, "required": ["a<b", "k", "l"]}}}]
    c = K.ForcedCall(K.forced_call_program(lt, "f", "hermes"))
    head = '<tool_call>\n{"name": "f", "arguments": {"a\\u003cb": "hi'
    assert c.forced_text("").endswith('{"a\\u003cb": ') and not c.allowed(head, "<") and c.allowed(head, "x")
    whole = head + '", "k": "x\\u003cy", "l": ["q"]}}\n</tool_call>'
    assert c.done(whole) and json.loads(C.parse_hermes(whole)[1][0]["function"]["arguments"]) == {"a<b": "hi", "k": "x<y", "l": ["q"]}
    assert not c.allowed(head + '", "k": "x\\u003cy", "l": ["q', "<")
    raw = K.ForcedCall(K.forced_call_program(tools, "get_weather", "qwenxml"))
    assert not raw.allowed("<tool_call>\n<function=get_weather>\n<parameter=city>\nOs", "<b")
    for bad_tools, choice, framing in ((tools, "absent", "hermes"), (tools, "required", "mistral"), ([], "required", "hermes"),
                                       ([{"type": "function", "function": {"name": "f", "parameters": {"$ref": "#/x"}}}], "f", "hermes")):
        with pytest.raises(K.Unsupported):
            K.forced_call_program(bad_tools, choice, framing)


def test_watched_calls_follow_the_schema_from_the_opener():
    from bloomery_b200.serve import constrain as K
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
                 "type": "object", "properties": {"unit": {"enum": ["c", "f"]}}, "required": ["unit"]}}},
             {"type": "function", "function": {"name": "now"}}]
    w = K.watched_calls(tools, "hermes")
    assert w.allowed("", "Let me <b>check</b> that. ") and w.done("Let me check") and w.forced_text("free") == ""
    pre = "I will call.\n<tool_call>"
    assert w.allowed("I will call.\n<tool_", "call>") and not w.done(pre)                  # no ending inside a call
    assert w.forced_text(pre) == '\n{"name": "'
    assert w.allowed(pre, '\n{"name": "now"') and not w.allowed(pre, '\n{"name": "later"') and not w.allowed(pre, '{"name"')
    one = pre + '\n{"name": "get_weather", "arguments": {"unit": "c"}}\n</tool_call>'
    assert w.done(one) and not w.closed(one) and w.allowed(one, "\n<tool_call>\n{") and w.allowed(one, " and that is all")
    assert not w.allowed(pre + '\n{"name": "get_weather", "arguments": {"unit": "', "k")
    two = one + "\n<tool_call>\n" + '{"name": "now", "arguments": {}}\n</tool_call>'
    assert w.done(two)
    # a framing the programs do not write, or a schema outside the subset, leaves the calls unwatched
    assert K.watched_calls(tools, "mistral") is None and K.watched_calls(tools, "glmxml") is not None
    assert K.watched_calls([{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {
        "a": {"type": "string", "pattern": "x+"}}}}}], "hermes") is None


def test_queue_depth_rule():
    from bloomery_b200.serve.cli import queue_depth_for
    from bloomery_b200.utils.exit_codes import Refusal
    assert queue_depth_for({}, 1) == 63 and queue_depth_for({"queue_depth": -1}, 8) == 56
    assert queue_depth_for({"queue_depth": 10}, 4) == 10 and queue_depth_for({"queue_depth": 0}, 4) == 0
    with pytest.raises(Refusal, match="the most is 60"):
        queue_depth_for({"queue_depth": 64}, 4)


def test_systemone_formulas_and_letter_rule():
    """The decision models' formulas on hand-computed cases: p(technical) = 1/(1+e^-2) = 0.8808 and its confidence
    (0.8808 - 1/2) / (1/2) = 0.7616; softmax(0, 1, 0.5) = (0.1863, 0.5065, 0.3072), its score 1.1209 and confidence
    1 - (0.1863 + 0.3072) / (2/3) = 0.2597; a noul of scores (1, -1) is 0.8808."""
    from bloomery_b200.serve import systemone as S
    assert abs(S.confidence_choice([0.7, 0.2, 0.1]) - 0.55) < 1e-12 and S.confidence_choice([0.25] * 4) == 0.0 and S.confidence_choice([1.0]) == 1.0
    enc = lambda t: [300 if ch in "bc" else ord(ch) for ch in t]      # noqa: E731 - a vocabulary that cannot tell b from c
    state, qs = S.read_request({"state": {"k": 1}, "questions": {
        "department": {"type": "choice", "criteria": {"technical": "Bugs", "billing": "Pay"}},
        "urgency": {"type": "score", "criteria": ["Can wait", "This week", "Today"]}, "outage": {"type": "noul"},
        "twin": {"type": "choice", "criteria": {"ab": "x", "ac": "y"}}}})
    assert state == '{"k": 1}'
    schema = S.plan(qs, enc)
    assert schema["required"] == ["department", "urgency", "outage", "twin"] and schema["properties"]["twin"] == {"enum": ["A", "B"]}
    assert schema["properties"]["department"] == {"enum": ["technical", "billing"]} and not qs[0].by_letter and qs[3].by_letter
    assert "A = ab: x" in S.schema_text(qs)
    assert S.first_tokens(['"ab"', '"ac"'], enc) is None and S.first_tokens(['"ab"', '"ac"'], lambda t: list(t.encode())) == [98, 99]
    assert S.answer(qs[0], "technical", [2.0, 0.0]) == {"type": "choice", "choice": "technical", "confidence": 0.7616,
                                                        "probabilities": {"technical": 0.8808, "billing": 0.1192}}
    assert S.answer(qs[1], 1, [0.0, 1.0, 0.5]) == {"type": "score", "score": 1.1209, "confidence": 0.2597,
                                                   "legend": {"0": "Can wait", "1": "This week", "2": "Today"},
                                                   "probabilities": {"0": 0.1863, "1": 0.5065, "2": 0.3072}}
    assert S.answer(qs[2], True, [1.0, -1.0]) == {"type": "noul", "noul": 0.8808}
    assert S.answer(qs[3], "B", [0.0, 0.0])["choice"] == "ac"         # the answer names the option, never the letter
    # the pick rows are looked up where each question's options part in the canonical document
    doc = '{"department": "billing", "urgency": 2, "outage": false, "twin": "A"}'
    rows = []
    for q, sc in zip(qs, ([2.0, 0.0], [0.0, 1.0, 0.5], [1.0, -1.0], [3.0, 1.0])):
        lead = len(S._common(q.literals))
        row = [0.0] * 301
        for lit, v in zip(q.literals, sc):
            row[enc(lit[lead:])[0]] = v
        at = doc.index(json.dumps(q.id) + ": ") + len(json.dumps(q.id)) + 2 + lead
        rows.append((at, row))
    got = S.answers(qs, doc, rows, enc)
    assert got["department"]["choice"] == "billing" and got["department"]["probabilities"]["technical"] == 0.8808
    assert got["urgency"]["score"] == 1.1209 and got["outage"]["noul"] == 0.8808 and got["twin"]["choice"] == "ab"
    with pytest.raises(S.SystemOneError):
        S.answers(qs, doc[:-5], rows, enc)
    with pytest.raises(S.SystemOneError):
        S.plan(S.read_request({"state": "s", "questions": {"q": {"type": "choice", "criteria": {f"a{i:02d}": "x" for i in range(27)}}}})[1], enc)
    with pytest.raises(S.SystemOneError, match="not finite"):
        S.probabilities([0.0, float("inf")])


def test_start_screen_reads_the_record_lines_as_printed():
    from bloomery_b200.serve import screen as S
    from bloomery_b200.utils import records
    plain = S.Style.of({"TERM": "dumb", "LANG": "en_US.UTF-8"})
    assert plain == S.Style(False, False, False)
    assert S.Style.of({"LANG": "en_US.UTF-8", "COLORTERM": "truecolor"}) == S.Style(True, True, True)
    assert S.Style.of({"LC_ALL": "C", "LANG": "en_US.UTF-8", "NO_COLOR": "1"}) == S.Style(False, False, False)
    assert S.Style.of({"NO_COLOR": "", "LANG": "C.UTF-8"}).color                         # set but empty does not count
    assert "38;5;" in S.Style(True, False, True).paint("x", S.ORANGE) and "38;2;255;140;40" in S.Style(True, True, True).paint("x", S.ORANGE)
    got: list = []
    S.arm({}, True, "on")
    records.tap(S.note)
    import io
    sink = io.StringIO()
    records.write("plan", _out=sink, model="m", devices=[0, 1], weights_bytes=32 << 30, kv_bytes=4 << 30, ctx=32768, slots=4, place="tp2")
    records.write("need", _out=sink, host_bytes=8 << 30, cache_ram=8 << 30)
    records.write("ctx", _out=sink, asked=0, served=16384, trained=262144, rule="fitted")
    records.write("ctx", _out=sink, asked=0, served=32768, trained=262144, rule="fitted")       # the last line of a kind is the row
    records.write("parallel", _out=sink, slots=4, slot_ctx=8192, source="auto")
    lines = S.records()
    assert len(lines) == 5 and lines[0].startswith("plan\t")
    wide = S.draw(lines, "http://127.0.0.1:8080", 120, plain, live_keys=True)
    assert "serving on http://127.0.0.1:8080" in wide and "cards x2     32.0 GiB" in wide and "host          8.0 GiB" in wide
    assert "context    32,768 (fitted)" in wide and "16,384" not in wide and "slots      4 (from auto)" in wide
    assert "prompt cache 8.0 GiB" in wide and "d shows the live view" in wide and "unread" not in wide
    assert any("where the model went" in ln and "how it serves" in ln for ln in wide.splitlines())       # side by side
    narrow = S.draw(lines, "http://x", 50, plain)
    assert not any("where the model went" in ln and "how it serves" in ln for ln in narrow.splitlines())
    assert all(len(ln) <= 50 for ln in narrow.splitlines()) and "d shows" not in narrow
    # a fact whose record was not printed is left off; a value that is no number is named, never dropped
    few = S.draw(['ctx\t{"served":"lots"}', 'need\tnot json'], "http://x", 80, plain)
    assert "where the model went" not in few and "ctx.served='lots'" in few and "need: not json" in few
    with pytest.raises(ValueError):
        S.draw(lines, "http://x", 3, plain)
    # piped stderr is never armed
    assert S.arm({}, False, "on") is False and S.draw_if_armed("http://x") is False
    assert S.arm({}, True, "off") is False
    S.arm({}, True, "on")
    out = io.StringIO()
    assert S.draw_if_armed("http://y", env={"TERM": "dumb"}, out=out) and "serving on http://y" in out.getvalue()
    S.arm({}, False)
    # the live view: the newest request lines under a line of counters, cut to the width
    ring = S.Ring(3)
    for i in range(5):
        ring.push(f"bloomery-serve: request {i} /completion: prompt 10 ids")
    view = S.live_view(ring, {"rounds": 12, "ids": 340}, 40, plain)
    assert "request 4" in view and "request 1" not in view and "rounds 12" in view and all(len(ln) <= 40 for ln in view.splitlines())
    assert "no request has ended yet" in S.live_view(S.Ring(), {}, 40, plain)
    assert S.watch_keys(lambda ch: None, stdin=io.StringIO("d")) is None                 # stdin is no terminal: no keys
