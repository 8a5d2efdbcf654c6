"""Property tests of the text surfaces that take untrusted input: chat templates, tool-call scanners,
the streaming scanner, the JSON constraint and the safetensors header reader.  Counterpart of the
reference's fuzz targets (``fuzz/README.md``: jinja parse / render and the four tool-call scanners):
whatever the bytes, these either answer or raise their own error type -- never another exception,
never a hang."""
import json
import struct

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from bloomery_b200.serve import chat as C

SET = settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
text = st.text(alphabet=st.characters(blacklist_categories=("Cs",)), max_size=200)
tagged = st.lists(st.sampled_from(["<tool_call>", "</tool_call>", "<function=", "</function>", "<parameter=", "</parameter>",
                                   "[TOOL_CALLS]", "{", "}", "[", "]", '"name"', ":", '"arguments"', ",", "<arg_key>",
                                   "</arg_key>", "<arg_value>", "</arg_value>", "x", " ", "\n", '"', "\\"]),
                  max_size=40).map("".join)


@SET
@given(st.one_of(text, tagged), st.sampled_from(["hermes", "qwen_xml", "glm_xml", "mistral"]))
def test_tool_call_scanners_answer_or_pass_text_through(s, fmt):
    content, calls = C.parse_tool_calls(s, fmt)
    assert isinstance(content, str) and isinstance(calls, list)
    for c in calls:
        assert c["type"] == "function" and isinstance(c["function"]["name"], str)
        json.loads(c["function"]["arguments"])               # arguments are always a JSON document


@SET
@given(st.one_of(text, tagged), st.integers(min_value=1, max_value=7))
def test_streaming_scanner_equals_one_shot_on_any_split(s, step):
    whole_content, whole_calls = C.parse_tool_calls(s, "hermes")
    stream = C.ToolCallStream("hermes")
    content, calls = "", []
    for i in range(0, len(s), step):
        c, k = stream.push(s[i:i + step])
        content += c
        calls += k
    content += stream.flush()
    assert [c["function"] for c in calls] == [c["function"] for c in whole_calls]
    if not whole_calls:
        assert content == s or content.strip() == whole_content.strip()


@SET
@given(text)
def test_templates_render_or_raise_template_error(src):
    try:
        t = C.ChatTemplate(src)
        out = t.render_text([{"role": "user", "content": "hi"}])
        assert isinstance(out, str)
    except C.TemplateError:
        pass


@SET
@given(st.lists(st.fixed_dictionaries({"role": st.sampled_from(["system", "user", "assistant", "tool"]), "content": text}),
                min_size=1, max_size=5))
def test_default_template_keeps_untrusted_text_out_of_the_control_channel(msgs):
    t = C.ChatTemplate()
    out = t.render_text(msgs)
    assert isinstance(out, str)
    assert C.G0 not in out and C.G1 not in out          # guard marks never survive into the rendered text


@SET
@given(text, text)
def test_json_constraint_never_raises(prefix, piece):
    jc = C.JsonConstraint({"type": "object"})
    assert jc.allowed(prefix, piece) in (True, False)
    assert jc.closed(prefix) in (True, False) and jc.done(prefix) in (True, False)


@SET
@given(st.binary(max_size=200))
def test_safetensors_reader_refuses_garbage_with_its_own_error(tmp_path_factory, blob):
    from bloomery_b200.formats.safetensors import Safetensors, SafetensorsError
    p = tmp_path_factory.mktemp("st") / "x.safetensors"
    p.write_bytes(blob)
    try:
        Safetensors(str(p)).close()
    except SafetensorsError:
        pass


def test_safetensors_header_tricks_are_refused(tmp_path):
    from bloomery_b200.formats.safetensors import Safetensors, SafetensorsError
    def file_with(header: dict, data: bytes = b"\0" * 64):
        hj = json.dumps(header).encode()
        p = tmp_path / "h.safetensors"
        p.write_bytes(struct.pack("<Q", len(hj)) + hj + data)
        return str(p)
    bad = [
        {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}},                 # shape does not match bytes
        {"a": {"dtype": "F32", "shape": [4], "data_offsets": [60, 76]}},               # past the end of the file
        {"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}, "b": {"dtype": "F32", "shape": [4], "data_offsets": [8, 24]}},
        {"a": {"dtype": "Q9", "shape": [4], "data_offsets": [0, 16]}},
        {"a": {"dtype": "F32", "shape": [4]}},
        {"a": {"dtype": "F32", "shape": [4], "data_offsets": [16, 0]}},
    ]
    for h in bad:
        with pytest.raises(SafetensorsError):
            Safetensors(file_with(h))
    ok = Safetensors(file_with({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}, "__metadata__": {"k": "v"}}))
    assert ok.tensor("a").shape == (4,) and ok.metadata == {"k": "v"}


@SET
@given(st.binary(max_size=600), st.binary(max_size=64), st.integers(min_value=0, max_value=96), st.integers(min_value=0, max_value=12))
def test_compressed_scale_decoders_refuse_or_answer(fixed, exc, rows, cols):
    """Whatever bytes stand where a checkpoint's compressed scales should be, the decoders answer with rows x cols bytes
    or raise their own error."""
    import numpy as np
    from bloomery_b200.formats import csf
    f8 = np.frombuffer(fixed, dtype=np.uint8)
    words = np.frombuffer(exc[:len(exc) // 4 * 4], dtype=np.uint32)
    try:
        out = csf.decode_csf("s", f8, words, rows, cols)
        assert out.shape == (rows, cols)
    except csf.CsfError:
        pass
    half = np.frombuffer(exc[:len(exc) // 2 * 2], dtype=np.uint16)
    try:
        out = csf.decode_csf32("s", f8[:rows], f8[rows:rows + rows * cols // 2], words[:1], half, half[::-1].copy(), rows, cols)
        assert out.shape == (rows, cols)
    except csf.CsfError:
        pass


@SET
@given(st.integers(min_value=1, max_value=4), st.integers(min_value=1, max_value=9), st.integers(min_value=0, max_value=2 ** 32 - 1))
def test_compressed_scale_round_trip_on_any_bytes(slabs, cols, seed):
    import numpy as np
    from bloomery_b200.formats import csf
    sc = np.random.default_rng(seed).integers(0, 256, size=(32 * slabs, cols), dtype=np.uint8)       # no window at all
    p = csf.encode_csf32(sc) if (32 * slabs * cols) % 2 == 0 else None
    if p is not None:
        assert np.array_equal(csf.decode_csf32("s", p["csf32_bases"], p["csf32_codes"], p["csf32_page_bases"], p["csf32_offsets"],
                                               p["csf32_exceptions"], 32 * slabs, cols), sc)
    if cols % 2 == 0:
        q = csf.encode_csf(sc)
        assert np.array_equal(csf.decode_csf("s", q["nvfp4_csf_fixed"], q["nvfp4_csf_exceptions"], 32 * slabs, cols), sc)


_json_values = st.recursive(st.one_of(st.none(), st.booleans(), st.integers(-99, 99), st.text(alphabet='ab"{}[]\\ <>/', max_size=6)),
                            lambda kids: st.one_of(st.lists(kids, max_size=3), st.dictionaries(st.text(alphabet="ab}", max_size=3), kids, max_size=3)),
                            max_leaves=8)


@SET
@given(st.lists(st.tuples(st.text(alphabet="abc_", min_size=1, max_size=6), st.dictionaries(st.text(alphabet="xy{", max_size=3), _json_values, max_size=3),
                          st.text(alphabet="ab <\n", max_size=8)), min_size=1, max_size=3),
       st.integers(min_value=1, max_value=9), st.booleans())
def test_call_deltas_reassemble_to_the_one_shot_calls_on_any_split(calls, step, compact):
    """Whatever the chunking and the JSON spacing, the streamed deltas of well-formed calls carry each name once, first,
    and argument fragments that join to the call's arguments; text outside the calls passes through."""
    sep = (",", ":") if compact else (", ", ": ")
    s = ""
    for name, args, between in calls:
        s += between.replace("<", "") + "<tool_call>\n" + json.dumps({"name": name, "arguments": args}, separators=sep) + "\n</tool_call>"
    whole_content, whole_calls = C.parse_hermes(s)
    stream = C.ToolCallDeltas()
    content, got = "", {}
    for i in range(0, len(s), step):
        c, ds = stream.push(s[i:i + step])
        content += c
        for d in ds:
            slot = got.setdefault(d["index"], {"name": None, "args": ""})
            if "name" in d["function"]:
                assert slot["name"] is None and slot["args"] == "" and d["type"] == "function" and d["id"]
                slot["name"] = d["function"]["name"]
            slot["args"] += d["function"]["arguments"]
    content += stream.flush()
    assert stream.open_call is None
    assert [(got[i]["name"], json.loads(got[i]["args"])) for i in sorted(got)] == [
        (c["function"]["name"], json.loads(c["function"]["arguments"])) for c in whole_calls]
    assert content.strip() == whole_content.strip() or "".join(content.split()) == "".join(whole_content.split())


@SET
@given(st.one_of(text, tagged), st.integers(min_value=1, max_value=7))
def test_call_deltas_answer_or_raise_their_own_error(s, step):
    stream = C.ToolCallDeltas()
    try:
        for i in range(0, len(s), step):
            t, ds = stream.push(s[i:i + step])
            assert isinstance(t, str) and isinstance(ds, list)
        assert isinstance(stream.flush(), str)
    except C.ToolStreamError as exc:
        assert isinstance(exc.name, str)
