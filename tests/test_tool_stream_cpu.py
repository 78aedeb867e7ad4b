"""Incremental tool-call streaming: the name is announced when its string closes, argument text
arrives in fragments, and the concatenation equals what the end-of-text parser extracts
(reference behaviour: src/server/tool_calls/incremental.rs and its stream-parity tests)."""
import json

import pytest

from mlxcel_b200.server.tool_calls import IncrementalToolCallStreamer, parse_tool_calls

CASES = [
    ('I will call. <tool_call>\n{"name": "get_weather", "arguments": {"city": "Seoul {x}", "days": [1, 2, {"a": "}"}]}}\n'
     '</tool_call> and <tool_call>{"arguments": {"q": 1}, "name": "search"}</tool_call> done', None),
    ('<|python_tag|>{"name": "f", "parameters": {"a": "b\\"c"}}; {"name": "g", "parameters": {}}', None),
    ('[TOOL_CALLS] [{"name": "h", "arguments": {"k": [1, 2]}}, {"name": "i", "arguments": {}}]', None),
    ('[TOOL_CALLS]get_x[ARGS]{"a": {"b": 2}}', None),
    ('x <function=foo>{"a": 1}</function> y', None),
    ('<tool_call>{"function": {"name": "f", "arguments": "{\\"a\\": 1}"}}</tool_call>', {"f"}),
    ('<tool_call>{"name": "nope", "arguments": {"a": 1}}</tool_call><tool_call>{"name": "f", "arguments": {}}</tool_call>', {"f"}),
]


def _stream(text, allowed, step):
    f = IncrementalToolCallStreamer(allowed)
    vis, ds = "", []
    for i in range(0, len(text), step):
        v, d = f.feed(text[i:i + step])
        vis += v
        ds += d
    v, d = f.flush()
    return vis + v, ds + d, f


@pytest.mark.parametrize("text,allowed", CASES)
@pytest.mark.parametrize("step", [1, 4, 9, 10_000])
def test_streamed_calls_equal_the_final_parse(text, allowed, step):
    vis, ds, f = _stream(text, allowed, step)
    content, want = parse_tool_calls(text, allowed)
    got = {}
    for d in ds:
        c = got.setdefault(d["index"], dict(name=None, args="", id=None))
        if "id" in d:
            assert c["id"] is None, "a call is announced once"
            c.update(id=d["id"], name=d["function"]["name"])
        else:
            assert c["id"] is not None, "fragments follow the announcement"
        c["args"] += d["function"]["arguments"]
    assert sorted(got) == list(range(len(want)))
    for i, w in enumerate(want):
        assert got[i]["name"] == w.name
        assert json.loads(got[i]["args"]) == json.loads(w.arguments)
    assert " ".join(vis.split()) == " ".join(content.split())
    assert f.n == len(want)


def test_arguments_arrive_before_the_region_closes():
    f = IncrementalToolCallStreamer({"get_weather"})
    v, d = f.feed('<tool_call>{"name": "get_weather", "argum')
    assert v == "" and len(d) == 1 and d[0]["function"] == {"name": "get_weather", "arguments": ""}
    v, d = f.feed('ents": {"city": "Se')
    assert [x["function"]["arguments"] for x in d] == ['{"city": "Se']
    v, d = f.feed('oul"}}')
    assert "".join(x["function"]["arguments"] for x in d) == 'oul"}'
    v, d = f.feed("</tool_call>tail")
    assert d == [] and v == "tail"


def test_marker_prefixes_are_held_and_released():
    f = IncrementalToolCallStreamer()
    v1, _ = f.feed("a <tool")
    v2, _ = f.feed("box> b")
    v3, _ = f.flush()
    assert v1 == "a " and v1 + v2 + v3 == "a <toolbox> b"
