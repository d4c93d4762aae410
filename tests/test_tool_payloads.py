"""Tool-call payload normalisation and schema-conformance observation (pure Python)."""

import json

from modular_b200.serve.parser.conformance import (MAX_REPORTED_ERRORS, check_response_format, check_tool_calls,
                                                    tool_schemas)
from modular_b200.serve.parser.normalization import (anchor_object_schemas, tool_call_arguments_as_mappings,
                                                      tools_with_parameters)


def test_tool_call_arguments_become_mappings_without_touching_the_input():
    calls = [{"id": "a", "function": {"name": "f", "arguments": '{"x": 1}'}},
             {"id": "b", "function": {"name": "g", "arguments": ""}},
             {"id": "c", "function": {"name": "h"}},
             {"id": "d", "function": {"name": "i", "arguments": {"y": [2]}}},
             {"id": "e", "function": {"name": "j", "arguments": "{not json"}},
             {"id": "f"}]
    before = json.dumps(calls)
    out = tool_call_arguments_as_mappings(calls)
    assert [c.get("function", {}).get("arguments") for c in out] == [{"x": 1}, {}, {}, {"y": [2]}, "{not json", None]
    assert json.dumps(calls) == before


def test_tools_without_parameters_get_an_empty_mapping():
    tools = [{"type": "function", "function": {"name": "now", "parameters": None}},
             {"type": "function", "function": {"name": "add", "parameters": {"type": "object"}}},
             {"type": "function", "function": {"name": "ping"}}, {"type": "other"}]
    out = tools_with_parameters(tools)
    assert out[0]["function"]["parameters"] == {} and out[2]["function"]["parameters"] == {}
    assert out[1]["function"]["parameters"] == {"type": "object"} and out[3] == {"type": "other"}
    assert tools[0]["function"]["parameters"] is None


def test_object_shaped_schemas_are_anchored_at_every_depth():
    schema = {"properties": {"a": {"required": ["b"], "properties": {"b": {"type": "string"}}},
                             "list": {"type": "array", "items": {"additionalProperties": False}},
                             "any": {}},
              "anyOf": [{"patternProperties": {"^x": {}}}, {"type": "null"}],
              "$defs": {"d": {"properties": {}}}}
    out = anchor_object_schemas(schema)
    assert out["type"] == "object" and out["properties"]["a"]["type"] == "object"
    assert out["properties"]["list"]["items"]["type"] == "object"
    assert out["properties"]["any"] == {}                       # "any value" stays
    assert out["anyOf"][0]["type"] == "object" and out["anyOf"][1] == {"type": "null"}
    assert out["$defs"]["d"]["type"] == "object"
    assert "type" not in schema and "type" not in schema["properties"]["a"]      # input untouched
    typed = {"type": "object", "properties": {"n": {"type": ["integer", "null"]}}}
    assert anchor_object_schemas(typed) is typed                # nothing to change: same object back


def test_tool_call_conformance_outcomes():
    tools = [{"type": "function", "function": {"name": "weather", "parameters": {
                  "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer", "minimum": 1}},
                  "required": ["city"], "additionalProperties": False}}},
             {"type": "function", "function": {"name": "now"}}]
    schemas, names = tool_schemas(tools)
    assert set(schemas) == {"weather"} and names == {"weather", "now"}
    res = check_tool_calls([("weather", '{"city": "Oslo", "days": 2}'), ("weather", '{"days": 0, "zip": 1}'),
                            ("weather", '{"city": '), ("now", ""), ("nope", "{}"), ("weather", {"city": "Rome"})],
                           schemas, names)
    assert [r.outcome for r in res] == ["valid", "schema_mismatch", "invalid_json", "valid", "unknown_tool", "valid"]
    bad = res[1]
    assert sorted(e.split("@")[0] for e in bad.errors) == ["additionalProperties", "minimum", "required"]
    assert all("0" not in e.split("@")[0] for e in bad.errors)       # keywords and paths only, no values
    many = check_tool_calls([("weather", json.dumps({f"k{i}": i for i in range(12)}))],
                            {"weather": {"type": "object", "properties": {f"k{i}": {"type": "string"} for i in range(12)}}})
    assert len(many[0].errors) == MAX_REPORTED_ERRORS and many[0].more_errors == 12 - MAX_REPORTED_ERRORS
    # a schema that does not compile proves nothing about the model
    assert check_tool_calls([("f", "{}")], {"f": {"type": "no-such-type"}})[0].outcome == "valid"


def test_response_format_conformance():
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}
    assert check_response_format('{"ok": true}', schema).outcome == "valid"
    assert check_response_format("", schema).outcome == "invalid_json"
    r = check_response_format('{"ok": "yes"}', schema)
    assert r.outcome == "schema_mismatch" and r.errors == ["type@$.ok"]


def test_chat_route_uses_both(monkeypatch):
    """The chat route decodes earlier tool-call arguments for the template, fills in missing tool parameters, and
    counts a generated call that breaks its schema."""
    from modular_b200.serve.router import openai_routes as R
    from modular_b200.serve.schemas.openai import ChatCompletionRequest
    from modular_b200.serve.telemetry.metrics import METRICS

    seen = {}

    class Tok:
        def apply_chat_template(self, msgs, tools=None, add_generation_prompt=True):
            seen["msgs"], seen["tools"] = msgs, tools
            return "prompt"

    class Pipe:
        tokenizer = Tok()

    req = ChatCompletionRequest(model="m", messages=[
        {"role": "user", "content": "hi"},
        {"role": "assistant", "tool_calls": [{"id": "1", "type": "function",
                                              "function": {"name": "weather", "arguments": '{"city": "Oslo"}'}}]},
        {"role": "tool", "tool_call_id": "1", "content": "rain"}],
        tools=[{"type": "function", "function": {"name": "weather", "parameters": {
            "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}},
            {"type": "function", "function": {"name": "now", "parameters": None}}])
    assert R._chat_prompt(Pipe(), req) == "prompt"
    assert seen["msgs"][1]["tool_calls"][0]["function"]["arguments"] == {"city": "Oslo"}
    assert seen["tools"][1]["function"]["parameters"] == {}

    def count():
        return METRICS.tool_call_nonconforming._value.get() if METRICS.enabled else 0

    n0 = count()
    R._observe_conformance(req, tool_calls=[{"function": {"name": "weather", "arguments": "{}"}},
                                            {"function": {"name": "weather", "arguments": '{"city": "Rome"}'}},
                                            {"function": {"name": "missing", "arguments": "{}"}}])
    if METRICS.enabled:
        assert count() == n0 + 2
