"""Request-side clean-up of OpenAI tool payloads and response-format schemas.

* Chat templates iterate ``tool_calls[*].function.arguments`` as a mapping, while clients send the JSON-encoded
  string the OpenAI schema prescribes: :func:`tool_call_arguments_as_mappings` decodes them.
* ``tools[*].function.parameters: null`` means "no parameters": :func:`tools_with_parameters`.
* A JSON Schema node without ``type`` but with ``properties`` / ``required`` / ... accepts *any* value as far as
  the standard goes; a grammar compiled from it may let the model open a string it never has to close.
  :func:`anchor_object_schemas` writes the implied ``"type": "object"`` into such nodes, at every depth.

None of the functions mutates its input; unchanged sub-trees are shared with it.

Reference: max/python/max/serve/parser/tool_call_normalization.py (normalize_tool_call_arguments :21,
normalize_response_format_schema :84, _normalize_tools_parameters :186).
"""

from __future__ import annotations

import json
from typing import Any

_IMPLIES_OBJECT = ("properties", "required", "additionalProperties", "patternProperties")
_CHILD = ("items", "additionalItems", "contains", "not", "if", "then", "else")
_CHILD_MAPS = ("properties", "patternProperties", "$defs", "definitions")
_CHILD_LISTS = ("allOf", "anyOf", "oneOf", "prefixItems")


def tool_call_arguments_as_mappings(tool_calls: list) -> list:
    """Copies of ``tool_calls`` whose ``function.arguments`` are decoded: a JSON string becomes what it encodes,
    ``None`` / ``""`` / a missing key become ``{}``, mappings and lists stay, and a string that is not valid JSON is
    left alone (the template then shows the client's mistake instead of hiding it)."""
    out = []
    for call in tool_calls:
        call = dict(call) if isinstance(call, dict) else call
        fn = call.get("function") if isinstance(call, dict) else None
        if isinstance(fn, dict):
            fn = dict(fn)
            args = fn.get("arguments")
            if args is None or args == "":
                fn["arguments"] = {}
            elif isinstance(args, str):
                try:
                    fn["arguments"] = json.loads(args)
                except json.JSONDecodeError:
                    pass
            call["function"] = fn
        out.append(call)
    return out


def tools_with_parameters(tools: list) -> list:
    """Copies of ``tools`` in which a missing or ``null`` ``function.parameters`` is an empty mapping."""
    out = []
    for tool in tools:
        tool = dict(tool) if isinstance(tool, dict) else tool
        fn = tool.get("function") if isinstance(tool, dict) else None
        if isinstance(fn, dict):
            fn = dict(fn)
            if fn.get("parameters") is None:
                fn["parameters"] = {}
            tool["function"] = fn
        out.append(tool)
    return out


def anchor_object_schemas(schema: Any) -> Any:
    """``schema`` with ``"type": "object"`` added to every (sub)schema that omits ``type`` but uses an
    object-only keyword. ``{}`` ("any value") and nodes that already name a type are kept. Returns the input object
    itself when nothing had to change."""
    if not isinstance(schema, dict):
        return schema
    new = None      # a shallow copy, made on the first change

    def put(key, value):
        nonlocal new
        if new is None:
            new = dict(schema)
        new[key] = value

    if "type" not in schema and any(k in schema for k in _IMPLIES_OBJECT):
        put("type", "object")
    for key in _CHILD:
        child = schema.get(key)
        if isinstance(child, dict):
            fixed = anchor_object_schemas(child)
            if fixed is not child:
                put(key, fixed)
    for key in _CHILD_MAPS:
        children = schema.get(key)
        if isinstance(children, dict):
            fixed = {name: anchor_object_schemas(c) for name, c in children.items()}
            if any(fixed[name] is not children[name] for name in children):
                put(key, fixed)
    for key in _CHILD_LISTS:
        children = schema.get(key)
        if isinstance(children, list):
            fixed = [anchor_object_schemas(c) for c in children]
            if any(a is not b for a, b in zip(fixed, children)):
                put(key, fixed)
    return schema if new is None else new
