"""Did the model's tool calls and JSON answers match the schemas the client declared?

Observation only: the checks feed the serve log and the metrics, never change a response and never raise. Only
names that come from the developer's schema are reported - function name, failing JSON Schema keyword and the JSON
path of the offending node - never argument values or validator messages (which quote them).

Schemas are validated as JSON Schema draft 7 whatever ``$schema`` they declare. A schema that does not compile,
or whose references cannot be resolved, proves nothing about the model and counts as ``valid``.

Reference: max/python/max/serve/parser/tool_call_validation.py (check_tool_call_conformance :106,
check_response_format_conformance :189).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from functools import lru_cache
from typing import Any, Collection, Mapping, Optional, Sequence

MAX_REPORTED_ERRORS = 5


@dataclass
class Conformance:
    outcome: str                       # valid | invalid_json | unknown_tool | schema_mismatch
    function: Optional[str] = None     # tool calls only
    errors: list = field(default_factory=list)     # "keyword@json.path", at most MAX_REPORTED_ERRORS
    more_errors: int = 0


@lru_cache(maxsize=1024)
def _validator(schema_json: str):
    try:
        from jsonschema import Draft7Validator

        schema = json.loads(schema_json)
        Draft7Validator.check_schema(schema)
        return Draft7Validator(schema)
    except Exception:      # noqa: BLE001 - missing package, broken schema: nothing to hold against the model
        return None


def _validate(instance: Any, schema: Mapping) -> Optional[tuple]:
    """(errors, more) of ``instance`` against ``schema``; None when the schema cannot be used."""
    try:
        v = _validator(json.dumps(schema, sort_keys=True, separators=(",", ":")))
    except (TypeError, ValueError):
        return None
    if v is None:
        return None
    errors, more = [], 0
    try:
        for e in v.iter_errors(instance):
            if len(errors) < MAX_REPORTED_ERRORS:
                errors.append(f"{e.validator}@{e.json_path}")
            else:
                more += 1
    except Exception:      # noqa: BLE001 - e.g. an unresolvable $ref
        return None
    return errors, more


def check_tool_calls(calls: Sequence[tuple], schemas_by_name: Mapping[str, Mapping],
                     known_tools: Optional[Collection[str]] = None) -> list:
    """One :class:`Conformance` per ``(name, arguments)``. ``arguments``: the JSON text the model wrote (blank =
    ``{}``) or an already decoded value. A declared tool without a parameter schema is ``valid``; a name that was
    never declared is ``unknown_tool``."""
    declared = schemas_by_name.keys() if known_tools is None else known_tools
    out = []
    for name, args in calls:
        schema = schemas_by_name.get(name)
        if schema is None:
            out.append(Conformance("valid" if name in declared else "unknown_tool", name))
            continue
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except json.JSONDecodeError:
                out.append(Conformance("invalid_json", name))
                continue
        res = _validate(args, schema)
        if res is None or not res[0]:
            out.append(Conformance("valid", name))
        else:
            out.append(Conformance("schema_mismatch", name, res[0], res[1]))
    return out


def check_response_format(content: str, schema: Mapping) -> Conformance:
    """The final message text of a request that asked for JSON (``json_schema`` / ``json_object``). Empty text is
    ``invalid_json``: the client asked for a document and got none."""
    try:
        doc = json.loads(content)
    except (json.JSONDecodeError, TypeError):
        return Conformance("invalid_json")
    res = _validate(doc, schema)
    if res is None or not res[0]:
        return Conformance("valid")
    return Conformance("schema_mismatch", None, res[0], res[1])


def tool_schemas(tools: Optional[Sequence[Mapping]]) -> tuple:
    """(parameter schema by function name, all declared names) of an OpenAI ``tools`` list."""
    schemas, names = {}, set()
    for t in tools or ():
        fn = t.get("function") if isinstance(t, Mapping) else None
        if isinstance(fn, Mapping) and isinstance(fn.get("name"), str):
            names.add(fn["name"])
            if isinstance(fn.get("parameters"), Mapping) and fn["parameters"]:
                schemas[fn["name"]] = fn["parameters"]
    return schemas, names
