"""Finds the JSON objects embedded in free text.

Models emit tool calls as JSON somewhere in their answer, sometimes after a marker token, sometimes several
separated by ``;`` or new lines, sometimes followed by chatter. A brace scanner that knows about string
literals and escapes cuts out every balanced top-level ``{...}`` span; spans that do not parse are skipped.
Reference: max/python/max/serve/parser/json_utils.py (``parse_json_from_text``).
"""

from __future__ import annotations

import json
from typing import Iterator


def _object_spans(text: str) -> Iterator[tuple[int, int]]:
    depth, start, in_str, esc = 0, -1, False, False
    for i, ch in enumerate(text):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"' and depth > 0:
            in_str = True
        elif ch == "{":
            if depth == 0:
                start = i
            depth += 1
        elif ch == "}" and depth > 0:
            depth -= 1
            if depth == 0:
                yield start, i + 1


def parse_json_objects(text: str) -> list[dict]:
    """Every top-level JSON object in ``text``, in order of appearance."""
    out = []
    for a, b in _object_spans(text):
        try:
            obj = json.loads(text[a:b])
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict):
            out.append(obj)
    return out


def first_object_start(text: str) -> int:
    """Index of the first ``{`` that is not inside a string literal of an enclosing object, or -1."""
    return text.find("{")
