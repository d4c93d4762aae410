"""Tool-call parsers, selected by name (``tool_parser`` runtime option).

``llama``: Llama-3 chat templates make the model answer with a JSON object ``{"name": ..., "parameters":
{...}}`` (optionally after ``<|python_tag|>``, several objects separated by ``;``). ``hermes``: Qwen /
Hermes style ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks next to normal text.

A parser has two modes: ``parse_complete(text)`` for a finished answer and ``parse_delta(chunk)`` for
streaming, which withholds text that may still turn into a tool call and releases either plain content or
finished calls. Reference: max/python/max/serve/parser/llama_tool_parser.py (the reference does not stream
Llama tool calls; here the call is emitted as soon as its JSON object closes).
"""

from __future__ import annotations

import json
import uuid
from dataclasses import dataclass, field
from typing import Callable, Optional

from .json_utils import parse_json_objects


@dataclass
class ParsedToolCall:
    name: str
    arguments: str                      # JSON text, as the OpenAI API carries it
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:16])

    def to_openai(self, index: Optional[int] = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ParsedResponse:
    content: Optional[str]
    tool_calls: list


class ToolParser:
    """Base class: subclasses implement ``parse_complete`` and may refine ``parse_delta``."""

    def __init__(self) -> None:
        self._buffer = ""
        self._emitted = 0
        self._plain = False      # plain content has been released: the rest of the answer is content too

    def reset(self) -> None:
        self._buffer, self._emitted, self._plain = "", 0, False

    def parse_complete(self, text: str) -> ParsedResponse:
        raise NotImplementedError

    def may_start_call(self, text: str) -> bool:
        """True while ``text`` (everything generated so far) could still be, or contain, a tool call."""
        raise NotImplementedError

    def parse_delta(self, chunk: str, final: bool = False) -> tuple[str, list]:
        """Feeds a piece of generated text. Returns ``(content_to_emit, finished_calls)``; text that might
        belong to a call is held back until the answer ends or the call completes."""
        if self._plain:
            return chunk, []
        self._buffer += chunk
        if not final and self.may_start_call(self._buffer):
            return "", self._try_partial()
        try:
            parsed = self.parse_complete(self._buffer)
        except ValueError:
            parsed = ParsedResponse(self._buffer, [])      # JSON that is not a tool call: ordinary content
        calls = parsed.tool_calls[self._emitted:]
        self._emitted = len(parsed.tool_calls)
        if parsed.tool_calls:
            return "", calls
        content, self._buffer, self._plain = self._buffer, "", True
        return content, []

    def _try_partial(self) -> list:
        """Calls whose JSON is already complete inside the held-back text."""
        try:
            parsed = self.parse_complete(self._buffer)
        except ValueError:
            return []
        calls = parsed.tool_calls[self._emitted:]
        self._emitted = len(parsed.tool_calls)
        return calls


_REGISTRY: dict[str, Callable[[], ToolParser]] = {}


def register_tool_parser(name: str):
    def deco(cls):
        _REGISTRY[name] = cls
        return cls
    return deco


def get_tool_parser(name: Optional[str]) -> Optional[ToolParser]:
    if not name:
        return None
    if name not in _REGISTRY:
        raise ValueError(f"unknown tool parser {name!r} (available: {sorted(_REGISTRY)})")
    return _REGISTRY[name]()


@register_tool_parser("llama")
class LlamaToolParser(ToolParser):
    MARKER = "<|python_tag|>"

    def parse_complete(self, text: str) -> ParsedResponse:
        body = text.strip()
        if body.startswith(self.MARKER):
            body = body[len(self.MARKER):].lstrip()
        calls = []
        if body.startswith("{"):
            for obj in parse_json_objects(body):
                if "name" not in obj or not ("parameters" in obj or "arguments" in obj):
                    raise ValueError("tool call JSON needs both a name and parameters")
                args = obj.get("parameters", obj.get("arguments"))
                calls.append(ParsedToolCall(str(obj["name"]), args if isinstance(args, str) else json.dumps(args)))
        return ParsedResponse(None if calls else text, calls)

    def may_start_call(self, text: str) -> bool:
        body = text.lstrip()
        if not body:
            return True
        return body.startswith("{") or self.MARKER.startswith(body[: len(self.MARKER)]) or body.startswith(self.MARKER)


@register_tool_parser("hermes")
class HermesToolParser(ToolParser):
    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def parse_complete(self, text: str) -> ParsedResponse:
        calls, content, pos = [], [], 0
        while True:
            a = text.find(self.OPEN, pos)
            if a < 0:
                content.append(text[pos:])
                break
            content.append(text[pos:a])
            b = text.find(self.CLOSE, a)
            inner = text[a + len(self.OPEN): b if b >= 0 else len(text)]
            for obj in parse_json_objects(inner):
                if "name" in obj:
                    args = obj.get("arguments", obj.get("parameters", {}))
                    calls.append(ParsedToolCall(str(obj["name"]), args if isinstance(args, str) else json.dumps(args)))
            if b < 0:
                break
            pos = b + len(self.CLOSE)
        rest = "".join(content).strip()
        return ParsedResponse(rest or None, calls)

    def may_start_call(self, text: str) -> bool:
        if self.OPEN in text:
            return text.rfind(self.OPEN) > text.rfind(self.CLOSE)     # an unclosed block
        tail = text[-(len(self.OPEN) - 1):]
        return any(self.OPEN.startswith(tail[i:]) for i in range(len(tail)))   # a partial opening tag

    def parse_delta(self, chunk: str, final: bool = False) -> tuple[str, list]:
        self._buffer += chunk
        if not final and self.may_start_call(self._buffer):
            # release the text in front of the (possible) tag, keep the rest
            cut = self._buffer.find(self.OPEN)
            if cut < 0:
                cut = max(0, len(self._buffer) - (len(self.OPEN) - 1))
            head, self._buffer = self._buffer[:cut], self._buffer[cut:]
            return head, []
        parsed = self.parse_complete(self._buffer)
        self._buffer = ""
        return parsed.content or "", parsed.tool_calls
