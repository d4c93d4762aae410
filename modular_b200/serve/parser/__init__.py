"""Parsers that turn generated text into structured parts of a chat answer: tool calls and reasoning spans.

``normalization`` cleans tool payloads and response-format schemas on the way in, ``conformance`` observes whether
generated tool calls and JSON answers match the declared schemas.

Reference: max/python/max/serve/parser/ (``llama_tool_parser.py``, ``json_utils.py``,
``tool_call_normalization.py``, ``tool_call_validation.py``) and the ``tool_parser`` / ``reasoning_parser`` runtime
options (pipelines/lib/pipeline_runtime_config.py).
"""

from .json_utils import parse_json_objects
from .reasoning import ReasoningSplitter, split_reasoning
from .tool_parser import (HermesToolParser, LlamaToolParser, ParsedToolCall, ToolParser, get_tool_parser,
                          register_tool_parser)

__all__ = ["parse_json_objects", "ReasoningSplitter", "split_reasoning", "HermesToolParser", "LlamaToolParser",
           "ParsedToolCall", "ToolParser", "get_tool_parser", "register_tool_parser"]
