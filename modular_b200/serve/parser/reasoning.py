"""Splits a generated answer into its reasoning span (``<think>...</think>``) and the visible content.

The API reports the two separately (``reasoning_content`` / ``content``), also while streaming. Reference:
``reasoning_parser`` option of the reference's runtime config and the reasoning-span split in
max/python/max/serve/pipelines/llm.py.
"""

from __future__ import annotations

from typing import Optional


def split_reasoning(text: str, open_tag: str = "<think>", close_tag: str = "</think>") -> tuple[Optional[str], str]:
    """(reasoning, content) of a complete answer. A missing opening tag with a closing one means the chat
    template already opened the span."""
    b = text.find(close_tag)
    if b < 0:
        if text.lstrip().startswith(open_tag):
            return text.lstrip()[len(open_tag):], ""
        return None, text
    a = text.find(open_tag)
    start = a + len(open_tag) if 0 <= a < b else 0
    return text[start:b].strip() or None, text[b + len(close_tag):].lstrip("\n")


class ReasoningSplitter:
    """Streaming form: ``push(chunk)`` returns ``(reasoning_delta, content_delta)``."""

    def __init__(self, open_tag: str = "<think>", close_tag: str = "</think>", starts_in_reasoning: bool = False):
        self.open, self.close = open_tag, close_tag
        self.state = "reasoning" if starts_in_reasoning else "start"
        self.buf = ""

    def push(self, chunk: str, final: bool = False) -> tuple[str, str]:
        self.buf += chunk
        reasoning, content = "", ""
        while True:
            if self.state == "start":
                s = self.buf.lstrip()
                if s.startswith(self.open):
                    self.buf = s[len(self.open):]
                    self.state = "reasoning"
                    continue
                if not final and s and self.open.startswith(s):
                    break                      # may still become the opening tag
                if not s and not final:
                    break
                self.state = "content"
                continue
            if self.state == "reasoning":
                i = self.buf.find(self.close)
                if i >= 0:
                    reasoning += self.buf[:i]
                    self.buf = self.buf[i + len(self.close):].lstrip("\n")
                    self.state = "content"
                    continue
                keep = 0 if final else len(self.close) - 1     # a partial closing tag stays in the buffer
                cut = max(0, len(self.buf) - keep)
                reasoning += self.buf[:cut]
                self.buf = self.buf[cut:]
                break
            content += self.buf
            self.buf = ""
            break
        return reasoning, content
