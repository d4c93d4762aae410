"""Incremental, UTF-8-safe detokenisation with stop-string detection.

Tokens arrive one chunk at a time; text may only be emitted when it cannot change any more:
* a token can end in the middle of a multi-byte character (the decoder then yields U+FFFD),
  so the tail is held back until it decodes cleanly;
* some tokenizers change the rendering of a token depending on its predecessor (leading
  spaces), so decoding always re-reads a small window of previous tokens;
* while the emitted text could still grow into one of the stop strings, the overlapping
  suffix is held back; when a stop string completes, output is cut before it.

Reference: max/python/max/serve/pipelines/incremental_detokenizer.py.
"""

from __future__ import annotations

from typing import Optional, Sequence


class IncrementalDetokenizer:
    def __init__(self, tokenizer, stop: Optional[Sequence[str]] = None, skip_special_tokens: bool = True,
                 window: int = 6):
        self.tok = tokenizer
        self.stop = [s for s in (stop or []) if s]
        self.skip_special = skip_special_tokens
        self.window = window
        self.ids: list[int] = []
        self.prefix_offset = 0      # start of the re-decode window
        self.read_offset = 0        # tokens already turned into text
        self.text = ""              # all decoded text so far
        self.emitted = 0            # characters already handed out
        self.stopped = False

    def _decode_new(self) -> str:
        prefix = self.tok.decode(self.ids[self.prefix_offset:self.read_offset], self.skip_special)
        full = self.tok.decode(self.ids[self.prefix_offset:], self.skip_special)
        if full.endswith("�"):
            return ""               # incomplete multi-byte sequence: wait for more tokens
        new = full[len(prefix):]
        self.prefix_offset = max(self.read_offset - self.window, 0) if len(self.ids) > self.window else 0
        self.prefix_offset = max(len(self.ids) - self.window, 0)
        self.read_offset = len(self.ids)
        return new

    def _holdback(self) -> int:
        """Characters at the end of ``text`` that might be the start of a stop string."""
        hold = 0
        for s in self.stop:
            for k in range(min(len(s) - 1, len(self.text) - self.emitted), 0, -1):
                if self.text.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        return hold

    def push(self, token_ids: Sequence[int], final: bool = False) -> str:
        """Add tokens; returns the text that became safe to emit."""
        if self.stopped:
            return ""
        self.ids.extend(int(t) for t in token_ids)
        self.text += self._decode_new()
        if final and self.read_offset < len(self.ids):
            self.text += self.tok.decode(self.ids[self.read_offset:], self.skip_special)
            self.read_offset = len(self.ids)
        for s in self.stop:
            pos = self.text.find(s, max(0, self.emitted - len(s) + 1))
            if pos != -1:
                out = self.text[self.emitted:pos]
                self.text = self.text[:pos]
                self.emitted = pos
                self.stopped = True
                return out
        end = len(self.text) - (0 if final else self._holdback())
        out = self.text[self.emitted:end]
        self.emitted = max(self.emitted, end)
        return out
