"""Tokenizers: build request contexts from text, decode generated ids back to text.

``TextTokenizer`` delegates to a Hugging Face ``AutoTokenizer`` loaded from a local
directory (reference: max/python/max/pipelines/lib/tokenizer.py:413, ``new_context`` :672).
``ByteTokenizer`` is a dependency-free fallback (UTF-8 bytes + a few specials) used by
random-weight runs and tests, where no tokenizer files exist.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Sequence, Union

import numpy as np

from .context import SamplingParams, TextContext


class PipelineTokenizer:
    eos_token_ids: tuple = ()
    vocab_size: int = 0

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        raise NotImplementedError

    def apply_chat_template(self, messages: list, tools=None, add_generation_prompt: bool = True) -> str:
        parts = []
        for m in messages:
            content = m.get("content", "")
            if isinstance(content, list):
                content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
            parts.append(f"<|{m.get('role', 'user')}|>\n{content}\n")
        if add_generation_prompt:
            parts.append("<|assistant|>\n")
        return "".join(parts)

    def new_context(self, prompt: Union[str, Sequence[int]], max_length: int,
                    sampling_params: Optional[SamplingParams] = None, request_id: Optional[str] = None,
                    model_name: str = "") -> TextContext:
        ids = self.encode(prompt) if isinstance(prompt, str) else list(prompt)
        if len(ids) == 0:
            raise ValueError("prompt encodes to zero tokens")
        if len(ids) >= max_length:
            raise ValueError(f"prompt has {len(ids)} tokens, max_length is {max_length}")
        if not isinstance(prompt, str):
            # ids a client sends directly index the embedding table: they must lie inside the vocabulary
            vocab = int(getattr(self, "vocab_size", 0) or 0)
            lo, hi = min(ids), max(ids)
            if lo < 0 or (vocab and hi >= vocab):
                raise ValueError(f"prompt token ids must be in [0, {vocab or 'vocab size'}); got {lo if lo < 0 else hi}")
        sp = sampling_params or SamplingParams()
        if sp.stop:
            # single-token stop strings become stop ids; longer ones are matched on text downstream
            extra = []
            for s in sp.stop:
                t = self.encode(s, add_special_tokens=False)
                if len(t) == 1:
                    extra.append(t[0])
            if extra:
                sp.stop_token_ids = list(sp.stop_token_ids or []) + extra
        return TextContext.from_prompt(np.asarray(ids, dtype=np.int64), max_length, request_id, sp,
                                       self.eos_token_ids, model_name=model_name)


class ByteTokenizer(PipelineTokenizer):
    """ids 0..255 are bytes, 256 = BOS, 257 = EOS; ids above map to '?' when decoding."""

    BOS, EOS = 256, 257

    def vocab_bytes(self, vocab_size: int) -> list:
        """Byte string of every token id (for grammar compilers)."""
        return [bytes([i]) if i < 256 else (b"<s>" if i == self.BOS else b"</s>" if i == self.EOS else b"")
                for i in range(vocab_size)]

    def __init__(self, vocab_size: int = 258):
        self.vocab_size = max(vocab_size, 258)
        self.eos_token_ids = (self.EOS,)

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.BOS] if add_special_tokens else []) + ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        out = bytearray()
        for i in ids:
            i = int(i)
            if i < 256:
                out.append(i)
            elif not skip_special_tokens:
                out.extend(f"<{i}>".encode())
            elif i > self.EOS:
                out.extend(b"?")
        return out.decode("utf-8", errors="replace")


class TextTokenizer(PipelineTokenizer):
    def __init__(self, model_path: str, trust_remote_code: bool = False, max_length: Optional[int] = None):
        from transformers import AutoTokenizer

        self.delegate = AutoTokenizer.from_pretrained(model_path, trust_remote_code=trust_remote_code,
                                                      local_files_only=True)
        self.vocab_size = len(self.delegate)
        eos = set()
        if self.delegate.eos_token_id is not None:
            eos.add(int(self.delegate.eos_token_id))
        gen = Path(model_path) / "generation_config.json"
        if gen.exists():
            e = json.loads(gen.read_text()).get("eos_token_id")
            if isinstance(e, int):
                eos.add(e)
            elif isinstance(e, list):
                eos.update(int(x) for x in e)
        self.eos_token_ids = tuple(sorted(eos))

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        return list(self.delegate.encode(text, add_special_tokens=add_special_tokens))

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.delegate.decode(list(map(int, ids)), skip_special_tokens=skip_special_tokens)

    def apply_chat_template(self, messages: list, tools=None, add_generation_prompt: bool = True) -> str:
        if getattr(self.delegate, "chat_template", None):
            return self.delegate.apply_chat_template(messages, tools=tools, tokenize=False,
                                                     add_generation_prompt=add_generation_prompt)
        return super().apply_chat_template(messages, tools, add_generation_prompt)


def load_tokenizer(model_path: str, vocab_size: int = 258, trust_remote_code: bool = False) -> PipelineTokenizer:
    p = Path(model_path) if model_path else None
    if p is not None and (p / "tokenizer.json").exists() or (p is not None and (p / "tokenizer.model").exists()):
        return TextTokenizer(str(p), trust_remote_code)
    return ByteTokenizer(vocab_size)
