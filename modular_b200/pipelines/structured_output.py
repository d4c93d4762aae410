"""Grammar-constrained decoding: JSON / JSON-schema / regex / EBNF through xgrammar.

``StructuredOutputBackend`` compiles a grammar per request (cached by xgrammar), hands out a
``GrammarState`` that lives in the request's context, and fills the packed token bitmask
``[rows, ceil(vocab / 32)]`` int32 (bit = token allowed) that ``ops.apply_token_bitmask`` applies to
the logits before sampling. After a token is sampled the state ``accept``s it; when the grammar
is complete only the stop tokens remain allowed, so the request ends with EOS.

Reference: max/python/max/pipelines/lib/pipeline_variants/structured_output_backend.py,
``StructuredOutputHelper`` (pipeline_variants/utils.py:345) and the response_format handling in
serve/router/openai_routes.py.
"""

from __future__ import annotations

import json
from typing import Optional, Sequence

import numpy as np
import torch


def response_format_to_spec(response_format) -> Optional[dict]:
    """OpenAI ``response_format`` (dict or pydantic object) -> {"type", ...} grammar spec, or None for text."""
    if response_format is None:
        return None
    rf = response_format if isinstance(response_format, dict) else response_format.model_dump(exclude_none=True)
    t = rf.get("type", "text")
    if t == "text":
        return None
    if t == "json_object":
        return {"type": "json_object"}
    if t == "json_schema":
        js = rf.get("json_schema") or {}
        schema = js.get("schema", js) if isinstance(js, dict) else js
        return {"type": "json_schema", "schema": schema if isinstance(schema, str) else json.dumps(schema)}
    if t in ("regex", "ebnf"):
        return {"type": t, "pattern": rf.get("pattern") or rf.get("grammar") or ""}
    raise ValueError(f"unsupported response_format type {t!r}")


class GrammarState:
    """Per-request matcher."""

    def __init__(self, matcher):
        self.matcher = matcher

    def accept(self, token: int) -> bool:
        if self.matcher.is_terminated():
            return True
        return bool(self.matcher.accept_token(int(token)))

    @property
    def terminated(self) -> bool:
        return bool(self.matcher.is_terminated())

    def fill(self, bitmask: torch.Tensor, row: int) -> None:
        self.matcher.fill_next_token_bitmask(bitmask, row)


class StructuredOutputBackend:
    def __init__(self, tokenizer, vocab_size: int):
        import xgrammar as xgr

        self.xgr, self.vocab_size = xgr, vocab_size
        hf = getattr(tokenizer, "hf_tokenizer", None)
        if hf is not None:
            self.info = xgr.TokenizerInfo.from_huggingface(hf, vocab_size=vocab_size)
        else:
            vocab = tokenizer.vocab_bytes(vocab_size) if hasattr(tokenizer, "vocab_bytes") else \
                [tokenizer.decode([i]).encode("utf-8") for i in range(vocab_size)]
            self.info = xgr.TokenizerInfo(vocab, vocab_type=xgr.VocabType.RAW, vocab_size=vocab_size,
                                          stop_token_ids=sorted(tokenizer.eos_token_ids))
        self.compiler = xgr.GrammarCompiler(self.info)
        self.words = (vocab_size + 31) // 32

    def compile(self, spec: dict) -> GrammarState:
        t = spec["type"]
        if t == "json_object":
            cg = self.compiler.compile_builtin_json_grammar()
        elif t == "json_schema":
            cg = self.compiler.compile_json_schema(spec["schema"], any_whitespace=not spec.get("compact", False))
        elif t == "regex":
            cg = self.compiler.compile_regex(spec["pattern"])
        elif t == "ebnf":
            cg = self.compiler.compile_grammar(spec["pattern"])
        else:
            raise ValueError(f"unknown grammar type {t!r}")
        return GrammarState(self.xgr.GrammarMatcher(cg))

    def bitmask_for(self, states: Sequence[Optional[GrammarState]]) -> torch.Tensor:
        """int32 [len(states), words]; rows without a grammar allow everything."""
        bm = torch.full((len(states), self.words), -1, dtype=torch.int32)
        for i, st in enumerate(states):
            if st is not None:
                st.fill(bm, i)
        return bm


def apply_token_bitmask_reference(logits: torch.Tensor, bitmask: torch.Tensor) -> None:
    """In place: logits[r, v] = -inf where bit v of bitmask[r] is clear."""
    V = logits.shape[1]
    bits = torch.from_numpy(np.unpackbits(bitmask.cpu().numpy().view(np.uint8), axis=1, bitorder="little")[:, :V])
    logits.masked_fill_(~bits.bool().to(logits.device), float("-inf"))
