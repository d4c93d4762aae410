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


class GrammarGate:
    """Compiles the grammars of new requests on worker threads while the scheduler keeps serving.

    Building a matcher for a large schema can take seconds; done inline it would stall every request that shares
    the step loop. The scheduler hands a constrained request to :meth:`submit` and admits it to prefill only once
    :meth:`ready`; :meth:`install` then puts the matcher on the context or returns the message for the client when
    the grammar does not compile (the request fails, the server goes on). All methods are called from the
    scheduler thread; only the compilation runs elsewhere (the grammar backend releases the GIL while it works).

    Reference: max/python/max/serve/scheduler/batch_constructor/grammar_gate.py:41 (AsyncGrammarGate).
    """

    def __init__(self, backend, workers: Optional[int] = None):
        import os

        self.backend = backend
        self.workers = workers or max(1, (os.cpu_count() or 2) // 2)
        self._pool = None
        self._jobs: dict = {}

    def submit(self, ctx) -> bool:
        """Starts the compilation for ``ctx`` if it needs one and none runs yet. True when the request now waits."""
        spec = ctx.sampling_params.response_format
        if spec is None or ctx.grammar_state is not None:
            return False
        if ctx.request_id not in self._jobs:
            if self._pool is None:
                from concurrent.futures import ThreadPoolExecutor

                self._pool = ThreadPoolExecutor(max_workers=self.workers, thread_name_prefix="grammar-compile")
            self._jobs[ctx.request_id] = self._pool.submit(self.backend.compile, spec)
        return True

    def ready(self, ctx) -> bool:
        job = self._jobs.get(ctx.request_id)
        return job is None or job.done()

    def install(self, ctx) -> Optional[str]:
        """After :meth:`ready`: the matcher goes onto the context (None), or the reason it could not be built."""
        job = self._jobs.pop(ctx.request_id, None)
        if job is None:
            return None
        try:
            ctx.grammar_state = job.result()
        except Exception as e:      # noqa: BLE001 - whatever the backend raises is the client's answer
            import re

            last = str(e).strip().splitlines()[-1] if str(e).strip() else type(e).__name__
            last = re.sub(r"^\[[^\]]*\]\s*\S+:\d+:\s*", "", last)      # "[time] file.cc:123: " of native backends
            return f"the grammar of this request cannot be compiled: {last}"
        for t in ctx.tokens.generated:      # tokens from before a preemption are replayed into the fresh matcher
            if t >= 0:
                ctx.grammar_state.accept(int(t))
        return None

    def release(self, request_id: str) -> None:
        job = self._jobs.pop(request_id, None)
        if job is not None:
            job.cancel()

    def shutdown(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=False, cancel_futures=True)
            self._pool = None
