"""API-side token generator: tokenise, submit to the worker, stream detokenised chunks.

Reference: max/python/max/serve/pipelines/llm.py:234 ``TokenGeneratorPipeline``
(``next_token_chunk`` :279, ``_coalesce_chunks`` :178): TTFT / ITL / TPOT are recorded here,
chunks are coalesced up to ``stream_min_chunk_tokens``, stop strings end the stream and cancel
the request on the worker.
"""

from __future__ import annotations

import time
import uuid
from dataclasses import dataclass, field
from typing import AsyncIterator, Optional, Sequence, Union

from ...pipelines.context import GenerationStatus, SamplingParams
from ..telemetry import tracing
from ..telemetry.metrics import METRICS
from ..worker_interface import ModelWorkerProxy
from .incremental_detokenizer import IncrementalDetokenizer


@dataclass
class TokenChunk:
    text: str
    token_ids: list
    finish_reason: Optional[str] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    logprobs: Optional[list] = None     # entries {"token", "logprob", "top"} aligned with token_ids


def finish_reason_of(status: GenerationStatus, stopped_on_string: bool = False) -> Optional[str]:
    if stopped_on_string or status is GenerationStatus.END_OF_SEQUENCE:
        return "stop"
    if status is GenerationStatus.MAXIMUM_LENGTH:
        return "length"
    if status is GenerationStatus.CANCELLED:
        return "cancelled"
    return None


class TokenGeneratorPipeline:
    def __init__(self, model_name: str, tokenizer, proxy: ModelWorkerProxy, max_length: int,
                 stream_min_chunk_tokens: int = 1):
        self.model_name = model_name
        self.tokenizer = tokenizer
        self.proxy = proxy
        self.max_length = max_length
        self.min_chunk = max(1, stream_min_chunk_tokens)

    async def next_token_chunk(self, prompt: Union[str, Sequence[int]], sampling_params: SamplingParams,
                               request_id: Optional[str] = None, lora_name: Optional[str] = None,
                               cache_salt: int = 0) -> AsyncIterator[TokenChunk]:
        rid = request_id or uuid.uuid4().hex
        t_in = time.perf_counter()
        with tracing.span("max.tokenize", {"request.id": rid}):
            ctx = self.tokenizer.new_context(prompt, self.max_length, sampling_params, rid, self.model_name)
        ctx.lora_name = lora_name
        ctx.cache_salt = cache_salt
        n_prompt = ctx.tokens.prompt_len
        METRICS.input_processing_ms.observe((time.perf_counter() - t_in) * 1e3)
        METRICS.input_tokens_per_request.observe(n_prompt)
        if isinstance(prompt, str):
            METRICS.input_characters.inc(len(prompt))
        detok = IncrementalDetokenizer(self.tokenizer, sampling_params.stop) if sampling_params.detokenize else None
        t_start = time.perf_counter()
        t_last: Optional[float] = None
        n_out = 0
        METRICS.request_count.inc()
        METRICS.input_tokens.inc(n_prompt)
        buf_ids: list = []
        buf_lps: list = []
        buf_text = ""
        async for out in self.proxy.stream(ctx):
            if out.final_status is GenerationStatus.ERROR:
                METRICS.request_errors.inc()
                if getattr(self.proxy, "dead", None):
                    from ..worker_interface.interface import WorkerGone

                    raise WorkerGone(self.proxy.dead)
                raise ValueError(getattr(out, "error", None) or "the request could not be served")
            now = time.perf_counter()
            if out.tokens:
                if t_last is None:
                    METRICS.ttft_ms.observe((now - t_start) * 1e3)
                else:
                    METRICS.itl_ms.observe((now - t_last) * 1e3 / len(out.tokens))
                t_last = now
                n_out += len(out.tokens)
            text = detok.push(out.tokens, final=out.is_done) if detok is not None else ""
            METRICS.output_processing_ms.observe((time.perf_counter() - now) * 1e3)
            stopped = detok is not None and detok.stopped
            buf_ids.extend(out.tokens)
            if getattr(out, "log_probabilities", None):
                buf_lps.extend(out.log_probabilities)
            buf_text += text
            done = out.is_done or stopped
            if done or len(buf_ids) >= self.min_chunk:
                reason = finish_reason_of(out.final_status, stopped) if done else None
                yield TokenChunk(buf_text, buf_ids, reason, n_prompt, n_out, buf_lps or None)
                buf_ids, buf_lps, buf_text = [], [], ""
            if done:
                break
        if tracing.tracing_enabled():
            # the generation as one finished span (the stream yields in between, so it is not a `with` block)
            with tracing.span("max.generate", {"request.id": rid, "gen.prompt_tokens": n_prompt,
                                               "gen.output_tokens": n_out,
                                               "gen.duration_ms": (time.perf_counter() - t_start) * 1e3}):
                pass
        METRICS.output_tokens.inc(n_out)
        METRICS.output_tokens_per_request.observe(n_out)
        if n_out > 1 and t_last is not None:
            METRICS.tpot_ms.observe((t_last - t_start) * 1e3 / n_out)
        METRICS.request_time_ms.observe((time.perf_counter() - t_start) * 1e3)

    async def all_tokens(self, prompt, sampling_params: SamplingParams, request_id: Optional[str] = None,
                         lora_name: Optional[str] = None, cache_salt: int = 0) -> TokenChunk:
        text, ids, reason, n_prompt, n_out, lps = "", [], None, 0, 0, []
        async for ch in self.next_token_chunk(prompt, sampling_params, request_id, lora_name, cache_salt):
            text += ch.text
            ids.extend(ch.token_ids)
            lps.extend(ch.logprobs or [])
            reason = ch.finish_reason or reason
            n_prompt, n_out = ch.prompt_tokens, ch.completion_tokens
        return TokenChunk(text, ids, reason, n_prompt, n_out, lps or None)

    async def embed(self, prompt: Union[str, Sequence[int]], pooling: str = "default",
                    request_id: Optional[str] = None):
        """One pooled embedding; returns (vector, prompt_tokens)."""
        rid = request_id or uuid.uuid4().hex
        ctx = self.tokenizer.new_context(prompt, self.max_length, SamplingParams(max_new_tokens=1), rid, self.model_name)
        ctx.task, ctx.pooling = "embed", pooling
        METRICS.request_count.inc()
        METRICS.input_tokens.inc(ctx.tokens.prompt_len)
        async for out in self.proxy.stream(ctx):
            if hasattr(out, "embedding"):
                return out.embedding, out.prompt_tokens
            raise ValueError("this model worker cannot produce embeddings")
        raise RuntimeError("embeddings request ended without an answer")
