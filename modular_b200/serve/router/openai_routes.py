"""OpenAI-compatible routes: /v1/completions, /v1/chat/completions, /v1/models, health.

Reference: max/python/max/serve/router/openai_routes.py (``openai_create_chat_completion``
:1873, ``OpenAIChatResponseGenerator`` :434 with ``_stream`` :592 / ``complete`` :998,
``openai_create_completion`` :2972, ``/v1/models`` :3165). Streaming uses server-sent events
terminated by ``data: [DONE]``; usage accounting, finish reasons and the OpenAI error envelope
follow the public API.
"""

from __future__ import annotations

import json
import uuid
from typing import AsyncIterator, Optional, Union

from fastapi import APIRouter, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse

from ...pipelines.context import SamplingParams
from ..schemas.openai import (ChatChoice, ChatChoiceMessage, ChatChunkChoice, ChatCompletionChunk,
                              ChatCompletionRequest, ChatCompletionResponse, ChatDelta, CompletionChoice,
                              CompletionRequest, CompletionResponse, ErrorBody, ErrorResponse, ModelCard,
                              ModelList, Usage, EmbeddingData, EmbeddingsRequest, EmbeddingsResponse)
from ..telemetry.metrics import METRICS
from ..worker_interface import RequestQueueFull

router = APIRouter()


def error_response(status: int, message: str, err_type: str = "invalid_request_error", code=None) -> JSONResponse:
    body = ErrorResponse(error=ErrorBody(message=message, type=err_type, code=code or status))
    return JSONResponse(status_code=status, content=body.model_dump())


def sampling_from_request(req, default_max_tokens: Optional[int]) -> SamplingParams:
    stop = [req.stop] if isinstance(req.stop, str) else req.stop
    max_tokens = req.max_tokens
    if max_tokens is None and getattr(req, "max_completion_tokens", None) is not None:
        max_tokens = req.max_completion_tokens
    from ...pipelines.structured_output import response_format_to_spec
    try:
        spec = response_format_to_spec(getattr(req, "response_format", None))
        return SamplingParams(
            response_format=spec,
            top_k=req.top_k if req.top_k not in (None, 0) else -1,
            top_p=req.top_p if req.top_p is not None else 1.0,
            min_p=req.min_p or 0.0,
            temperature=req.temperature if req.temperature is not None else 1.0,
            frequency_penalty=req.frequency_penalty or 0.0,
            presence_penalty=req.presence_penalty or 0.0,
            repetition_penalty=req.repetition_penalty or 1.0,
            max_new_tokens=max_tokens if max_tokens is not None else default_max_tokens,
            min_new_tokens=req.min_tokens or 0, ignore_eos=req.ignore_eos, stop=stop,
            stop_token_ids=req.stop_token_ids, seed=req.seed or 0, logprobs=_logprobs_requested(req))
    except ValueError as e:
        raise HTTPException(status_code=400, detail=str(e)) from e


def _logprobs_requested(req) -> int:
    """Number of alternatives per token (0 = off). Completions: ``logprobs: N``; chat: ``logprobs: true`` +
    ``top_logprobs: N``."""
    lp = getattr(req, "logprobs", None)
    if lp is None or lp is False:
        return 0
    if lp is True:
        return max(1, int(getattr(req, "top_logprobs", None) or 1))
    return max(1, int(lp))


def _completion_logprobs(pipeline, ch) -> Optional[dict]:
    if not ch.logprobs:
        return None
    dec = lambda t: pipeline.tokenizer.decode([t])
    return {"tokens": [dec(e["token"]) for e in ch.logprobs],
            "token_logprobs": [e["logprob"] for e in ch.logprobs],
            "top_logprobs": [{dec(t): lp for t, lp in e["top"]} for e in ch.logprobs]}


def _chat_logprobs(pipeline, ch) -> Optional[dict]:
    if not ch.logprobs:
        return None
    dec = lambda t: pipeline.tokenizer.decode([t])
    return {"content": [{"token": dec(e["token"]), "logprob": e["logprob"],
                         "top_logprobs": [{"token": dec(t), "logprob": lp} for t, lp in e["top"]]}
                        for e in ch.logprobs]}


def _pipeline(request: Request):
    p = getattr(request.app.state, "pipeline", None)
    if p is None:
        raise HTTPException(status_code=503, detail="model worker is not ready")
    return p


def _check_model(request: Request, name: str) -> None:
    served = request.app.state.model_names
    if name not in served:
        raise HTTPException(status_code=404, detail=f"model {name!r} is not served here (available: {sorted(served)})")


def _sse(obj) -> bytes:
    if isinstance(obj, str):
        return f"data: {obj}\n\n".encode()
    return f"data: {obj.model_dump_json(exclude_none=True)}\n\n".encode()


# ------------------------------------------------------------------ models / health
@router.get("/v1/models")
async def list_models(request: Request) -> ModelList:
    return ModelList(data=[ModelCard(id=n) for n in sorted(request.app.state.model_names)])


@router.get("/v1/models/{model_id:path}")
async def get_model(model_id: str, request: Request):
    if model_id not in request.app.state.model_names:
        return error_response(404, f"model {model_id!r} not found", "not_found_error")
    return ModelCard(id=model_id)


@router.get("/v1/health")
async def v1_health() -> dict:
    return {"status": "ok"}


# ------------------------------------------------------------------ completions
def _prompts_of(req: CompletionRequest) -> list:
    p = req.prompt
    if isinstance(p, str):
        return [p]
    if isinstance(p, list) and p and isinstance(p[0], int):
        return [p]
    if isinstance(p, list) and p:
        return list(p)
    raise HTTPException(status_code=400, detail="prompt must be a non-empty string, token list, or list of those")


@router.post("/v1/completions")
async def create_completion(req: CompletionRequest, request: Request):
    pipeline = _pipeline(request)
    _check_model(request, req.model)
    if req.n != 1:
        return error_response(400, "n > 1 is not supported")
    prompts = _prompts_of(req)
    sp = sampling_from_request(req, None)
    rid = getattr(request.state, "request_id", uuid.uuid4().hex)
    cid = f"cmpl-{rid}"
    try:
        if req.stream:
            if len(prompts) != 1:
                return error_response(400, "streaming supports a single prompt")

            async def gen() -> AsyncIterator[bytes]:
                usage = Usage()
                try:
                    async for ch in pipeline.next_token_chunk(prompts[0], sp, rid):
                        usage = Usage(prompt_tokens=ch.prompt_tokens, completion_tokens=ch.completion_tokens,
                                      total_tokens=ch.prompt_tokens + ch.completion_tokens)
                        yield _sse(CompletionResponse(id=cid, model=req.model, choices=[
                            CompletionChoice(text=ch.text, finish_reason=ch.finish_reason)]))
                    if req.stream_options and req.stream_options.include_usage:
                        yield _sse(CompletionResponse(id=cid, model=req.model, choices=[], usage=usage))
                except Exception as e:  # noqa: BLE001
                    METRICS.request_errors.inc()
                    yield _sse(json.dumps(ErrorResponse(error=ErrorBody(message=str(e), type="server_error")).model_dump()))
                yield _sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        choices, usage = [], Usage()
        for i, p in enumerate(prompts):
            ch = await pipeline.all_tokens(p, sp, f"{rid}-{i}")
            text = ch.text
            if req.echo and isinstance(p, str):
                text = p + text
            choices.append(CompletionChoice(index=i, text=text, finish_reason=ch.finish_reason,
                                            logprobs=_completion_logprobs(pipeline, ch)))
            usage.prompt_tokens += ch.prompt_tokens
            usage.completion_tokens += ch.completion_tokens
        usage.total_tokens = usage.prompt_tokens + usage.completion_tokens
        return CompletionResponse(id=cid, model=req.model, choices=choices, usage=usage)
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except ValueError as e:
        return error_response(400, str(e))


# ------------------------------------------------------------------ chat completions
def _chat_prompt(pipeline, req: ChatCompletionRequest) -> str:
    msgs = [m.model_dump(exclude_none=True) for m in req.messages]
    if not msgs:
        raise HTTPException(status_code=400, detail="messages must not be empty")
    return pipeline.tokenizer.apply_chat_template(msgs, tools=req.tools, add_generation_prompt=True)


@router.post("/v1/chat/completions")
async def create_chat_completion(req: ChatCompletionRequest, request: Request):
    pipeline = _pipeline(request)
    _check_model(request, req.model)
    if req.n != 1:
        return error_response(400, "n > 1 is not supported")
    if req.response_format is not None and req.response_format.type != "text":
        if not request.app.state.structured_output:
            return error_response(400, "response_format requires the server to run with --enable-structured-output")
    sp = sampling_from_request(req, None)
    prompt = _chat_prompt(pipeline, req)
    rid = getattr(request.state, "request_id", uuid.uuid4().hex)
    cid = f"chatcmpl-{rid}"
    try:
        if req.stream:
            async def gen() -> AsyncIterator[bytes]:
                usage = Usage()
                yield _sse(ChatCompletionChunk(id=cid, model=req.model,
                                               choices=[ChatChunkChoice(delta=ChatDelta(role="assistant", content=""))]))
                try:
                    async for ch in pipeline.next_token_chunk(prompt, sp, rid):
                        usage = Usage(prompt_tokens=ch.prompt_tokens, completion_tokens=ch.completion_tokens,
                                      total_tokens=ch.prompt_tokens + ch.completion_tokens)
                        if ch.text or ch.finish_reason:
                            yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[ChatChunkChoice(
                                delta=ChatDelta(content=ch.text or None), finish_reason=ch.finish_reason)]))
                    if req.stream_options and req.stream_options.include_usage:
                        yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[], usage=usage))
                except Exception as e:  # noqa: BLE001
                    METRICS.request_errors.inc()
                    yield _sse(json.dumps(ErrorResponse(error=ErrorBody(message=str(e), type="server_error")).model_dump()))
                yield _sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        ch = await pipeline.all_tokens(prompt, sp, rid)
        usage = Usage(prompt_tokens=ch.prompt_tokens, completion_tokens=ch.completion_tokens,
                      total_tokens=ch.prompt_tokens + ch.completion_tokens)
        return ChatCompletionResponse(id=cid, model=req.model, usage=usage, choices=[
            ChatChoice(message=ChatChoiceMessage(content=ch.text), finish_reason=ch.finish_reason,
                       logprobs=_chat_logprobs(pipeline, ch))])
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except ValueError as e:
        return error_response(400, str(e))


# ------------------------------------------------------------------ embeddings
@router.post("/v1/embeddings")
async def create_embeddings(req: EmbeddingsRequest, request: Request):
    import base64
    import struct

    pipeline = _pipeline(request)
    _check_model(request, req.model)
    inp = req.input
    if isinstance(inp, str) or (isinstance(inp, list) and inp and isinstance(inp[0], int)):
        inputs = [inp]
    else:
        inputs = list(inp)
    if not inputs:
        return error_response(400, "input must not be empty")
    if req.encoding_format not in ("float", "base64"):
        return error_response(400, "encoding_format must be float or base64")
    rid = getattr(request.state, "request_id", uuid.uuid4().hex)
    data, n_tok = [], 0
    try:
        for i, item in enumerate(inputs):
            vec, n = await pipeline.embed(item, req.pooling or "last", f"{rid}-{i}")
            if req.dimensions:
                vec = vec[: req.dimensions]
                norm = sum(v * v for v in vec) ** 0.5 or 1.0
                vec = [v / norm for v in vec]
            n_tok += n
            emb = vec if req.encoding_format == "float" else base64.b64encode(struct.pack(f"<{len(vec)}f", *vec)).decode()
            data.append(EmbeddingData(index=i, embedding=emb))
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except ValueError as e:
        return error_response(400, str(e))
    return EmbeddingsResponse(data=data, model=req.model, usage=Usage(prompt_tokens=n_tok, total_tokens=n_tok))
