"""OpenAI-compatible routes: /v1/completions, /v1/chat/completions, /v1/models, health.

Reference: max/python/max/serve/router/openai_routes.py (``openai_create_chat_completion``
:1873, ``OpenAIChatResponseGenerator`` :434 with ``_stream`` :592 / ``complete`` :998,
``openai_create_completion`` :2972, ``/v1/models`` :3165). Streaming uses server-sent events
terminated by ``data: [DONE]``; usage accounting, finish reasons and the OpenAI error envelope
follow the public API.
"""

from __future__ import annotations

import json
import logging
import uuid
from typing import AsyncIterator, Optional, Union

from fastapi import APIRouter, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse

from ...pipelines.context import SamplingParams
import asyncio
import hashlib

from ..parser import ReasoningSplitter, get_tool_parser, split_reasoning
from ..parser.conformance import check_response_format, check_tool_calls, tool_schemas
from ..parser.normalization import anchor_object_schemas, tool_call_arguments_as_mappings, tools_with_parameters
from ..schemas.openai import (ChatChoice, ChatChoiceMessage, ChatChunkChoice, ChatCompletionChunk,
                              ChatCompletionRequest, ChatCompletionResponse, ChatDelta, CompletionChoice,
                              CompletionRequest, CompletionResponse, ErrorBody, ErrorResponse, ModelCard,
                              ModelList, Usage, EmbeddingData, EmbeddingsRequest, EmbeddingsResponse,
                              LoadLoraRequest, UnloadLoraRequest)
from ..telemetry.metrics import METRICS
from ..worker_interface import RequestQueueFull, WorkerGone

logger = logging.getLogger("modular_b200.serve")

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
        if spec is not None and spec.get("type") == "json_schema":
            # untyped nodes with object keywords would let the grammar accept a bare, never-ending string
            try:
                spec = dict(spec, schema=json.dumps(anchor_object_schemas(json.loads(spec["schema"]))))
            except (TypeError, ValueError):
                pass
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
            stop_token_ids=req.stop_token_ids, seed=req.seed or 0, logprobs=_logprobs_requested(req),
            logit_bias=getattr(req, "logit_bias", None))
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


def _check_model(request: Request, name: str) -> Optional[str]:
    """Validates the ``model`` field; returns the LoRA adapter it names (requests address an adapter by using its
    name as the model, reference: openai_routes.py LoRA handling) or None for the base model."""
    served = request.app.state.model_names
    if name in served:
        return None
    if name in getattr(request.app.state, "lora_names", ()):
        return name
    raise HTTPException(status_code=404, detail=f"model {name!r} is not served here (available: "
                                                f"{sorted(served | set(getattr(request.app.state, 'lora_names', ())))})")


def _salt_of(req) -> int:
    s = getattr(req, "cache_salt", None)
    if not s:
        return 0
    return int.from_bytes(hashlib.blake2b(str(s).encode(), digest_size=8).digest(), "little") & 0x7FFFFFFFFFFFFFFF


def _with_seed(sp: SamplingParams, i: int) -> SamplingParams:
    """The i-th of ``n`` samples of one request: same parameters, its own seed."""
    if i == 0:
        return sp
    import dataclasses
    return dataclasses.replace(sp, seed=(sp.seed or 0) + i)


async def _merge_streams(gens: list):
    """Yields (index, item) from several async generators as items arrive."""
    q: asyncio.Queue = asyncio.Queue()
    done = object()

    async def pump(i, g):
        try:
            async for item in g:
                await q.put((i, item))
        except Exception as e:  # noqa: BLE001
            await q.put((i, e))
        finally:
            await q.put((i, done))

    tasks = [asyncio.ensure_future(pump(i, g)) for i, g in enumerate(gens)]
    left = len(tasks)
    try:
        while left:
            i, item = await q.get()
            if item is done:
                left -= 1
            elif isinstance(item, Exception):
                raise item
            else:
                yield i, item
    finally:
        for t in tasks:
            t.cancel()


def _sse(obj) -> bytes:
    if isinstance(obj, str):
        return f"data: {obj}\n\n".encode()
    return f"data: {obj.model_dump_json(exclude_none=True)}\n\n".encode()


# ------------------------------------------------------------------ models / health
@router.get("/v1/models")
async def list_models(request: Request) -> ModelList:
    names = set(request.app.state.model_names) | set(getattr(request.app.state, "lora_names", ()))
    return ModelList(data=[ModelCard(id=n) for n in sorted(names)])


@router.get("/v1/models/{model_id:path}")
async def get_model(model_id: str, request: Request):
    if model_id not in request.app.state.model_names and model_id not in getattr(request.app.state, "lora_names", ()):
        return error_response(404, f"model {model_id!r} not found", "not_found_error")
    return ModelCard(id=model_id)


# ------------------------------------------------------------------ LoRA administration
@router.post("/v1/load_lora_adapter")
async def load_lora_adapter(req: LoadLoraRequest, request: Request):
    """Loads a PEFT-layout adapter directory (or .safetensors file) into the model worker; requests then select it
    with ``model = lora_name``. Reference: max/python/max/serve/router/openai_routes.py:3217."""
    rpc = getattr(request.app.state, "rpc", None)
    if rpc is None:
        return error_response(503, "model worker is not ready", "service_unavailable")
    if req.lora_name in request.app.state.model_names:
        return error_response(400, f"{req.lora_name!r} is the name of the base model")
    try:
        await rpc.call("load_lora", {"name": req.lora_name, "path": req.lora_path, "alpha": req.alpha}, timeout_s=120.0)
    except (RuntimeError, TimeoutError) as e:
        return error_response(400, f"could not load adapter {req.lora_name!r}: {e}")
    request.app.state.lora_names = set(getattr(request.app.state, "lora_names", ())) | {req.lora_name}
    return {"status": "success", "message": f"LoRA adapter {req.lora_name!r} loaded"}


@router.post("/v1/unload_lora_adapter")
async def unload_lora_adapter(req: UnloadLoraRequest, request: Request):
    """Reference: max/python/max/serve/router/openai_routes.py:3295."""
    rpc = getattr(request.app.state, "rpc", None)
    if rpc is None:
        return error_response(503, "model worker is not ready", "service_unavailable")
    if req.lora_name not in getattr(request.app.state, "lora_names", ()):
        return error_response(404, f"LoRA adapter {req.lora_name!r} is not loaded", "not_found_error")
    try:
        await rpc.call("unload_lora", {"name": req.lora_name}, timeout_s=30.0)
    except (RuntimeError, TimeoutError) as e:
        return error_response(400, f"could not unload adapter {req.lora_name!r}: {e}")
    request.app.state.lora_names = set(request.app.state.lora_names) - {req.lora_name}
    return {"status": "success", "message": f"LoRA adapter {req.lora_name!r} unloaded"}


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
    lora = _check_model(request, req.model)
    if req.n < 1 or req.n > 16:
        return error_response(400, "n must be between 1 and 16")
    prompts = _prompts_of(req)
    sp = sampling_from_request(req, None)
    salt = _salt_of(req)
    rid = getattr(request.state, "request_id", uuid.uuid4().hex)
    cid = f"cmpl-{rid}"
    try:
        if req.stream:
            if len(prompts) != 1:
                return error_response(400, "streaming supports a single prompt")

            async def gen() -> AsyncIterator[bytes]:
                usages = [Usage() for _ in range(req.n)]
                try:
                    streams = [pipeline.next_token_chunk(prompts[0], _with_seed(sp, i), f"{rid}-{i}" if req.n > 1 else rid,
                                                         lora, salt) for i in range(req.n)]
                    async for i, ch in _merge_streams(streams):
                        usages[i] = Usage(prompt_tokens=ch.prompt_tokens, completion_tokens=ch.completion_tokens)
                        yield _sse(CompletionResponse(id=cid, model=req.model, choices=[
                            CompletionChoice(index=i, text=ch.text, finish_reason=ch.finish_reason)]))
                    if req.stream_options and req.stream_options.include_usage:
                        u = Usage(prompt_tokens=usages[0].prompt_tokens,
                                  completion_tokens=sum(x.completion_tokens for x in usages))
                        u.total_tokens = u.prompt_tokens + u.completion_tokens
                        yield _sse(CompletionResponse(id=cid, model=req.model, choices=[], usage=u))
                except Exception as e:  # noqa: BLE001
                    METRICS.request_errors.inc()
                    yield _sse(json.dumps(ErrorResponse(error=ErrorBody(message=str(e), type="server_error")).model_dump()))
                yield _sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        jobs = [(pi, si) for pi in range(len(prompts)) for si in range(req.n)]
        results = await asyncio.gather(*[
            pipeline.all_tokens(prompts[pi], _with_seed(sp, si), f"{rid}-{pi}-{si}", lora, salt) for pi, si in jobs])
        choices, usage = [], Usage()
        for k, ((pi, si), ch) in enumerate(zip(jobs, results)):
            text = ch.text
            if req.echo and isinstance(prompts[pi], str):
                text = prompts[pi] + text
            choices.append(CompletionChoice(index=k, text=text, finish_reason=ch.finish_reason,
                                            logprobs=_completion_logprobs(pipeline, ch)))
            if si == 0:
                usage.prompt_tokens += ch.prompt_tokens
            usage.completion_tokens += ch.completion_tokens
        usage.total_tokens = usage.prompt_tokens + usage.completion_tokens
        return CompletionResponse(id=cid, model=req.model, choices=choices, usage=usage)
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except WorkerGone as e:
        return error_response(503, str(e), "service_unavailable")
    except ValueError as e:
        return error_response(400, str(e))


# ------------------------------------------------------------------ chat completions
def _chat_prompt(pipeline, req: ChatCompletionRequest) -> str:
    msgs = [m.model_dump(exclude_none=True) for m in req.messages]
    if not msgs:
        raise HTTPException(status_code=400, detail="messages must not be empty")
    for m in msgs:      # templates walk the arguments of earlier tool calls as mappings; clients send JSON strings
        if m.get("tool_calls"):
            m["tool_calls"] = tool_call_arguments_as_mappings(m["tool_calls"])
    tools = tools_with_parameters(req.tools) if req.tools else req.tools
    return pipeline.tokenizer.apply_chat_template(msgs, tools=tools, add_generation_prompt=True)


def _tool_parser_for(request: Request, req: ChatCompletionRequest):
    """A fresh tool-call parser when the request offers tools and does not forbid their use."""
    if not req.tools or req.tool_choice == "none":
        return None
    return get_tool_parser(getattr(request.app.state, "tool_parser", None) or "llama")


def _observe_conformance(req, tool_calls=None, content=None) -> None:
    """Counts and logs (names and JSON paths only, no values) tool calls and JSON answers that do not match what the
    request declared. Never changes the response and never raises."""
    try:
        if tool_calls:
            schemas, names = tool_schemas(req.tools)
            for r in check_tool_calls([(c["function"]["name"], c["function"].get("arguments", "")) for c in tool_calls],
                                      schemas, names):
                if r.outcome != "valid":
                    METRICS.tool_call_nonconforming.inc()
                    logger.info("tool call %s: %s %s (+%d)", r.function, r.outcome, r.errors, r.more_errors)
        rf = getattr(req, "response_format", None)
        if content is not None and rf is not None and rf.type in ("json_schema", "json_object"):
            js = getattr(rf, "json_schema", None) or {}
            schema = (js.get("schema", js) if isinstance(js, dict) else {}) if rf.type == "json_schema" else {"type": "object"}
            r = check_response_format(content, schema if isinstance(schema, dict) else {})
            if r.outcome != "valid":
                METRICS.response_format_nonconforming.inc()
                logger.info("response_format: %s %s (+%d)", r.outcome, r.errors, r.more_errors)
    except Exception:      # noqa: BLE001 - observation must not fail a request
        pass


def _finish_message(text: str, parser, reasoning_on: bool, req=None):
    """(message, finish_reason override) of a complete answer."""
    reasoning = None
    if reasoning_on:
        reasoning, text = split_reasoning(text)
    if parser is not None:
        try:
            parsed = parser.parse_complete(text)
        except ValueError:
            parsed = None
        if parsed is not None and parsed.tool_calls:
            calls = [c.to_openai() for c in parsed.tool_calls]
            if req is not None:
                _observe_conformance(req, tool_calls=calls)
            return ChatChoiceMessage(content=parsed.content, reasoning_content=reasoning, tool_calls=calls), "tool_calls"
    if req is not None:
        _observe_conformance(req, content=text)
    return ChatChoiceMessage(content=text, reasoning_content=reasoning), None


@router.post("/v1/chat/completions")
async def create_chat_completion(req: ChatCompletionRequest, request: Request):
    pipeline = _pipeline(request)
    lora = _check_model(request, req.model)
    if req.n < 1 or req.n > 16:
        return error_response(400, "n must be between 1 and 16")
    if req.response_format is not None and req.response_format.type != "text":
        if not request.app.state.structured_output:
            return error_response(400, "response_format requires the server to run with --enable-structured-output")
    for m in req.messages:
        # content parts other than text (images, audio, video, files) would otherwise vanish from the prompt
        for part in (m.content if isinstance(m.content, list) else ()):
            kind = part.get("type", "text") if isinstance(part, dict) else "text"
            if kind != "text":
                return error_response(400, f"content parts of type {kind!r} are not supported: this server takes text")
    sp = sampling_from_request(req, None)
    salt = _salt_of(req)
    prompt = _chat_prompt(pipeline, req)
    reasoning_on = bool(getattr(request.app.state, "reasoning_parser", None))
    try:
        _tool_parser_for(request, req)
    except ValueError as e:
        return error_response(400, str(e))
    rid = getattr(request.state, "request_id", uuid.uuid4().hex)
    cid = f"chatcmpl-{rid}"
    try:
        if req.stream:
            async def gen() -> AsyncIterator[bytes]:
                n = req.n
                usages = [Usage() for _ in range(n)]
                parsers = [_tool_parser_for(request, req) for _ in range(n)]
                splitters = [ReasoningSplitter() if reasoning_on else None for _ in range(n)]
                n_calls = [0] * n
                for i in range(n):
                    yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[
                        ChatChunkChoice(index=i, delta=ChatDelta(role="assistant", content=""))]))
                try:
                    streams = [pipeline.next_token_chunk(prompt, _with_seed(sp, i), f"{rid}-{i}" if n > 1 else rid, lora, salt)
                               for i in range(n)]
                    async for i, ch in _merge_streams(streams):
                        usages[i] = Usage(prompt_tokens=ch.prompt_tokens, completion_tokens=ch.completion_tokens)
                        final = ch.finish_reason is not None
                        text, reasoning = ch.text, ""
                        if splitters[i] is not None:
                            reasoning, text = splitters[i].push(text, final)
                        calls = []
                        if parsers[i] is not None:
                            text, calls = parsers[i].parse_delta(text, final)
                        if reasoning:
                            yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[ChatChunkChoice(
                                index=i, delta=ChatDelta(reasoning_content=reasoning))]))
                        for c in calls:
                            yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[ChatChunkChoice(
                                index=i, delta=ChatDelta(tool_calls=[c.to_openai(index=n_calls[i])]))]))
                            n_calls[i] += 1
                        reason = ch.finish_reason
                        if final and n_calls[i] and reason == "stop":
                            reason = "tool_calls"
                        if text or reason:
                            yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[ChatChunkChoice(
                                index=i, delta=ChatDelta(content=text or None), finish_reason=reason)]))
                    if req.stream_options and req.stream_options.include_usage:
                        u = Usage(prompt_tokens=usages[0].prompt_tokens,
                                  completion_tokens=sum(x.completion_tokens for x in usages))
                        u.total_tokens = u.prompt_tokens + u.completion_tokens
                        yield _sse(ChatCompletionChunk(id=cid, model=req.model, choices=[], usage=u))
                except Exception as e:  # noqa: BLE001
                    METRICS.request_errors.inc()
                    yield _sse(json.dumps(ErrorResponse(error=ErrorBody(message=str(e), type="server_error")).model_dump()))
                yield _sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        results = await asyncio.gather(*[
            pipeline.all_tokens(prompt, _with_seed(sp, i), f"{rid}-{i}" if req.n > 1 else rid, lora, salt)
            for i in range(req.n)])
        usage = Usage(prompt_tokens=results[0].prompt_tokens,
                      completion_tokens=sum(r.completion_tokens for r in results))
        usage.total_tokens = usage.prompt_tokens + usage.completion_tokens
        choices = []
        for i, ch in enumerate(results):
            msg, reason = _finish_message(ch.text, _tool_parser_for(request, req), reasoning_on, req)
            choices.append(ChatChoice(index=i, message=msg, logprobs=_chat_logprobs(pipeline, ch),
                                      finish_reason=reason if (reason and ch.finish_reason == "stop") else ch.finish_reason))
        return ChatCompletionResponse(id=cid, model=req.model, usage=usage, choices=choices)
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except WorkerGone as e:
        return error_response(503, str(e), "service_unavailable")
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
            vec, n = await pipeline.embed(item, req.pooling or "default", f"{rid}-{i}")
            if req.dimensions:
                vec = vec[: req.dimensions]
                norm = sum(v * v for v in vec) ** 0.5 or 1.0
                vec = [v / norm for v in vec]
            n_tok += n
            emb = vec if req.encoding_format == "float" else base64.b64encode(struct.pack(f"<{len(vec)}f", *vec)).decode()
            data.append(EmbeddingData(index=i, embedding=emb))
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except WorkerGone as e:
        return error_response(503, str(e), "service_unavailable")
    except ValueError as e:
        return error_response(400, str(e))
    return EmbeddingsResponse(data=data, model=req.model, usage=Usage(prompt_tokens=n_tok, total_tokens=n_tok))
