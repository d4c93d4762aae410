"""KServe v2, SageMaker and OpenResponses front ends over the same token generator.

* KServe v2 (``/v2/...``): liveness / readiness / model metadata and ``infer`` with one BYTES
  input tensor ``text_input`` (optional scalar parameters ``max_tokens``, ``temperature``, ...);
  the answer is a BYTES tensor ``text_output``.
* SageMaker: ``GET /ping`` and ``POST /invocations``; the body is an OpenAI chat-completions or
  completions request (chosen by the presence of ``messages``) and is handled by those routes.
* OpenResponses (``POST /v1/responses``): ``input`` is a string or a list of role/content items;
  the result is a ``response`` object with one ``message`` output item, optionally streamed as
  ``response.output_text.delta`` / ``response.completed`` events.

Reference: max/python/max/serve/router/kserve_routes.py, sagemaker_routes.py,
openresponses_routes.py (route tables) and serve/api_server.py:330 (router selection by
``Settings.api_types``).
"""

from __future__ import annotations

import json
import time
import uuid
from typing import Any, AsyncIterator, Optional, Union

from fastapi import APIRouter, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse
from pydantic import BaseModel, Field

from ...pipelines.context import SamplingParams
from ..schemas.openai import ChatCompletionRequest, CompletionRequest
from ..worker_interface import RequestQueueFull
from .openai_routes import (_check_model, _pipeline, create_chat_completion, create_completion,
                            error_response)

kserve_router = APIRouter()
sagemaker_router = APIRouter()
responses_router = APIRouter()


# ------------------------------------------------------------------------------ KServe v2
class KServeTensor(BaseModel):
    name: str
    shape: list[int] = Field(default_factory=lambda: [1])
    datatype: str = "BYTES"
    data: list[Any]


class KServeInferRequest(BaseModel):
    id: Optional[str] = None
    inputs: list[KServeTensor]
    parameters: dict[str, Any] = Field(default_factory=dict)


@kserve_router.get("/v2/health/live")
async def kserve_live() -> dict:
    return {"live": True}


@kserve_router.get("/v2/health/ready")
async def kserve_ready(request: Request):
    ready = getattr(request.app.state, "pipeline", None) is not None
    return JSONResponse(status_code=200 if ready else 503, content={"ready": ready})


@kserve_router.get("/v2/models/{name:path}/ready")
async def kserve_model_ready(name: str, request: Request):
    _check_model(request, name)
    return {"name": name, "ready": getattr(request.app.state, "pipeline", None) is not None}


@kserve_router.get("/v2/models/{name:path}")
async def kserve_model_metadata(name: str, request: Request) -> dict:
    _check_model(request, name)
    return {"name": name, "versions": ["1"], "platform": "modular_b200",
            "inputs": [{"name": "text_input", "datatype": "BYTES", "shape": [-1]}],
            "outputs": [{"name": "text_output", "datatype": "BYTES", "shape": [-1]}]}


def _sampling_from_params(p: dict) -> SamplingParams:
    try:
        return SamplingParams(
            max_new_tokens=p.get("max_tokens"), temperature=float(p.get("temperature", 1.0)),
            top_k=int(p.get("top_k", -1)), top_p=float(p.get("top_p", 1.0)), min_p=float(p.get("min_p", 0.0)),
            seed=int(p.get("seed", 0)), ignore_eos=bool(p.get("ignore_eos", False)), stop=p.get("stop"))
    except (TypeError, ValueError) as e:
        raise HTTPException(status_code=400, detail=f"bad parameters: {e}") from e


@kserve_router.post("/v2/models/{name:path}/infer")
async def kserve_infer(name: str, req: KServeInferRequest, request: Request):
    pipeline = _pipeline(request)
    _check_model(request, name)
    texts = [t for t in req.inputs if t.name in ("text_input", "prompt", "input")]
    if len(texts) != 1 or texts[0].datatype != "BYTES" or not texts[0].data:
        return error_response(400, "expected exactly one BYTES input tensor named text_input")
    sp = _sampling_from_params(req.parameters)
    rid = req.id or getattr(request.state, "request_id", uuid.uuid4().hex)
    try:
        outs = []
        for i, prompt in enumerate(texts[0].data):
            if not isinstance(prompt, str):
                return error_response(400, "text_input data must be strings")
            outs.append((await pipeline.all_tokens(prompt, sp, f"{rid}-{i}")).text)
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except ValueError as e:
        return error_response(400, str(e))
    return {"id": rid, "model_name": name, "model_version": "1",
            "outputs": [{"name": "text_output", "datatype": "BYTES", "shape": [len(outs)], "data": outs}]}


# ------------------------------------------------------------------------------ SageMaker
@sagemaker_router.get("/ping")
async def sagemaker_ping(request: Request):
    ready = getattr(request.app.state, "pipeline", None) is not None
    return JSONResponse(status_code=200 if ready else 503, content={"status": "ok" if ready else "starting"})


@sagemaker_router.post("/invocations")
async def sagemaker_invocations(request: Request):
    try:
        body = await request.json()
    except json.JSONDecodeError:
        return error_response(400, "body must be JSON")
    if not isinstance(body, dict):
        return error_response(400, "body must be a JSON object")
    body.setdefault("model", sorted(request.app.state.model_names)[0])
    try:
        if "messages" in body:
            return await create_chat_completion(ChatCompletionRequest(**body), request)
        return await create_completion(CompletionRequest(**body), request)
    except (TypeError, ValueError) as e:
        return error_response(400, f"invalid request: {e}")


# ------------------------------------------------------------------------------ OpenResponses
class ResponsesRequest(BaseModel):
    model: str
    input: Union[str, list[dict]]
    instructions: Optional[str] = None
    max_output_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    stream: bool = False


def _responses_messages(req: ResponsesRequest) -> list[dict]:
    msgs = [{"role": "system", "content": req.instructions}] if req.instructions else []
    if isinstance(req.input, str):
        return msgs + [{"role": "user", "content": req.input}]
    for item in req.input:
        content = item.get("content", "")
        if isinstance(content, list):   # [{"type": "input_text", "text": ...}, ...]
            content = "".join(part.get("text", "") for part in content if isinstance(part, dict))
        msgs.append({"role": item.get("role", "user"), "content": content})
    if not msgs:
        raise HTTPException(status_code=400, detail="input must not be empty")
    return msgs


def _response_object(rid: str, model: str, text: str, status: str, usage: Optional[dict]) -> dict:
    return {"id": rid, "object": "response", "created_at": int(time.time()), "status": status, "model": model,
            "output": [{"type": "message", "id": f"msg_{rid}", "role": "assistant", "status": status,
                        "content": [{"type": "output_text", "text": text, "annotations": []}]}],
            "usage": usage}


@responses_router.post("/v1/responses")
async def create_response(req: ResponsesRequest, request: Request):
    pipeline = _pipeline(request)
    _check_model(request, req.model)
    prompt = pipeline.tokenizer.apply_chat_template(_responses_messages(req), add_generation_prompt=True)
    try:
        sp = SamplingParams(max_new_tokens=req.max_output_tokens,
                            temperature=req.temperature if req.temperature is not None else 1.0,
                            top_p=req.top_p if req.top_p is not None else 1.0)
    except ValueError as e:
        return error_response(400, str(e))
    rid = "resp_" + getattr(request.state, "request_id", uuid.uuid4().hex)

    def usage_of(ch) -> dict:
        return {"input_tokens": ch.prompt_tokens, "output_tokens": ch.completion_tokens,
                "total_tokens": ch.prompt_tokens + ch.completion_tokens}

    try:
        if not req.stream:
            ch = await pipeline.all_tokens(prompt, sp, rid)
            status = "completed" if ch.finish_reason in ("stop", None) else "incomplete"
            return _response_object(rid, req.model, ch.text, status, usage_of(ch))

        async def gen() -> AsyncIterator[bytes]:
            def ev(name: str, payload: dict) -> bytes:
                return f"event: {name}\ndata: {json.dumps({'type': name, **payload})}\n\n".encode()

            yield ev("response.created", {"response": _response_object(rid, req.model, "", "in_progress", None)})
            text, last = "", None
            async for ch in pipeline.next_token_chunk(prompt, sp, rid):
                last = ch
                if ch.text:
                    text += ch.text
                    yield ev("response.output_text.delta", {"item_id": f"msg_{rid}", "delta": ch.text})
            yield ev("response.output_text.done", {"item_id": f"msg_{rid}", "text": text})
            yield ev("response.completed",
                     {"response": _response_object(rid, req.model, text, "completed", usage_of(last) if last else None)})

        return StreamingResponse(gen(), media_type="text/event-stream")
    except RequestQueueFull as e:
        return error_response(429, str(e), "rate_limit_error")
    except ValueError as e:
        return error_response(400, str(e))
