"""OpenAI-compatible request and response models (the subset the routers implement).

Reference: max/python/max/serve/schemas/openai.py. Unknown request fields are accepted and
ignored so that stock OpenAI clients work unchanged.
"""

from __future__ import annotations

import time
import uuid
from typing import Any, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field


class _Req(BaseModel):
    model_config = ConfigDict(extra="allow")


class StreamOptions(_Req):
    include_usage: bool = False


class ResponseFormat(_Req):
    type: Literal["text", "json_object", "json_schema"] = "text"
    json_schema: Optional[dict] = None


class _SamplingMixin(_Req):
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    repetition_penalty: Optional[float] = None
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    seed: Optional[int] = None
    ignore_eos: bool = False
    min_tokens: Optional[int] = None
    logit_bias: Optional[dict[str, float]] = None    # token id -> additive bias in [-100, 100]
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    logprobs: Optional[Union[bool, int]] = None
    top_logprobs: Optional[int] = None
    user: Optional[str] = None
    cache_salt: Optional[str] = None    # requests with different salts never share prefix-cache pages


class CompletionRequest(_SamplingMixin):
    model: str
    prompt: Union[str, list[str], list[int], list[list[int]]]
    echo: bool = False
    suffix: Optional[str] = None


class ChatMessage(_Req):
    role: str
    content: Optional[Union[str, list[dict]]] = None
    name: Optional[str] = None
    tool_calls: Optional[list[dict]] = None
    tool_call_id: Optional[str] = None


class ChatCompletionRequest(_SamplingMixin):
    model: str
    messages: list[ChatMessage]
    max_completion_tokens: Optional[int] = None
    tools: Optional[list[dict]] = None
    tool_choice: Optional[Union[str, dict]] = None
    response_format: Optional[ResponseFormat] = None


class EmbeddingRequest(_Req):
    model: str
    input: Union[str, list[str], list[int], list[list[int]]]
    encoding_format: Literal["float", "base64"] = "float"


class Usage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class CompletionChoice(BaseModel):
    index: int = 0
    text: str = ""
    logprobs: Optional[Any] = None
    finish_reason: Optional[str] = None


class CompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: f"cmpl-{uuid.uuid4().hex}")
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[CompletionChoice] = Field(default_factory=list)
    usage: Optional[Usage] = None


class ChatChoiceMessage(BaseModel):
    role: str = "assistant"
    content: Optional[str] = None
    reasoning_content: Optional[str] = None
    tool_calls: Optional[list[dict]] = None


class ChatChoice(BaseModel):
    index: int = 0
    message: ChatChoiceMessage = Field(default_factory=ChatChoiceMessage)
    logprobs: Optional[Any] = None
    finish_reason: Optional[str] = None


class ChatCompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: f"chatcmpl-{uuid.uuid4().hex}")
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[ChatChoice] = Field(default_factory=list)
    usage: Optional[Usage] = None


class ChatDelta(BaseModel):
    role: Optional[str] = None
    content: Optional[str] = None
    reasoning_content: Optional[str] = None
    tool_calls: Optional[list[dict]] = None


class ChatChunkChoice(BaseModel):
    index: int = 0
    delta: ChatDelta = Field(default_factory=ChatDelta)
    finish_reason: Optional[str] = None


class ChatCompletionChunk(BaseModel):
    id: str = ""
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: list[ChatChunkChoice] = Field(default_factory=list)
    usage: Optional[Usage] = None


class ModelCard(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "modular_b200"


class ModelList(BaseModel):
    object: str = "list"
    data: list[ModelCard] = Field(default_factory=list)


class LoadLoraRequest(_Req):
    lora_name: str
    lora_path: str
    alpha: Optional[float] = None


class UnloadLoraRequest(_Req):
    lora_name: str


class ErrorBody(BaseModel):
    message: str
    type: str = "invalid_request_error"
    param: Optional[str] = None
    code: Optional[Union[int, str]] = None


class ErrorResponse(BaseModel):
    error: ErrorBody


class EmbeddingsRequest(BaseModel):
    model: str
    input: Union[str, list[str], list[int], list[list[int]]]
    encoding_format: str = "float"
    dimensions: Optional[int] = None
    pooling: Optional[str] = None      # extension: "last" | "mean" | "cls" (encoders); default: the model's own
    user: Optional[str] = None


class EmbeddingData(BaseModel):
    object: str = "embedding"
    index: int = 0
    embedding: Union[list[float], str]


class EmbeddingsResponse(BaseModel):
    object: str = "list"
    data: list[EmbeddingData]
    model: str
    usage: Usage
