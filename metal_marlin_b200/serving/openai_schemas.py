"""OpenAI-compatible request / response schemas.
Parity: reference ``metal_marlin/serving/openai_schemas.py`` (field names and defaults)."""
from __future__ import annotations

import time
import uuid
from typing import Dict, List, Literal, Optional, Union

from pydantic import BaseModel, Field


class ChatMessage(BaseModel):
    role: Literal["system", "user", "assistant", "tool"]
    content: str


class ChatCompletionRequest(BaseModel):
    model: str
    messages: List[ChatMessage] = Field(..., min_length=1)
    temperature: float = Field(1.0, ge=0.0, le=2.0)
    top_p: float = Field(1.0, gt=0.0, le=1.0)
    top_k: int = Field(0, ge=0)
    max_tokens: Optional[int] = Field(None, ge=1)
    stream: bool = False
    stop: Optional[Union[str, List[str]]] = None
    n: int = Field(1, ge=1, le=8)
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    user: Optional[str] = None


class CompletionRequest(BaseModel):
    model: str
    prompt: Union[str, List[str]]
    max_tokens: int = Field(16, ge=1)
    temperature: float = Field(1.0, ge=0.0, le=2.0)
    top_p: float = Field(1.0, gt=0.0, le=1.0)
    top_k: int = Field(0, ge=0)
    stream: bool = False
    stop: Optional[Union[str, List[str]]] = None
    n: int = Field(1, ge=1, le=8)
    echo: bool = False
    repetition_penalty: float = 1.0
    seed: Optional[int] = None


class Usage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class ChatChoice(BaseModel):
    index: int = 0
    message: ChatMessage
    finish_reason: Optional[str] = "stop"


class ChatCompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: "chatcmpl-" + uuid.uuid4().hex[:24])
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: List[ChatChoice]
    usage: Usage = Field(default_factory=Usage)


class ChatDelta(BaseModel):
    role: Optional[str] = None
    content: Optional[str] = None


class ChatChunkChoice(BaseModel):
    index: int = 0
    delta: ChatDelta
    finish_reason: Optional[str] = None


class ChatCompletionChunk(BaseModel):
    id: str
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: List[ChatChunkChoice]


class CompletionChoice(BaseModel):
    index: int = 0
    text: str
    finish_reason: Optional[str] = "stop"
    logprobs: Optional[Dict] = None


class CompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: "cmpl-" + uuid.uuid4().hex[:24])
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: List[CompletionChoice]
    usage: Usage = Field(default_factory=Usage)


class ModelInfo(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "metal-marlin"


class ModelList(BaseModel):
    object: str = "list"
    data: List[ModelInfo]


class PerplexityRequest(BaseModel):
    text: str
    chunk_size: int = Field(100, ge=2)
    include_token_ppls: bool = False
    model: Optional[str] = None


class PerplexityResponse(BaseModel):
    perplexity: float
    tokens: int
    loss: float
    chunk_perplexities: List[float]
    chunk_size: int
    token_ppls: Optional[List[float]] = None
