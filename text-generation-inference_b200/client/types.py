"""Request and response models of the HTTP API (pydantic).

Field names follow the router's JSON (``router/src/api.hpp``), which in turn keeps the wire
format of the reference (``router/src/lib.rs:303-1519``; client-side mirror in
``clients/python/text_generation/types.py``).
"""
from __future__ import annotations

from enum import Enum
from typing import Any, Dict, List, Optional, Union

from pydantic import BaseModel, Field, field_validator


class GrammarType(str, Enum):
    Json = "json"
    Regex = "regex"


class Grammar(BaseModel):
    type: GrammarType
    value: Union[str, Dict[str, Any]]


class Parameters(BaseModel):
    do_sample: bool = False
    max_new_tokens: Optional[int] = None
    repetition_penalty: Optional[float] = None
    frequency_penalty: Optional[float] = None
    return_full_text: bool = False
    stop: List[str] = Field(default_factory=list)
    seed: Optional[int] = None
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    typical_p: Optional[float] = None
    truncate: Optional[int] = None
    best_of: Optional[int] = None
    watermark: bool = False
    details: bool = False
    decoder_input_details: bool = False
    top_n_tokens: Optional[int] = None
    grammar: Optional[Grammar] = None
    adapter_id: Optional[str] = None

    @field_validator("best_of")
    @classmethod
    def _best_of(cls, v, info):
        if v is not None:
            if v <= 0:
                raise ValueError("`best_of` must be strictly positive")
            d = info.data
            sampling = d.get("do_sample") or any(d.get(k) is not None for k in ("temperature", "top_k", "top_p", "typical_p"))
            if v > 1 and not sampling:
                raise ValueError("`best_of` > 1 needs sampling to be active")
        return v

    @field_validator("repetition_penalty", "temperature")
    @classmethod
    def _positive(cls, v):
        if v is not None and v <= 0:
            raise ValueError("must be strictly positive")
        return v

    @field_validator("top_p", "typical_p")
    @classmethod
    def _unit_interval(cls, v):
        if v is not None and not 0 < v < 1:
            raise ValueError("must be > 0.0 and < 1.0")
        return v

    @field_validator("top_k", "truncate", "top_n_tokens")
    @classmethod
    def _strictly_positive_int(cls, v):
        if v is not None and v <= 0:
            raise ValueError("must be strictly positive")
        return v


class Request(BaseModel):
    inputs: str
    parameters: Optional[Parameters] = None
    stream: bool = False

    @field_validator("inputs")
    @classmethod
    def _inputs(cls, v):
        if not v:
            raise ValueError("`inputs` cannot be empty")
        return v


class InputToken(BaseModel):
    id: int
    text: str
    logprob: Optional[float] = None


class Token(BaseModel):
    id: int
    text: str
    logprob: Optional[float] = None
    special: bool = False


class FinishReason(str, Enum):
    Length = "length"
    EndOfSequenceToken = "eos_token"
    StopSequence = "stop_sequence"


class BestOfSequence(BaseModel):
    generated_text: str
    finish_reason: FinishReason
    generated_tokens: int
    seed: Optional[int] = None
    prefill: List[InputToken] = Field(default_factory=list)
    tokens: List[Token] = Field(default_factory=list)
    top_tokens: Optional[List[List[Token]]] = None


class Details(BaseModel):
    finish_reason: FinishReason
    generated_tokens: int
    seed: Optional[int] = None
    prefill: List[InputToken] = Field(default_factory=list)
    tokens: List[Token] = Field(default_factory=list)
    top_tokens: Optional[List[List[Token]]] = None
    best_of_sequences: Optional[List[BestOfSequence]] = None


class Response(BaseModel):
    generated_text: str
    details: Optional[Details] = None


class StreamDetails(BaseModel):
    finish_reason: FinishReason
    generated_tokens: int
    seed: Optional[int] = None
    input_length: Optional[int] = None


class StreamResponse(BaseModel):
    index: Optional[int] = None
    token: Token
    top_tokens: Optional[List[Token]] = None
    generated_text: Optional[str] = None
    details: Optional[StreamDetails] = None


# ---- OpenAI-compatible chat / completion -------------------------------------------------------
class Message(BaseModel):
    role: str
    content: Optional[Union[str, List[Dict[str, Any]]]] = None
    name: Optional[str] = None
    tool_calls: Optional[Any] = None


class Tool(BaseModel):
    type: str = "function"
    function: Dict[str, Any]


class ChatRequest(BaseModel):
    model: str = "tgi"
    messages: List[Message]
    frequency_penalty: Optional[float] = None
    logit_bias: Optional[List[float]] = None
    logprobs: Optional[bool] = None
    top_logprobs: Optional[int] = None
    max_tokens: Optional[int] = None
    n: Optional[int] = None
    presence_penalty: Optional[float] = None
    stream: bool = False
    seed: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    tools: Optional[List[Tool]] = None
    tool_prompt: Optional[str] = None
    tool_choice: Optional[Union[str, Dict[str, Any]]] = None
    response_format: Optional[Dict[str, Any]] = None
    stop: Optional[List[str]] = None


class Usage(BaseModel):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0


class ChatChoice(BaseModel):
    index: int
    message: Message
    logprobs: Optional[Any] = None
    finish_reason: Optional[str] = None


class ChatComplete(BaseModel):
    id: str
    object: str
    created: int
    model: str
    system_fingerprint: str = ""
    choices: List[ChatChoice]
    usage: Optional[Usage] = None


class ChatDelta(BaseModel):
    role: Optional[str] = None
    content: Optional[str] = None
    tool_calls: Optional[Any] = None


class ChatChunkChoice(BaseModel):
    index: int
    delta: ChatDelta
    logprobs: Optional[Any] = None
    finish_reason: Optional[str] = None


class ChatCompletionChunk(BaseModel):
    id: str
    object: str
    created: int
    model: str
    system_fingerprint: str = ""
    choices: List[ChatChunkChoice]
    usage: Optional[Usage] = None


class CompletionRequest(BaseModel):
    model: str = "tgi"
    prompt: Union[str, List[str]]
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    frequency_penalty: Optional[float] = None
    repetition_penalty: Optional[float] = None
    seed: Optional[int] = None
    stream: bool = False
    stop: Optional[List[str]] = None
    suffix: Optional[str] = None


class CompletionChoice(BaseModel):
    index: int
    text: str
    logprobs: Optional[Any] = None
    finish_reason: Optional[str] = None


class Completion(BaseModel):
    id: str
    object: str
    created: int
    model: str
    system_fingerprint: str = ""
    choices: List[CompletionChoice]
    usage: Optional[Usage] = None


class DeployedModel(BaseModel):
    model_id: str
    sha: Optional[str] = None
