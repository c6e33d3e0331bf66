"""Value types exchanged between the model runner and the gRPC servicer.

Same role as ``server/text_generation_server/models/types.py:13-110`` of the reference.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import List, Optional

from ..proto import generate_v3 as pb


class Batch(ABC):
    @abstractmethod
    def to_pb(self):
        ...

    @classmethod
    @abstractmethod
    def from_pb(cls, batch_pb, tokenizer, dtype, device) -> "Batch":
        ...

    @abstractmethod
    def filter(self, request_ids: List[int]) -> "Batch":
        ...

    @classmethod
    @abstractmethod
    def concatenate(cls, batches: List["Batch"]) -> "Batch":
        ...

    @abstractmethod
    def __len__(self) -> int:
        ...


@dataclass
class GeneratedText:
    text: str
    generated_tokens: int
    finish_reason: int
    seed: Optional[int]

    def to_pb(self):
        m = pb.GeneratedText(text=self.text, generated_tokens=self.generated_tokens, finish_reason=self.finish_reason)
        if self.seed is not None:
            m.seed = self.seed
        return m


@dataclass
class Tokens:
    token_ids: List[int]
    logprobs: List[float]
    texts: List[str]
    is_special: List[bool]

    def to_pb(self):
        return pb.Tokens(ids=self.token_ids, logprobs=self.logprobs, texts=self.texts, is_special=self.is_special)

    def __len__(self):
        return len(self.token_ids)

    def __add__(self, other: "Tokens") -> "Tokens":
        return Tokens(self.token_ids + other.token_ids, self.logprobs + other.logprobs,
                      self.texts + other.texts, self.is_special + other.is_special)


@dataclass
class Generation:
    request_id: int
    prefill_tokens: Optional[Tokens]
    tokens: Tokens
    generated_text: Optional[GeneratedText]
    top_tokens: Optional[List[Tokens]]

    def to_pb(self):
        m = pb.Generation(request_id=self.request_id, tokens=self.tokens.to_pb())
        if self.prefill_tokens is not None:
            m.prefill_tokens.CopyFrom(self.prefill_tokens.to_pb())
        if self.generated_text is not None:
            m.generated_text.CopyFrom(self.generated_text.to_pb())
        if self.top_tokens is not None:
            for t in self.top_tokens:
                m.top_tokens.append(t.to_pb())
        return m
