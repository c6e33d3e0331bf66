"""Base class of model runners: shard identity, ``Info`` answer, incremental detokenisation.

Same role as ``server/text_generation_server/models/model.py:29-181`` of the reference.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Optional, Tuple, Type

import torch

from ..proto import generate_v3 as pb
from .types import Batch, Generation


class Model(ABC):
    def __init__(self, model, tokenizer, requires_padding: bool, dtype: torch.dtype, device: torch.device,
                 rank: int = 0, world_size: int = 1, sliding_window: Optional[int] = None, speculate: int = 0,
                 support_chunking: bool = True, use_prefix_caching: bool = True, block_size: int = 16,
                 attention_impl: str = "paged-sm100"):
        self.model = model
        self.tokenizer = tokenizer
        self.all_special_ids = set(getattr(tokenizer, "all_special_ids", []) or [])
        self.requires_padding = requires_padding
        self.dtype, self.device = dtype, device
        self.rank, self.world_size = rank, world_size
        self.sliding_window = sliding_window if sliding_window != -1 else None
        self.speculate = speculate
        # Chunked prefill expands one request over several forward passes; a speculative step assumes
        # one new token per request and sequence, so the two are exclusive (as in the reference,
        # ``models/model.py:73-92``).
        self.support_chunking = support_chunking and speculate == 0
        self.use_prefix_caching = use_prefix_caching
        self.block_size = block_size
        self.attention_impl = attention_impl

    @property
    def info(self):
        m = pb.InfoResponse(
            requires_padding=self.requires_padding, dtype=str(self.dtype), device_type=self.device.type,
            speculate=self.speculate, support_chunking=self.support_chunking,
            use_prefix_caching=self.use_prefix_caching, attention_impl=self.attention_impl,
            block_size=self.block_size,
        )
        if self.sliding_window is not None:
            m.window_size = self.sliding_window
        return m

    @property
    @abstractmethod
    def batch_type(self) -> Type[Batch]:
        ...

    @abstractmethod
    def generate_token(self, batch) -> Tuple[List[Generation], Optional[Batch], Tuple[int, int]]:
        ...

    def warmup(self, batch, max_input_tokens: Optional[int], max_total_tokens: Optional[int]):
        self.generate_token(batch)
        return None, max_input_tokens or 0, max_total_tokens or 0

    def decode_token(self, all_input_ids: List[int], prefix_offset: int = 0, read_offset: int = 0,
                     skip_special_tokens: bool = False) -> Tuple[str, int, int]:
        """Text of the tokens after ``read_offset``, decoded with left context so that byte-fallback
        and space-prefix tokenisers render correctly; returns ``("", same offsets)`` while the tail
        is an incomplete UTF-8 sequence (ends with U+FFFD)."""
        prefix_text = self.tokenizer.decode(all_input_ids[prefix_offset:read_offset],
                                            skip_special_tokens=skip_special_tokens)
        new_text = self.tokenizer.decode(all_input_ids[prefix_offset:], skip_special_tokens=skip_special_tokens)
        if len(new_text) > len(prefix_text) and not new_text.endswith("�"):
            return new_text[len(prefix_text):], read_offset, len(all_input_ids)
        return "", prefix_offset, read_offset

    def check_initialized(self):
        pass
