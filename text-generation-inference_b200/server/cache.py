"""Batches kept between RPCs, keyed by batch id (reference: ``server/text_generation_server/cache.py:10-34``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch


class Cache:
    def __init__(self):
        self.cache: Dict[int, object] = {}

    def pop(self, batch_id: int):
        return self.cache.pop(batch_id, None)

    def set(self, entry):
        if entry is not None:
            self.cache[entry.batch_id] = entry

    def delete(self, batch_id: int):
        batch = self.pop(batch_id)
        if batch is not None:
            del batch
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def clear(self):
        for k in list(self.cache.keys()):
            self.delete(k)

    def __len__(self):
        return len(self.cache)
