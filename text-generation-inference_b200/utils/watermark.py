"""Green-list watermarking of generated text ("A Watermark for Large Language Models", arXiv:2301.10226).

Behaviour of the reference's ``utils/watermark.py:22-98``: the previous token seeds a generator
(``hash_key * token``), a fraction ``gamma`` of the vocabulary drawn from it is the green list, and
green tokens get a bias ``delta`` on their logits.  ``WATERMARK_GAMMA`` / ``WATERMARK_DELTA`` set
the two constants.
"""
from __future__ import annotations

import os
from typing import List, Union

import torch

GAMMA = float(os.getenv("WATERMARK_GAMMA", 0.5))
DELTA = float(os.getenv("WATERMARK_DELTA", 2.0))


class WatermarkProcessor:
    def __init__(self, gamma: float = GAMMA, delta: float = DELTA, hash_key: int = 15485863, device="cpu"):
        self.gamma, self.delta, self.hash_key = gamma, delta, hash_key
        self.device = torch.device(device)
        self.rng = torch.Generator(device="cpu")

    def _seed_rng(self, input_ids: Union[List[int], torch.Tensor]) -> None:
        if isinstance(input_ids, list):
            assert len(input_ids) >= 1, "requires at least a 1 token prefix sequence to seed rng"
            prev = input_ids[-1]
        else:
            assert len(input_ids) == 1, "one sequence at a time"
            seq = input_ids[0]
            assert seq.shape[-1] >= 1, "requires at least a 1 token prefix sequence to seed rng"
            prev = int(seq[-1].item())
        self.rng.manual_seed(self.hash_key * prev)

    def green_list(self, input_ids, vocab_size: int) -> torch.Tensor:
        self._seed_rng(input_ids)
        size = int(vocab_size * self.gamma)
        return torch.randperm(vocab_size, generator=self.rng)[:size]

    def __call__(self, input_ids, scores: torch.Tensor) -> torch.Tensor:
        green = self.green_list(input_ids, scores.shape[-1]).to(scores.device)
        mask = torch.zeros_like(scores, dtype=torch.bool)
        mask[-1, green] = True
        scores[mask] = scores[mask] + self.delta
        return scores
