"""LLaVA-NeXT "any resolution" images: a base view plus a grid of tiles at the best-fitting resolution.

Reference: ``custom_modeling/llava_next.py:39-303`` (``get_anyres_image_grid_shape``, ``unpad_image``,
``pack_image_features``) and the router's feature count for this family (``router/src/config.rs``).

An image is shown to the tower as ``1 + th * tw`` square views: the whole image resized to the tower's
resolution, and the image resized (aspect kept, centred, zero padded) to the one of ``image_grid_pinpoints``
that wastes the least, cut into ``th x tw`` tiles.  The tile features are laid out again as one
``(th * side) x (tw * side)`` map, the rows / columns that only saw padding are cut off, a learned
``image_newline`` row vector closes every remaining row, and the result follows the base view's rows.  The
number of placeholder rows therefore depends on the size of the image.
"""
from __future__ import annotations

import io
import math
from typing import List, Sequence, Tuple

import numpy as np
import torch

from .vlm_causal_lm import CLIP_MEAN, CLIP_STD, VlmCausalLM, VlmCausalLMBatch


def select_best_resolution(size_hw: Tuple[int, int], pinpoints: Sequence[Sequence[int]]) -> Tuple[int, int]:
    """The candidate (height, width) that keeps most of the image's pixels after an aspect-preserving resize,
    ties broken by the least padding."""
    H, W = size_hw
    best, best_eff, best_waste = None, -1, float("inf")
    for h, w in pinpoints:
        scale = min(w / W, h / H)
        eff = min(int(W * scale) * int(H * scale), W * H)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (int(h), int(w)), eff, waste
    return best


def _fit(size_hw: Tuple[int, int], target_hw: Tuple[int, int]) -> Tuple[int, int]:
    """Size of the image after the aspect-preserving resize into ``target_hw``."""
    H, W = size_hw
    th, tw = target_hw
    if tw / W < th / H:
        return min(math.ceil(H * tw / W), th), tw
    return th, min(math.ceil(W * th / H), tw)


def unpadded_map(size_hw: Tuple[int, int], map_hw: Tuple[int, int]) -> Tuple[int, int, int, int]:
    """(top, bottom, left, right) bounds of the feature map ``map_hw`` that cover the image and not its padding."""
    H, W = size_hw
    mh, mw = map_hw
    if W / H > mw / mh:
        new_h = int(round(H * (mw / W), 7))
        pad = (mh - new_h) // 2
        return pad, mh - pad, 0, mw
    new_w = int(round(W * (mh / H), 7))
    pad = (mw - new_w) // 2
    return 0, mh, pad, mw - pad


def anyres_rows(size_hw: Tuple[int, int], pinpoints, tile: int, side: int) -> int:
    """Placeholder rows of one image: base view + unpadded tile map with one newline column."""
    bh, bw = select_best_resolution(size_hw, pinpoints)
    top, bottom, left, right = unpadded_map(size_hw, (bh // tile * side, bw // tile * side))
    return side * side + (bottom - top) * (right - left + 1)


def anyres_views(data: bytes, pinpoints, tile: int, mean=CLIP_MEAN, std=CLIP_STD):
    """Decode an image into its views ``[1 + th * tw, 3, tile, tile]`` (base first, tiles row-major), its size
    (height, width) and the tile grid (th, tw)."""
    from PIL import Image

    img = Image.open(io.BytesIO(data)).convert("RGB")
    size = (img.height, img.width)
    bh, bw = select_best_resolution(size, pinpoints)
    nh, nw = _fit(size, (bh, bw))
    canvas = Image.new("RGB", (bw, bh), (0, 0, 0))
    canvas.paste(img.resize((nw, nh), Image.BICUBIC), ((bw - nw) // 2, (bh - nh) // 2))
    views = [img.resize((tile, tile), Image.BICUBIC)]
    for y in range(0, bh, tile):
        for x in range(0, bw, tile):
            views.append(canvas.crop((x, y, x + tile, y + tile)))
    arr = torch.from_numpy(np.stack([np.asarray(v, dtype=np.float32) / 255.0 for v in views])).permute(0, 3, 1, 2)
    arr = (arr - torch.tensor(mean).view(1, 3, 1, 1)) / torch.tensor(std).view(1, 3, 1, 1)
    return arr, size, (bh // tile, bw // tile)


class LlavaNextBatch(VlmCausalLMBatch):
    pinpoints: List[List[int]] = [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]]
    feature_side: int = 24

    @classmethod
    def image_payload(cls, data: bytes):
        views, size, grid = anyres_views(data, cls.pinpoints, cls.image_size, *cls.norm)
        return (views, size, grid), anyres_rows(size, cls.pinpoints, cls.image_size, cls.feature_side)


class LlavaNextCausalLM(VlmCausalLM):
    def __init__(self, *args, image_newline: torch.Tensor, pinpoints, **kw):
        super().__init__(*args, **kw)
        self.image_newline = image_newline
        side = int(round(math.sqrt(self.tokens_per_image)))
        base = self.batch_cls
        self.batch_cls = type("BoundLlavaNextBatch", (LlavaNextBatch,), dict(
            image_token_id=base.image_token_id, tokens_per_image=base.tokens_per_image, image_size=base.image_size,
            norm=base.norm, pinpoints=[list(p) for p in pinpoints], feature_side=side))
        self.side = side

    def image_features(self, payloads: list) -> List[torch.Tensor]:
        views = torch.cat([p[0] for p in payloads])
        feats = self.encode_images(views)                       # [sum(1 + tiles), side^2, H]
        out, cursor, s = [], 0, self.side
        for _, size, (th, tw) in payloads:
            base, tiles = feats[cursor], feats[cursor + 1:cursor + 1 + th * tw]
            cursor += 1 + th * tw
            H = tiles.shape[-1]
            fmap = tiles.view(th, tw, s, s, H).permute(0, 2, 1, 3, 4).reshape(th * s, tw * s, H)
            top, bottom, left, right = unpadded_map(size, (th * s, tw * s))
            fmap = fmap[top:bottom, left:right]
            newline = self.image_newline.to(fmap.dtype).view(1, 1, H).expand(fmap.shape[0], 1, H)
            out.append(torch.cat([base, torch.cat([fmap, newline], dim=1).reshape(-1, H)], dim=0))
        return out
