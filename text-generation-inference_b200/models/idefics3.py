"""Idefics3 / SmolVLM image splitting: a large image becomes a grid of tiles plus a global view.

Reference: ``models/vlm_causal_lm.py:60-136`` (``image_text_replacement`` builds the prompt text of a split image from
the processor's ``rows`` / ``cols``) over the image processor of ``transformers``
(``models/idefics3/image_processing_idefics3.py``: longest edge scaled to ``size.longest_edge``, both edges rounded up
to multiples of the tile, ``rows x cols`` tiles of ``max_image_size.longest_edge`` pixels, the whole image resized to
one more tile).  The prompt of one image is

    for every tile row:  <fake_token_around_image><row_r_col_c> + seq image rows, per tile;  then "\\n"
    then                 "\\n"<fake_token_around_image><global-img> + seq image rows <fake_token_around_image>

and an image that fits one tile is ``<fake_token_around_image><global-img>`` + seq rows + ``<fake_token_around_image>``.

Here the whole expansion of an image is one run of placeholder rows in the prompt (the router counts them with the
same arithmetic, ``router/src/images.cpp``); the runner fills the rows of the run with the embeddings of the marker
tokens and with the tiles' features in that order.  A tokenizer without the marker tokens (test fixtures, converted
checkpoints) gets the single global view without markers.
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .vlm_causal_lm import SIGLIP_MEAN, SIGLIP_STD, VlmCausalLM, VlmCausalLMBatch

UPPER_EDGE = 4096          # no edge of the resized image exceeds this


def tile_grid(height: int, width: int, longest_edge: int, tile: int) -> Tuple[int, int, int, int]:
    """``(resized height, resized width, rows, cols)``; ``rows == cols == 0`` when the image fits one tile."""
    aspect = width / height
    # 1. the longer edge becomes `longest_edge`, the other follows the aspect ratio and is made even
    if width >= height:
        w = longest_edge
        h = int(w / aspect)
        h += h % 2
    else:
        h = longest_edge
        w = int(h * aspect)
        w += w % 2
    h, w = max(h, 1), max(w, 1)
    aspect2 = w / h
    if w >= h and w > UPPER_EDGE:
        w = UPPER_EDGE
        h = int(w / aspect2)
    elif h > w and h > UPPER_EDGE:
        h = UPPER_EDGE
        w = int(h * aspect2)
    h, w = max(h, 1), max(w, 1)
    # 2. both edges up to multiples of the tile
    aspect3 = w / h
    if w >= h:
        w = math.ceil(w / tile) * tile
        h = int(w / aspect3)
        h = math.ceil(h / tile) * tile
    else:
        h = math.ceil(h / tile) * tile
        w = int(h * aspect3)
        w = math.ceil(w / tile) * tile
    if h > tile or w > tile:
        return h, w, math.ceil(h / tile), math.ceil(w / tile)
    return h, w, 0, 0


def expansion_length(rows: int, cols: int, seq: int, nl: int, nlnl: int) -> int:
    """Prompt rows of one image with marker tokens: ``nl`` / ``nlnl`` are the token counts of "\\n" and "\\n\\n"."""
    if rows == 0:
        return seq + 3
    return rows * cols * (seq + 2) + (rows - 1) * nl + nlnl + seq + 3


@dataclass
class Markers:
    fake: int
    global_img: int
    newline: List[int]
    double_newline: List[int]
    row_col: Dict[Tuple[int, int], int]


def find_markers(tokenizer, max_side: int = 8) -> Optional[Markers]:
    """The ids of the marker tokens, or ``None`` when the tokenizer does not have them."""
    conv = getattr(tokenizer, "convert_tokens_to_ids", None)
    if conv is None:
        return None
    unk = getattr(tokenizer, "unk_token_id", None)

    def one(tok):
        i = conv(tok)
        return None if i is None or i == unk or (isinstance(i, int) and i < 0) else int(i)

    fake, glob = one("<fake_token_around_image>"), one("<global-img>")
    if fake is None or glob is None:
        return None
    grid = {}
    for r in range(1, max_side + 1):
        for c in range(1, max_side + 1):
            i = one(f"<row_{r}_col_{c}>")
            if i is not None:
                grid[(r, c)] = i
    if (1, 1) not in grid:
        return None
    enc = lambda s: list(tokenizer(s, add_special_tokens=False)["input_ids"])     # noqa: E731
    return Markers(fake, glob, enc("\n"), enc("\n\n"), grid)


@dataclass
class SplitImage:
    views: torch.Tensor          # [rows * cols + 1, 3, S, S] (tiles in row-major order, then the global view), or [1, ...]
    rows: int
    cols: int


def split_views(data: bytes, longest_edge: int, tile: int, mean=SIGLIP_MEAN, std=SIGLIP_STD) -> SplitImage:
    from PIL import Image

    img = Image.open(io.BytesIO(data)).convert("RGB")
    h, w, rows, cols = tile_grid(img.height, img.width, longest_edge, tile)
    big = img.resize((w, h), Image.LANCZOS)

    def to_tensor(im):
        t = torch.frombuffer(bytearray(im.tobytes()), dtype=torch.uint8).view(im.height, im.width, 3)
        t = t.permute(2, 0, 1).float() / 255.0
        return (t - torch.tensor(mean).view(3, 1, 1)) / torch.tensor(std).view(3, 1, 1)

    if rows == 0:
        return SplitImage(to_tensor(big).unsqueeze(0), 0, 0)
    full = to_tensor(big)
    tiles = full.unfold(1, tile, tile).unfold(2, tile, tile)          # [3, rows, cols, tile, tile]
    tiles = tiles.permute(1, 2, 0, 3, 4).reshape(rows * cols, 3, tile, tile)
    glob = to_tensor(big.resize((tile, tile), Image.LANCZOS)).unsqueeze(0)
    return SplitImage(torch.cat([tiles, glob]).contiguous(), rows, cols)


class Idefics3Batch(VlmCausalLMBatch):
    longest_edge: int = 4 * 364
    do_split: bool = True
    markers: Optional[Markers] = None

    @classmethod
    def image_payload(cls, data: bytes):
        if cls.markers is None:
            return super().image_payload(data)
        if not cls.do_split:       # one global view between the markers
            view, _ = super().image_payload(data)
            return SplitImage(view.unsqueeze(0), 0, 0), expansion_length(0, 0, cls.tokens_per_image, 0, 0)
        sp = split_views(data, cls.longest_edge, cls.image_size, *cls.norm)
        if sp.rows and any((r, c) not in cls.markers.row_col for r in range(1, sp.rows + 1) for c in range(1, sp.cols + 1)):
            raise ValueError(f"the tokenizer has no marker for a {sp.rows} x {sp.cols} image grid")
        n = expansion_length(sp.rows, sp.cols, cls.tokens_per_image, len(cls.markers.newline), len(cls.markers.double_newline))
        return sp, n


class Idefics3CausalLM(VlmCausalLM):
    """Adds the split-image prompt layout to the generic vision-language runner."""

    def __init__(self, *args, longest_edge: int, do_split: bool = True, **kw):
        super().__init__(*args, **kw)
        self.markers = find_markers(self.tokenizer)
        base = self.batch_cls
        self.batch_cls = type("BoundIdefics3Batch", (Idefics3Batch,), dict(
            image_token_id=base.image_token_id, tokens_per_image=base.tokens_per_image, image_size=base.image_size,
            norm=base.norm, longest_edge=int(longest_edge), do_split=bool(do_split), markers=self.markers))

    def _embed(self, ids: List[int]) -> torch.Tensor:
        t = torch.tensor(ids, dtype=torch.int32, device=self.device)
        return self.model.embed_tokens(t, torch.zeros_like(t))

    def image_features(self, payloads: list) -> List[torch.Tensor]:
        if self.markers is None:
            return super().image_features(payloads)
        m = self.markers
        feats = self.encode_images(torch.cat([p.views for p in payloads]))        # [sum of views, seq, H]
        out, cursor = [], 0
        for p in payloads:
            n = p.views.shape[0]
            f = feats[cursor:cursor + n]
            cursor += n
            parts: List[torch.Tensor] = []
            for r in range(p.rows):
                for c in range(p.cols):
                    parts.append(self._embed([m.fake, m.row_col[(r + 1, c + 1)]]).to(f.dtype))
                    parts.append(f[r * p.cols + c])
                parts.append(self._embed(m.newline if r < p.rows - 1 else m.double_newline).to(f.dtype))
            parts.append(self._embed([m.fake, m.global_img]).to(f.dtype))
            parts.append(f[n - 1])
            parts.append(self._embed([m.fake]).to(f.dtype))
            out.append(torch.cat(parts, dim=0))
        return out


def processor_settings(path, image_size: int) -> Tuple[int, bool]:
    """``(size.longest_edge, do_image_splitting)`` of the checkpoint's ``preprocessor_config.json`` (defaults: four
    tiles along the longer edge, splitting on)."""
    import json
    from pathlib import Path

    f = Path(path) / "preprocessor_config.json"
    longest, split = 4 * image_size, True
    if f.exists():
        try:
            pc = json.loads(f.read_text())
            size = pc.get("size") or {}
            if isinstance(size, dict) and size.get("longest_edge"):
                longest = int(size["longest_edge"])
            split = bool(pc.get("do_image_splitting", True))
        except (OSError, ValueError):
            pass
    return longest, split
