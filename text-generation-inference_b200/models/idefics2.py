"""Idefics2 prompt layout: marker tokens around every image and the optional split into four quadrants plus the
whole image.

Reference: ``models/vlm_causal_lm.py:100-118`` (``image_text_replacement`` for Idefics2) over the processor of
``transformers`` (``models/idefics2/processing_idefics2.py``): one image becomes
``<fake_token_around_image>`` + L image rows + ``<fake_token_around_image>``; with ``do_image_splitting`` that string
is repeated for the four quadrants and the whole image and doubled markers collapse, i.e.
``<fake>`` + 5 x (L rows + ``<fake>``).  As for Idefics3 (``models/idefics3.py``) the expansion is one run of
placeholder rows in the prompt whose marker rows get the marker token's embedding; a tokenizer without the marker
token gets the plain L rows of the whole image.  Every view is resized to the tower's square input here (the
processor keeps the aspect ratio and pads).
"""
from __future__ import annotations

import io
from typing import List, Optional, Tuple

import torch

from .vlm_causal_lm import VlmCausalLM, VlmCausalLMBatch, preprocess_image


def expansion_length(views: int, seq: int) -> int:
    return views * (seq + 1) + 1


def find_fake_token(tokenizer) -> Optional[int]:
    conv = getattr(tokenizer, "convert_tokens_to_ids", None)
    if conv is None:
        return None
    i = conv("<fake_token_around_image>")
    unk = getattr(tokenizer, "unk_token_id", None)
    return None if i is None or i == unk or (isinstance(i, int) and i < 0) else int(i)


def quadrants_and_whole(data: bytes) -> List[bytes]:
    """PNG bytes of the four quadrants (top-left, top-right, bottom-left, bottom-right) and of the whole image."""
    from PIL import Image

    img = Image.open(io.BytesIO(data)).convert("RGB")
    w, h = img.size
    mw, mh = w // 2, h // 2
    boxes = [(0, 0, mw, mh), (mw, 0, w, mh), (0, mh, mw, h), (mw, mh, w, h)]
    out = []
    for box in boxes:
        buf = io.BytesIO()
        img.crop(box).save(buf, format="PNG")
        out.append(buf.getvalue())
    out.append(data)
    return out


class Idefics2Batch(VlmCausalLMBatch):
    fake_id: Optional[int] = None
    do_split: bool = False

    @classmethod
    def image_payload(cls, data: bytes):
        if cls.fake_id is None:
            return super().image_payload(data)
        parts = quadrants_and_whole(data) if cls.do_split and min(_size(data)) >= 2 else [data]
        views = torch.stack([preprocess_image(p, cls.image_size, *cls.norm) for p in parts])
        return views, expansion_length(len(parts), cls.tokens_per_image)

    @classmethod
    def join_adjacent(cls, payload, rows: int):
        if cls.fake_id is None:
            return payload, rows
        return _Joined(payload), rows - 1


class _Joined:
    """Views of an image that directly follows another image: its opening marker is the previous image's closing one
    (the processor collapses doubled markers)."""

    def __init__(self, views: torch.Tensor):
        self.views = views


def _size(data: bytes) -> Tuple[int, int]:
    from PIL import Image

    return Image.open(io.BytesIO(data)).size


class Idefics2CausalLM(VlmCausalLM):
    def __init__(self, *args, do_split: bool = False, **kw):
        super().__init__(*args, **kw)
        self.fake_id = find_fake_token(self.tokenizer)
        base = self.batch_cls
        self.batch_cls = type("BoundIdefics2Batch", (Idefics2Batch,), dict(
            image_token_id=base.image_token_id, tokens_per_image=base.tokens_per_image, image_size=base.image_size,
            norm=base.norm, fake_id=self.fake_id, do_split=bool(do_split)))

    def image_features(self, payloads: list) -> List[torch.Tensor]:
        if self.fake_id is None:
            return super().image_features(payloads)
        views = [p.views if isinstance(p, _Joined) else p for p in payloads]
        feats = self.encode_images(torch.cat(views))                      # [sum of views, L, H]
        t = torch.tensor([self.fake_id], dtype=torch.int32, device=self.device)
        fake = self.model.embed_tokens(t, torch.zeros_like(t)).to(feats.dtype)
        out, cursor = [], 0
        for p, vw in zip(payloads, views):
            parts = [] if isinstance(p, _Joined) else [fake]
            for v in range(vw.shape[0]):
                parts += [feats[cursor + v], fake]
            cursor += vw.shape[0]
            out.append(torch.cat(parts, dim=0))
        return out


def processor_split_setting(path) -> bool:
    """``do_image_splitting`` of the checkpoint's ``preprocessor_config.json`` (the processor's default is off)."""
    import json
    from pathlib import Path

    f = Path(path) / "preprocessor_config.json"
    if f.exists():
        try:
            return bool(json.loads(f.read_text()).get("do_image_splitting", False))
        except (OSError, ValueError):
            pass
    return False
