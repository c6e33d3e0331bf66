"""Qwen2-VL and Qwen2.5-VL: dynamic-resolution vision transformer, 2x2 patch merger and 3-axis rotary
positions.

Reference: ``custom_modeling/qwen2_vl.py`` and ``custom_modeling/qwen2_5_vl.py`` (vision blocks with 2-D
rotary embedding, ``PatchMerger``, ``get_position_ids``; the 2.5 tower uses RMSNorm, a gated SiLU MLP and
attention restricted to windows of 8 x 8 merged patches in all but a few "full attention" blocks) and the
Qwen2-VL branch of ``models/vlm_causal_lm.py`` (image-token expansion
``<|vision_start|><|image_pad|>*n<|vision_end|>``).

Differences from the fixed-resolution families of ``vlm_causal_lm.py``:

* an image keeps its aspect ratio: it is resized so that both sides are multiples of
  ``patch * merge`` (28) inside a pixel budget, cut into patches ordered merge-block by merge-block, and
  contributes ``(h / 28) * (w / 28)`` rows;
* the tower attends inside one image only (ragged batch of images, block-diagonal attention) and rotates
  q/k with the (row, column) of each patch;
* the language model's rotary embedding has three position streams (time, height, width) mixed by
  ``mrope_section``: text advances all three together, the rows of an image share the time index and
  spread over height/width.  The decoder gets the rotary table rows of the step ready-made
  (``ForwardMeta.rope_cos_sin``), so the fused rope + KV-cache kernel runs unchanged; after the prompt
  a sequence's three streams coincide again and only a constant offset (``pos_delta``) remains, which
  keeps decode on the CUDA-graph path.
"""
from __future__ import annotations

import io
import math
from typing import Dict, List, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..utils.weights import Weights
from .flash_causal_lm import FlashCausalLMBatch
from .vlm_causal_lm import CLIP_MEAN, CLIP_STD, VlmCausalLM


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Target size: both sides multiples of ``factor``, area inside ``[min_pixels, max_pixels]``, aspect
    ratio kept as closely as that allows."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("image aspect ratio must be below 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def patchify(pixels: torch.Tensor, patch: int, merge: int, temporal: int) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """``[3, H, W]`` -> (``[gh * gw, 3 * temporal * patch * patch]``, (1, gh, gw)); patches are ordered
    merge block by merge block (the ``merge x merge`` patches that become one row are consecutive) and a
    still image is repeated over the temporal axis."""
    C, H, W = pixels.shape
    gh, gw = H // patch, W // patch
    x = pixels.view(C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(1, 4, 2, 5, 0, 3, 6)                                     # [bh, bw, mh, mw, C, ph, pw]
    x = x.unsqueeze(5).expand(-1, -1, -1, -1, -1, temporal, -1, -1)         # [.., C, T, ph, pw]
    return x.reshape(gh * gw, C * temporal * patch * patch).contiguous(), (1, gh, gw)


def preprocess_qwen_image(data: bytes, patch: int, merge: int, temporal: int, min_pixels: int, max_pixels: int):
    from PIL import Image

    img = Image.open(io.BytesIO(data)).convert("RGB")
    if img.width <= 20:      # very narrow images are doubled first (reference: vlm_causal_lm.py:203-204)
        img = img.resize((img.width * 2, img.height * 2))
    h, w = smart_resize(img.height, img.width, patch * merge, min_pixels, max_pixels)
    img = img.resize((w, h), Image.BICUBIC)
    arr = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
    arr = (arr - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)
    return patchify(arr, patch, merge, temporal)


# ---- vision tower --------------------------------------------------------------------------------
def _rms_norm(x, weight, eps=1e-6):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class Qwen2VisionTower:
    def __init__(self, cfg: dict, w: Weights, prefix: str, v25: bool = False):
        g = w.get_tensor
        self.v25 = v25
        # Qwen2-VL calls the tower width `embed_dim` (and `hidden_size` is the text width); 2.5 calls it `hidden_size`
        self.embed_dim = int(cfg.get("hidden_size", 1280) if v25 else cfg.get("embed_dim", 1280))
        self.window = int(cfg.get("window_size", 112))
        self.full_blocks = set(cfg.get("fullatt_block_indexes", [7, 15, 23, 31])) if v25 else None
        self.heads = int(cfg.get("num_heads", 16))
        self.patch, self.merge = int(cfg.get("patch_size", 14)), int(cfg.get("spatial_merge_size", 2))
        self.temporal = int(cfg.get("temporal_patch_size", 2))
        self.head_dim = self.embed_dim // self.heads
        self.patch_w = g(f"{prefix}.patch_embed.proj.weight").reshape(self.embed_dim, -1)   # conv3d with kernel == stride
        self.blocks = []
        for i in range(int(cfg.get("depth", 32))):
            b = f"{prefix}.blocks.{i}"
            blk = dict(qkv=(g(f"{b}.attn.qkv.weight"), g(f"{b}.attn.qkv.bias")),
                       proj=(g(f"{b}.attn.proj.weight"), g(f"{b}.attn.proj.bias")))
            if v25:
                blk.update(n1=g(f"{b}.norm1.weight"), n2=g(f"{b}.norm2.weight"),
                           gate=(g(f"{b}.mlp.gate_proj.weight"), g(f"{b}.mlp.gate_proj.bias")),
                           up=(g(f"{b}.mlp.up_proj.weight"), g(f"{b}.mlp.up_proj.bias")),
                           down=(g(f"{b}.mlp.down_proj.weight"), g(f"{b}.mlp.down_proj.bias")))
            else:
                blk.update(n1=(g(f"{b}.norm1.weight"), g(f"{b}.norm1.bias")),
                           n2=(g(f"{b}.norm2.weight"), g(f"{b}.norm2.bias")),
                           fc1=(g(f"{b}.mlp.fc1.weight"), g(f"{b}.mlp.fc1.bias")),
                           fc2=(g(f"{b}.mlp.fc2.weight"), g(f"{b}.mlp.fc2.bias")))
            self.blocks.append(blk)
        m = f"{prefix}.merger"
        self.ln_q = g(f"{m}.ln_q.weight") if v25 else (g(f"{m}.ln_q.weight"), g(f"{m}.ln_q.bias"))
        self.m1 = (g(f"{m}.mlp.0.weight"), g(f"{m}.mlp.0.bias"))
        self.m2 = (g(f"{m}.mlp.2.weight"), g(f"{m}.mlp.2.bias"))
        self.act = cfg.get("hidden_act", "quick_gelu")

    def _rotary(self, grids: List[Tuple[int, int, int]], device) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos/sin ``[N, head_dim]``: first half of each rotary half turns with the patch row, second with the column."""
        quarter = self.head_dim // 4
        inv = 1.0 / (10000.0 ** (torch.arange(0, quarter, dtype=torch.float32, device=device) * 2 / (self.head_dim // 2)))
        rows = []
        for t, gh, gw in grids:
            hp = torch.arange(gh, device=device).view(gh // self.merge, self.merge, 1, 1).expand(-1, -1, gw // self.merge, self.merge)
            wp = torch.arange(gw, device=device).view(1, 1, gw // self.merge, self.merge).expand(gh // self.merge, self.merge, -1, -1)
            hp, wp = hp.permute(0, 2, 1, 3).reshape(-1), wp.permute(0, 2, 1, 3).reshape(-1)
            ang = torch.cat([hp.float()[:, None] * inv[None], wp.float()[:, None] * inv[None]], dim=-1)   # [n, head_dim/2]
            rows.append(ang.repeat(t, 1))
        ang = torch.cat(rows, 0)
        ang = torch.cat([ang, ang], dim=-1)
        return ang.cos(), ang.sin()

    @staticmethod
    def _rot(x, cos, sin):                                   # x [N, heads, D], NeoX halves, fp32 like the original
        xf = x.float()
        h = xf.shape[-1] // 2
        rot = torch.cat([-xf[..., h:], xf[..., :h]], dim=-1)
        return (xf * cos[:, None] + rot * sin[:, None]).to(x.dtype)

    def _windows(self, grids: List[Tuple[int, int, int]]) -> Tuple[torch.Tensor, List[int]]:
        """Qwen2.5-VL: order of the merged patches that makes every attention window contiguous, and the
        window boundaries in patches (windows are `window / merge / patch` merged patches on a side; border
        windows are smaller)."""
        side = self.window // self.merge // self.patch
        order, bounds, base = [], [0], 0
        m2 = self.merge ** 2
        for t, gh, gw in grids:
            lh, lw = gh // self.merge, gw // self.merge
            idx = torch.arange(t * lh * lw).view(t, lh, lw)
            ph, pw = side - lh % side, side - lw % side
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (lh + ph) // side, (lw + pw) // side
            idx = idx.view(t, nh, side, nw, side).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, side * side)
            for win in idx:
                keep = win[win >= 0]
                if keep.numel():
                    order.append(keep + base)
                    bounds.append(bounds[-1] + keep.numel() * m2)
            base += t * lh * lw
        return torch.cat(order), bounds

    def _attend(self, q, k, v, bounds):
        out = torch.empty_like(q)
        for lo, hi in zip(bounds[:-1], bounds[1:]):            # attention never crosses a segment
            o = F.scaled_dot_product_attention(q[lo:hi].transpose(0, 1)[None], k[lo:hi].transpose(0, 1)[None],
                                               v[lo:hi].transpose(0, 1)[None])
            out[lo:hi] = o[0].transpose(0, 1)
        return out

    @torch.no_grad()
    def __call__(self, patches: torch.Tensor, grids: List[Tuple[int, int, int]]) -> torch.Tensor:
        """``[sum(gh*gw), C*T*p*p]`` -> ``[sum(gh*gw) / merge^2, out_hidden]``"""
        x = F.linear(patches.to(self.patch_w.dtype), self.patch_w)
        cos, sin = self._rotary(grids, x.device)
        image_bounds = np.cumsum([0] + [gh * gw for t, gh, gw in grids for _ in range(t)]).tolist()
        C, m2 = self.embed_dim, self.merge ** 2
        order = None
        if self.v25:
            order, window_bounds = self._windows(grids)
            order = order.to(x.device)
            regroup = lambda a: a.view(-1, m2, a.shape[-1])[order].reshape(-1, a.shape[-1])
            x, cos, sin = regroup(x), regroup(cos), regroup(sin)
        for li, b in enumerate(self.blocks):
            h = _rms_norm(x, b["n1"]) if self.v25 else F.layer_norm(x, (C,), *b["n1"], 1e-6)
            qkv = F.linear(h, *b["qkv"]).view(-1, 3, self.heads, self.head_dim)
            q, k, v = self._rot(qkv[:, 0], cos, sin), self._rot(qkv[:, 1], cos, sin), qkv[:, 2]
            bounds = image_bounds if (not self.v25 or li in self.full_blocks) else window_bounds
            x = x + F.linear(self._attend(q, k, v, bounds).reshape(-1, C), *b["proj"])
            if self.v25:
                h = _rms_norm(x, b["n2"])
                x = x + F.linear(F.silu(F.linear(h, *b["gate"])) * F.linear(h, *b["up"]), *b["down"])
            else:
                h = F.linear(F.layer_norm(x, (C,), *b["n2"], 1e-6), *b["fc1"])
                h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else F.gelu(h)
                x = x + F.linear(h, *b["fc2"])
        x = _rms_norm(x, self.ln_q) if self.v25 else F.layer_norm(x, (C,), *self.ln_q, 1e-6)
        out = F.linear(F.gelu(F.linear(x.view(-1, C * m2), *self.m1)), *self.m2)
        if order is not None:
            out = out[torch.argsort(order)]                    # back to the order of the image rows
        return out


# ---- batch -----------------------------------------------------------------------------------------
class Qwen2VlBatch(FlashCausalLMBatch):
    """Per request: the patch matrices of its images, where their rows sit in the prompt, and the
    three position streams of the prompt."""

    image_token_id = 0
    vision_start_id = None
    vision_end_id = None
    patch, merge, temporal = 14, 2, 2
    min_pixels, max_pixels = 56 * 56, 14 * 14 * 4 * 1280

    @classmethod
    def batch_tokenized_inputs(cls, requests, tokenizer) -> List[List[int]]:
        out = []
        cls._pending = []
        for r in requests:
            ids: List[int] = []
            images = []                                      # (first row position, patches, grid)
            chunks = list(r.input_chunks.chunks) if r.HasField("input_chunks") else []
            if not chunks:
                ids = list(tokenizer(r.inputs, truncation=False, add_special_tokens=r.add_special_tokens)["input_ids"])
            first_text = True
            for c in chunks:
                if c.WhichOneof("chunk") == "text":
                    ids.extend(tokenizer(c.text, truncation=False,
                                         add_special_tokens=r.add_special_tokens and first_text)["input_ids"])
                    first_text = False
                else:
                    patches, grid = preprocess_qwen_image(c.image.data, cls.patch, cls.merge, cls.temporal,
                                                          cls.min_pixels, cls.max_pixels)
                    n = grid[0] * grid[1] * grid[2] // (cls.merge ** 2)
                    if cls.vision_start_id is not None:
                        ids.append(cls.vision_start_id)
                    images.append((len(ids), patches, grid))
                    ids.extend([cls.image_token_id] * n)
                    if cls.vision_end_id is not None:
                        ids.append(cls.vision_end_id)
            if r.truncate and len(ids) > r.truncate:
                raise ValueError("`truncate` cannot be combined with image inputs of this model")
            out.append(ids)
            cls._pending.append(images)
        return out

    @classmethod
    def from_tokenized(cls, batch_pb, batch_tokenized_inputs, tokenizer, dtype, device, speculate: int = 0):
        batch = super().from_tokenized(batch_pb, batch_tokenized_inputs, tokenizer, dtype, device, speculate)
        pending = getattr(cls, "_pending", None) or [[] for _ in batch.seqs]
        for s, images in zip(batch.seqs, pending):
            s.images = images
            s.mrope_pos, s.pos_delta = cls.position_streams(len(s.ids), images, cls.merge)
        cls._pending = []
        return batch

    @staticmethod
    def position_streams(n_tokens: int, images, merge: int) -> Tuple[np.ndarray, int]:
        """``[3, n_tokens]`` (time, height, width) positions and the offset decode positions carry."""
        pos = np.zeros((3, n_tokens), dtype=np.int32)
        cur, t = 0, 0                                        # next position value, next token
        for start, _, (gt, gh, gw) in images:
            n = start - t
            pos[:, t:start] = cur + np.arange(n, dtype=np.int32)[None]
            cur += n
            lh, lw = gh // merge, gw // merge
            rows = gt * lh * lw
            idx = np.arange(rows)
            pos[0, start:start + rows] = cur + idx // (lh * lw)
            pos[1, start:start + rows] = cur + (idx // lw) % lh
            pos[2, start:start + rows] = cur + idx % lw
            cur += max(gt, lh, lw)
            t = start + rows
        n = n_tokens - t
        pos[:, t:] = cur + np.arange(n, dtype=np.int32)[None]
        cur += n
        return pos, cur - n_tokens


class Qwen2VlCausalLM(VlmCausalLM):
    def __init__(self, model, tower: Qwen2VisionTower, tokenizer, dtype, device, rank, world, image_token_id: int,
                 vision_start_id, vision_end_id, min_pixels: int, max_pixels: int, **kw):
        from .flash_causal_lm import FlashCausalLM

        FlashCausalLM.__init__(self, model, tokenizer, dtype, device, rank, world, **kw)
        self.tower = tower
        self.image_token_id = image_token_id
        self.batch_cls = type("BoundQwen2VlBatch", (Qwen2VlBatch,), dict(
            image_token_id=image_token_id, vision_start_id=vision_start_id, vision_end_id=vision_end_id,
            patch=tower.patch, merge=tower.merge, temporal=tower.temporal, min_pixels=min_pixels,
            max_pixels=max_pixels))

    def build_meta(self, batch, counts):
        from .flash_causal_lm import FlashCausalLM

        meta, row_owner = FlashCausalLM.build_meta(self, batch, counts)
        if not any(s.prefilling and n > 0 for s, n in zip(batch.seqs, counts)):
            return meta, row_owner                           # decode: scalar positions (+ pos_delta) suffice
        T = sum(counts)
        pos3 = np.zeros((3, T), dtype=np.int64)
        jobs = []                                            # (row, rows, image key, offset inside the image)
        uniq: Dict[int, Tuple[torch.Tensor, Tuple[int, int, int]]] = {}
        t = 0
        for s, n in zip(batch.seqs, counts):
            if n == 0:
                continue
            if s.prefilling:
                lo, hi = s.cache_len, s.cache_len + n
                pos3[:, t:t + n] = s.mrope_pos[:, lo:hi]
                for start, patches, grid in getattr(s, "images", []):
                    rows = grid[0] * grid[1] * grid[2] // (self.tower.merge ** 2)
                    a, b = max(start, lo), min(start + rows, hi)
                    if a < b:
                        uniq.setdefault(id(patches), (patches, grid))
                        jobs.append((t + a - lo, b - a, id(patches), a - start))
            else:
                p = len(s.ids) - 1 + getattr(s, "pos_delta", 0)
                pos3[:, t:t + n] = p + np.arange(n)[None]
            t += n
        rot = self.model.rotary
        meta.rope_cos_sin = rot.mrope_rows(torch.from_numpy(pos3).to(self.device))
        meta.rope_rows = torch.arange(T, dtype=torch.int32, device=self.device)
        if jobs:
            keys = list(uniq)
            feats = self.tower(torch.cat([uniq[k][0] for k in keys]).to(self.device), [uniq[k][1] for k in keys])
            merge2 = self.tower.merge ** 2
            starts = np.cumsum([0] + [uniq[k][1][0] * uniq[k][1][1] * uniq[k][1][2] // merge2 for k in keys]).tolist()
            base = {k: starts[i] for i, k in enumerate(keys)}
            embeds = self.model.embed_tokens(meta.input_ids, meta.positions).clone()
            for row, n, key, off in jobs:
                embeds[row:row + n] = feats[base[key] + off: base[key] + off + n].to(embeds.dtype)
            meta.inputs_embeds = embeds
        return meta, row_owner


def load_qwen2_vl(path, cfg, weights: Weights, comm, rank, world, dtype, device, tokenizer, speculate, kv_cache_dtype,
                  max_prefill_tokens):
    from . import resolve_kv_dtype
    from .decoder import CausalDecoder

    text_cfg = cfg.text_config()
    vis = dict(cfg.get("vision_config") or {})
    tower = Qwen2VisionTower(vis, weights, "model.visual", v25=cfg.model_type == "qwen2_5_vl")
    model = CausalDecoder(text_cfg, weights, comm=comm, prefix="model.language_model")
    if not model.rotary.mrope_section:
        raise ValueError("qwen2_vl checkpoints need `mrope_section` in their rope parameters")
    return Qwen2VlCausalLM(
        model, tower, tokenizer, dtype, device, rank, world, int(cfg.get("image_token_id", 151655)),
        cfg.get("vision_start_token_id"), cfg.get("vision_end_token_id"),
        int(vis.get("min_pixels", 56 * 56)), int(vis.get("max_pixels", 14 * 14 * 4 * 1280)),
        speculate=speculate, kv_cache_dtype=resolve_kv_dtype(kv_cache_dtype, dtype),
        max_prefill_tokens=max_prefill_tokens)
