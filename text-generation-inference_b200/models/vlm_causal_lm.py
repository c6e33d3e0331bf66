"""Vision-language runner: image chunks -> vision tower -> projector -> rows of ``inputs_embeds``.

Reference: ``models/vlm_causal_lm.py:301-1133`` (batch with image inputs, image-token expansion,
encoder-output scatter), the vision towers ``custom_modeling/{clip,siglip}.py`` and the projectors of
``llava_next.py`` / ``flash_pali_gemma_modeling.py``.

A request's input is a list of chunks (text or image bytes).  Tokenisation replaces every image by
``n`` copies of the model's image token, where ``n`` is the number of feature rows the vision side
produces for one image.  At prefill the images of the chunk being processed are encoded (one ViT
forward per step for all of them), projected to the text hidden size and written over the
embeddings of the placeholder rows; the language model then runs on ``inputs_embeds`` unchanged
(same paged attention, same CUDA-graph decode, since decode steps never contain image rows).

Covered families: LLaVA-style (CLIP tower, 2-layer MLP projector, optional class-token drop; LLaVA-NeXT
with its any-resolution tiling in ``models/llava_next.py``), PaliGemma-style (SigLIP tower, linear projector, embedding
scale), Idefics2 (SigLIP-style tower, gated-MLP projection and a perceiver resampler that compresses
an image to a fixed number of latents; ``custom_modeling/idefics2.py``) and Idefics3 / SmolVLM
(pixel-shuffle connector; ``custom_modeling/idefics3.py``) and Gemma-3 (SigLIP tower, average-pooled
to ``mm_tokens_per_image`` rows, RMSNorm and a projection matrix; the rows of one image attend to each
other in both directions, which the attention kernels get as a per-row horizon;
``custom_modeling/flash_gemma3_modeling.py``).  The Idefics families run on the global
view of an image (the square resize to the tower's resolution); the sub-image tiling their
processors can add is not produced.  Towers are plain pre-norm ViTs evaluated with ``F.scaled_dot_product_attention``: the image
side is compute-light next to the decoder and runs once per request.
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..utils.weights import Weights, weight_files
from .decoder import CausalDecoder
from .flash_causal_lm import FlashCausalLM, FlashCausalLMBatch

CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
SIGLIP_MEAN, SIGLIP_STD = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)


# ---- vision tower ------------------------------------------------------------------------------
class _VitLayer:
    def __init__(self, w: Weights, prefix: str, heads: int, eps: float, act: str):
        g = w.get_tensor
        self.ln1 = (g(f"{prefix}.layer_norm1.weight"), g(f"{prefix}.layer_norm1.bias"))
        self.ln2 = (g(f"{prefix}.layer_norm2.weight"), g(f"{prefix}.layer_norm2.bias"))
        a = f"{prefix}.self_attn"
        self.qkv_w = torch.cat([g(f"{a}.q_proj.weight"), g(f"{a}.k_proj.weight"), g(f"{a}.v_proj.weight")], 0)
        self.qkv_b = torch.cat([g(f"{a}.q_proj.bias"), g(f"{a}.k_proj.bias"), g(f"{a}.v_proj.bias")], 0)
        self.o = (g(f"{a}.out_proj.weight"), g(f"{a}.out_proj.bias"))
        self.fc1 = (g(f"{prefix}.mlp.fc1.weight"), g(f"{prefix}.mlp.fc1.bias"))
        self.fc2 = (g(f"{prefix}.mlp.fc2.weight"), g(f"{prefix}.mlp.fc2.bias"))
        self.heads, self.eps, self.act = heads, eps, act

    def __call__(self, x: torch.Tensor) -> torch.Tensor:          # x [B, S, C]
        B, S, C = x.shape
        h = F.layer_norm(x, (C,), *self.ln1, self.eps)
        qkv = F.linear(h, self.qkv_w, self.qkv_b).view(B, S, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        attn = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2]).transpose(1, 2).reshape(B, S, C)
        x = x + F.linear(attn, *self.o)
        h = F.layer_norm(x, (C,), *self.ln2, self.eps)
        h = F.linear(h, *self.fc1)
        h = F.gelu(h, approximate="tanh") if self.act in ("gelu_pytorch_tanh", "gelu_fast", "gelu_new") else (
            h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else F.gelu(h))
        return x + F.linear(h, *self.fc2)


class VisionTower:
    """CLIP- or SigLIP-style ViT; returns the hidden states of layer ``feature_layer``."""

    def __init__(self, cfg: dict, w: Weights, prefix: str, kind: str, feature_layer: int = -1):
        self.kind = kind
        self.image_size, self.patch = int(cfg["image_size"]), int(cfg["patch_size"])
        self.hidden, heads = int(cfg["hidden_size"]), int(cfg["num_attention_heads"])
        eps = float(cfg.get("layer_norm_eps", 1e-5 if kind == "clip" else 1e-6))
        act = cfg.get("hidden_act", "quick_gelu" if kind == "clip" else "gelu_pytorch_tanh")
        e = f"{prefix}.embeddings"
        self.patch_w = w.get_tensor(f"{e}.patch_embedding.weight")
        self.patch_b = w.get_tensor(f"{e}.patch_embedding.bias") if w.has_tensor(f"{e}.patch_embedding.bias") else None
        self.pos = w.get_tensor(f"{e}.position_embedding.weight")
        self.cls = w.get_tensor(f"{e}.class_embedding") if kind == "clip" else None
        self.pre_ln = None
        if kind == "clip":
            name = "pre_layrnorm" if w.has_tensor(f"{prefix}.pre_layrnorm.weight") else "pre_layernorm"
            self.pre_ln = (w.get_tensor(f"{prefix}.{name}.weight"), w.get_tensor(f"{prefix}.{name}.bias"), eps)
        n_layers = int(cfg["num_hidden_layers"])
        use = n_layers + feature_layer + 1 if feature_layer < 0 else feature_layer
        self.layers = [_VitLayer(w, f"{prefix}.encoder.layers.{i}", heads, eps, act) for i in range(use)]
        self.post_ln = None
        if kind == "siglip" and use == n_layers and w.has_tensor(f"{prefix}.post_layernorm.weight"):
            self.post_ln = (w.get_tensor(f"{prefix}.post_layernorm.weight"), w.get_tensor(f"{prefix}.post_layernorm.bias"), eps)

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch) ** 2

    def __call__(self, pixels: torch.Tensor) -> torch.Tensor:       # [B, 3, S, S] -> [B, tokens, C]
        x = F.conv2d(pixels.to(self.patch_w.dtype), self.patch_w, self.patch_b, stride=self.patch)
        x = x.flatten(2).transpose(1, 2)
        if self.cls is not None:
            x = torch.cat([self.cls.view(1, 1, -1).expand(x.shape[0], -1, -1), x], dim=1)
        x = x + self.pos[: x.shape[1]].unsqueeze(0)
        if self.pre_ln is not None:
            x = F.layer_norm(x, (x.shape[-1],), *self.pre_ln)
        for layer in self.layers:
            x = layer(x)
        if self.post_ln is not None:
            x = F.layer_norm(x, (x.shape[-1],), *self.post_ln)
        return x


# ---- image preprocessing -------------------------------------------------------------------------
def preprocess_image(data: bytes, size: int, mean, std) -> torch.Tensor:
    """Decode, convert to RGB, resize to ``size`` x ``size`` (bicubic) and normalise: ``[3, size, size]``."""
    from PIL import Image

    img = Image.open(io.BytesIO(data)).convert("RGB").resize((size, size), Image.BICUBIC)
    arr = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
    m = torch.tensor(mean).view(3, 1, 1)
    s = torch.tensor(std).view(3, 1, 1)
    return (arr - m) / s


# ---- batch ---------------------------------------------------------------------------------------
class VlmCausalLMBatch(FlashCausalLMBatch):
    """Adds, per request, the decoded images and the prompt positions of their placeholder tokens."""

    image_token_id: int = 0
    image_start_id: Optional[int] = None      # tokens put around the placeholder rows (Gemma-3: begin / end of image)
    image_end_id: Optional[int] = None
    image_pad_ids: Tuple[int, ...] = ()       # tokens before the start and after the end token (Gemma-3: "\n\n")
    tokens_per_image: int = 0
    image_size: int = 224
    norm = (CLIP_MEAN, CLIP_STD)
    # PaliGemma: every text piece is "<bos>" + text + "\n" and is tokenised without further special tokens
    # (``models/vlm_causal_lm.py:194-197, 433-437`` of the reference); the newline separates prompt and answer
    text_wrap: Optional[Tuple[str, str]] = None

    @classmethod
    def image_payload(cls, data: bytes):
        """What the runner needs of one image, and the number of placeholder rows it takes in the prompt."""
        return preprocess_image(data, cls.image_size, *cls.norm), cls.tokens_per_image

    @classmethod
    def join_adjacent(cls, payload, rows: int):
        """Hook for layouts in which an image that directly follows another one shares a marker with it."""
        return payload, rows

    @classmethod
    def batch_tokenized_inputs(cls, requests, tokenizer) -> List[List[int]]:
        out = []
        cls._pending_images = []
        for r in requests:
            ids: List[int] = []
            images: List[Tuple[int, object, int]] = []      # (first placeholder position, payload, rows)
            chunks = list(r.input_chunks.chunks) if r.HasField("input_chunks") else []
            if not chunks:
                ids = list(tokenizer(r.inputs, truncation=False, add_special_tokens=r.add_special_tokens)["input_ids"])
            first_text = True
            after_image = False        # the previous chunk was an image (no text in between)
            for c in chunks:
                if c.WhichOneof("chunk") == "text":
                    after_image = after_image and not c.text
                    if cls.text_wrap is not None:
                        ids.extend(tokenizer(cls.text_wrap[0] + c.text + cls.text_wrap[1], truncation=False,
                                             add_special_tokens=False)["input_ids"])
                    else:
                        ids.extend(tokenizer(c.text, truncation=False,
                                             add_special_tokens=r.add_special_tokens and first_text)["input_ids"])
                    first_text = False
                else:
                    payload, rows = cls.image_payload(c.image.data)
                    if after_image:
                        payload, rows = cls.join_adjacent(payload, rows)
                    after_image = True
                    if cls.image_start_id is not None:
                        ids.extend(cls.image_pad_ids)
                        ids.append(cls.image_start_id)
                    images.append((len(ids), payload, rows))
                    ids.extend([cls.image_token_id] * rows)
                    if cls.image_end_id is not None:
                        ids.append(cls.image_end_id)
                        ids.extend(cls.image_pad_ids)
            if r.truncate and len(ids) > r.truncate:
                cut = len(ids) - r.truncate
                if any(pos < cut for pos, _, _ in images):
                    raise ValueError("truncation would cut through an image; raise `truncate` or shorten the prompt")
                ids = ids[cut:]
                images = [(pos - cut, px, rows) for pos, px, rows in images]
            out.append(ids)
            cls._pending_images.append(images)
        return out

    @classmethod
    def from_tokenized(cls, batch_pb, batch_tokenized_inputs, tokenizer, dtype, device, speculate: int = 0):
        batch = super().from_tokenized(batch_pb, batch_tokenized_inputs, tokenizer, dtype, device, speculate)
        pending = getattr(cls, "_pending_images", None) or [[] for _ in batch.seqs]
        for s, images in zip(batch.seqs, pending):
            s.images = images
        cls._pending_images = []
        return batch


class VlmCausalLM(FlashCausalLM):
    def __init__(self, model: CausalDecoder, tower: VisionTower, projector, tokenizer, dtype, device, rank, world,
                 image_token_id: int, drop_cls: bool, embed_scale: float = 1.0, image_wrap=(None, None),
                 bidirectional_images: bool = False, text_wrap=None, image_pad_ids=(), **kw):
        super().__init__(model, tokenizer, dtype, device, rank, world, **kw)
        self.bidirectional_images = bidirectional_images
        if bidirectional_images:
            # the rows of an image see each other: an image has to sit inside one prefill step
            self.support_chunking = False
            self.max_prefill_tokens = None
        self.tower, self.projector = tower, projector
        self.image_token_id, self.drop_cls, self.image_embed_scale = image_token_id, drop_cls, embed_scale
        self.tokens_per_image = projector.out_tokens(tower.num_patches)
        self.batch_cls = type("BoundVlmBatch", (VlmCausalLMBatch,), dict(
            image_token_id=image_token_id, tokens_per_image=self.tokens_per_image, image_size=tower.image_size,
            image_start_id=image_wrap[0], image_end_id=image_wrap[1], text_wrap=text_wrap,
            image_pad_ids=tuple(image_pad_ids),
            norm=(CLIP_MEAN, CLIP_STD) if tower.kind == "clip" else (SIGLIP_MEAN, SIGLIP_STD)))

    @property
    def batch_type(self):
        return self.batch_cls

    @torch.no_grad()
    def encode_images(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[N, 3, S, S]`` -> ``[N, tokens_per_image, hidden_text]``"""
        feats = self.tower(pixels.to(self.device))
        if self.drop_cls:
            feats = feats[:, 1:]
        out = self.projector(feats.to(self.dtype))
        if self.image_embed_scale != 1.0:
            out = out * self.image_embed_scale
        return out

    def image_features(self, payloads: list) -> List[torch.Tensor]:
        """Rows ``[rows_i, hidden_text]`` of every image of a step (one tower forward for all of them)."""
        return list(self.encode_images(torch.stack(payloads)))

    def build_meta(self, batch, counts):
        meta, row_owner = super().build_meta(batch, counts)
        # rows of this step that are image placeholders: (row in the ragged batch, image, offset)
        jobs: List[Tuple[int, int, torch.Tensor, int, int]] = []
        t = 0
        for s, n in zip(batch.seqs, counts):
            if s.prefilling and n > 0:
                lo, hi = s.cache_len, s.cache_len + n
                for pos, px, rows in getattr(s, "images", []):
                    a, b = max(pos, lo), min(pos + rows, hi)
                    if a < b:
                        jobs.append((t + a - lo, b - a, px, a - pos, id(px)))
            t += n
        if jobs and self.bidirectional_images:
            # horizon of every row of the step: its own position, or the last row of its image
            hz = meta.positions.clone()
            t = 0
            for s, n in zip(batch.seqs, counts):
                if s.prefilling and n > 0:
                    lo, hi = s.cache_len, s.cache_len + n
                    for pos, _, rows in getattr(s, "images", []):
                        a, b = max(pos, lo), min(pos + rows, hi)
                        if a < b:
                            hz[t + a - lo:t + b - lo] = pos + rows - 1
                t += n
            meta.attn_horizon = hz
        if jobs:
            uniq: Dict[int, int] = {}
            stack = []
            for _, _, px, _, key in jobs:
                if key not in uniq:
                    uniq[key] = len(stack)
                    stack.append(px)
            feats = self.image_features(stack)
            embeds = self.model.embed_tokens(meta.input_ids, meta.positions).clone()
            for row, n, _, off, key in jobs:
                embeds[row:row + n] = feats[uniq[key]][off:off + n].to(embeds.dtype)
            meta.inputs_embeds = embeds
        return meta, row_owner


class _MlpProjector:
    def __init__(self, w1, b1, w2, b2, act="gelu"):
        self.w1, self.b1, self.w2, self.b2, self.act = w1, b1, w2, b2, act

    def out_tokens(self, n: int) -> int:
        return n

    def __call__(self, x):                                   # [N, S, C] -> [N, S, H]
        N, S, C = x.shape
        h = ops.linear(x.reshape(N * S, C), self.w1, self.b1)
        h = F.gelu(h)
        return ops.linear(h, self.w2, self.b2).view(N, S, -1)


class _LinearProjector:
    def __init__(self, w, b):
        self.w, self.b = w, b

    def out_tokens(self, n: int) -> int:
        return n

    def __call__(self, x):
        N, S, C = x.shape
        return ops.linear(x.reshape(N * S, C), self.w, self.b).view(N, S, -1)


class _AvgPoolProjector:
    """Gemma-3: average-pool the patch grid to ``side x side`` rows, RMSNorm (unit offset), projection matrix."""

    def __init__(self, proj, norm_w, eps: float, side: int):
        self.proj, self.norm_w, self.eps, self.side = proj, norm_w, eps, int(side)

    def out_tokens(self, n: int) -> int:
        return self.side ** 2

    def __call__(self, x):                                   # [N, S, C] -> [N, side^2, H]
        N, S, C = x.shape
        grid = int(round(math.sqrt(S)))
        x = F.avg_pool2d(x.transpose(1, 2).reshape(N, C, grid, grid), grid // self.side)
        x = x.flatten(2).transpose(1, 2)
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.norm_w.float())
        return torch.matmul(v.to(x.dtype), self.proj)


class _PixelShuffleProjector:
    """Idefics3 connector: fold every ``scale x scale`` neighbourhood of patches into the channel dimension
    (row-major inside the neighbourhood), then one bias-free linear layer."""

    def __init__(self, w, scale: int):
        self.w, self.scale = w, int(scale)

    def out_tokens(self, n: int) -> int:
        return n // (self.scale ** 2)

    def __call__(self, x):
        N, S, C = x.shape
        side, f = int(round(math.sqrt(S))), self.scale
        x = x.view(N, side // f, f, side // f, f, C).permute(0, 1, 3, 2, 4, 5)      # [N, h', w', fh, fw, C]
        x = x.reshape(N * (side // f) ** 2, f * f * C)
        return ops.linear(x.contiguous(), self.w, None).view(N, (side // f) ** 2, -1)


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class _PerceiverProjector:
    """Idefics2 connector: gated MLP to the text width, then ``depth`` blocks in which a fixed set of
    latents attends (not causally) to the image rows and to itself."""

    def __init__(self, w: Weights, prefix: str, pcfg: dict, eps: float):
        g = w.get_tensor
        mp = f"{prefix}.modality_projection"
        self.mlp = (g(f"{mp}.gate_proj.weight"), g(f"{mp}.up_proj.weight"), g(f"{mp}.down_proj.weight"))
        rp = f"{prefix}.perceiver_resampler"
        self.latents = g(f"{rp}.latents")
        self.heads, self.kv_heads = int(pcfg.get("resampler_n_heads", 16)), int(pcfg.get("num_key_value_heads", 4))
        self.head_dim = int(pcfg.get("resampler_head_dim", 96))
        self.eps = eps
        self.layers = []
        for i in range(int(pcfg.get("resampler_depth", 3))):
            lp = f"{rp}.layers.{i}"
            self.layers.append(dict(
                ln_lat=g(f"{lp}.input_latents_norm.weight"), ln_ctx=g(f"{lp}.input_context_norm.weight"),
                q=g(f"{lp}.self_attn.q_proj.weight"), k=g(f"{lp}.self_attn.k_proj.weight"),
                v=g(f"{lp}.self_attn.v_proj.weight"), o=g(f"{lp}.self_attn.o_proj.weight"),
                ln_post=g(f"{lp}.post_attention_layernorm.weight"),
                mlp=(g(f"{lp}.mlp.gate_proj.weight"), g(f"{lp}.mlp.up_proj.weight"), g(f"{lp}.mlp.down_proj.weight"))))
        self.norm = g(f"{rp}.norm.weight")

    def out_tokens(self, n: int) -> int:
        return self.latents.shape[0]

    @staticmethod
    def _gated(x, mlp):
        return F.linear(F.silu(F.linear(x, mlp[0])) * F.linear(x, mlp[1]), mlp[2])

    def __call__(self, x):                                   # [N, S, C] -> [N, latents, H]
        ctx = self._gated(x, self.mlp)
        N = ctx.shape[0]
        lat = self.latents.to(ctx.dtype).unsqueeze(0).expand(N, -1, -1)
        L = lat.shape[1]
        for p in self.layers:
            hl, hc = _rms(lat, p["ln_lat"], self.eps), _rms(ctx, p["ln_ctx"], self.eps)
            kv_in = torch.cat([hc, hl], dim=1)
            q = F.linear(hl, p["q"]).view(N, L, self.heads, self.head_dim).transpose(1, 2)
            k = F.linear(kv_in, p["k"]).view(N, -1, self.kv_heads, self.head_dim).transpose(1, 2)
            v = F.linear(kv_in, p["v"]).view(N, -1, self.kv_heads, self.head_dim).transpose(1, 2)
            rep = self.heads // self.kv_heads
            a = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1))
            lat = lat + F.linear(a.transpose(1, 2).reshape(N, L, -1), p["o"])
            lat = lat + self._gated(_rms(lat, p["ln_post"], self.eps), p["mlp"])
        return _rms(lat, self.norm, self.eps)


def load_vlm(path, cfg, loader, process_group, rank, world, dtype, device, tokenizer, speculate, kv_cache_dtype,
             max_prefill_tokens):
    from . import resolve_kv_dtype
    from ..parallel.peer import make_comm

    mt = cfg.model_type
    # the same architectures are published with the language model under `language_model.model.*` or
    # `model.language_model.*`, and the Idefics text model has no inner `model.` level
    renames = [("language_model.model.", "model.language_model."), ("language_model.lm_head", "lm_head"),
               ("vision_tower.", "model.vision_tower."), ("multi_modal_projector.", "model.multi_modal_projector."),
               ("language_model.", "model.language_model."),       # Gemma-3 as saved by recent transformers
               ("model.text_model.model.", "model.text_model."),
               ("model.language_model.model.", "model.language_model."),
               # Qwen2-VL as first published: language model at the top level, tower under `visual.`
               ("model.language_model.model.", "model."), ("model.visual.", "visual.")]
    weights = Weights(weight_files(path), device, dtype, process_group=process_group, loader=loader, renames=renames)
    text_cfg = cfg.text_config()
    vis = dict(cfg.get("vision_config") or {})
    if mt in ("llava_next", "llava"):
        vis.setdefault("image_size", 336)
        vis.setdefault("patch_size", 14)
        tower = VisionTower(vis, weights, "vision_tower.vision_model", "clip",
                            feature_layer=int(cfg.get("vision_feature_layer", -2)))
        projector = _MlpProjector(weights.get_tensor("multi_modal_projector.linear_1.weight"),
                                  weights.get_tensor("multi_modal_projector.linear_1.bias"),
                                  weights.get_tensor("multi_modal_projector.linear_2.weight"),
                                  weights.get_tensor("multi_modal_projector.linear_2.bias"))
        drop_cls = cfg.get("vision_feature_select_strategy", "default") == "default"
        prefix, scale = "language_model", 1.0
        image_token = int(cfg.get("image_token_index", cfg.get("image_token_id", 32000)))
    elif mt == "paligemma":
        vis.setdefault("image_size", 224)
        vis.setdefault("patch_size", 14)
        tower = VisionTower(vis, weights, "vision_tower.vision_model", "siglip", feature_layer=-1)
        projector = _LinearProjector(weights.get_tensor("multi_modal_projector.linear.weight"),
                                     weights.get_tensor("multi_modal_projector.linear.bias"))
        drop_cls = False
        # Image rows are divided by sqrt(hidden) after the projector and every row of inputs_embeds is
        # multiplied by sqrt(hidden) at the entry of the Gemma decoder: the two cancel, and the
        # decoder here scales only the rows it embeds itself.
        prefix, scale = "language_model", 1.0
        image_token = int(cfg.get("image_token_index", 257152))
    elif mt in ("qwen2_vl", "qwen2_5_vl"):
        from .qwen2_vl import load_qwen2_vl

        hidden = int(text_cfg.get("hidden_size"))
        comm = make_comm(process_group, rank, world, device, hidden, int(max_prefill_tokens or 4096))
        runner = load_qwen2_vl(path, cfg, weights, comm, rank, world, dtype, device, tokenizer, speculate,
                               kv_cache_dtype, max_prefill_tokens)
        weights.close()
        return runner
    elif mt == "gemma3":
        vis.setdefault("image_size", 896)
        vis.setdefault("patch_size", 14)
        vis.setdefault("hidden_act", "gelu_pytorch_tanh")
        tower = VisionTower(vis, weights, "vision_tower.vision_model", "siglip", feature_layer=-1)
        side = int(round(math.sqrt(int(cfg.get("mm_tokens_per_image", 256)))))
        projector = _AvgPoolProjector(weights.get_tensor("multi_modal_projector.mm_input_projection_weight"),
                                      weights.get_tensor("multi_modal_projector.mm_soft_emb_norm.weight"),
                                      float(vis.get("layer_norm_eps", 1e-6)), side)
        drop_cls = False
        prefix, scale = "language_model", 1.0
        image_token = int(cfg.get("image_token_index", cfg.get("image_token_id", 262144)))
        extra = dict(image_wrap=(cfg.get("boi_token_index", cfg.get("boi_token_id")),
                                 cfg.get("eoi_token_index", cfg.get("eoi_token_id"))), bidirectional_images=True)
    elif mt in ("idefics2", "idefics3"):
        vis.setdefault("image_size", 364 if mt == "idefics3" else 980)
        vis.setdefault("patch_size", 14)
        vis.setdefault("hidden_act", "gelu_pytorch_tanh")
        tower = VisionTower(vis, weights, "model.vision_model", "siglip", feature_layer=-1)
        if mt == "idefics3":
            projector = _PixelShuffleProjector(weights.get_tensor("model.connector.modality_projection.proj.weight"),
                                               int(cfg.get("scale_factor", 2)))
        else:
            pcfg = dict(cfg.get("perceiver_config") or {})
            projector = _PerceiverProjector(weights, "model.connector", pcfg,
                                            float(pcfg.get("rms_norm_eps", text_cfg.get("rms_norm_eps", 1e-6))))
        drop_cls = False
        prefix, scale = "model.text_model", 1.0
        image_token = int(cfg.get("image_token_id", 32001 if mt == "idefics2" else 128257))
    else:
        raise NotImplementedError(f"vision-language model type {mt} has no native runner yet "
                                  "(llava / llava_next / paligemma / idefics2 / idefics3 are covered)")
    hidden = int(text_cfg.get("hidden_size"))
    comm = make_comm(process_group, rank, world, device, hidden, int(max_prefill_tokens or 4096))
    model = CausalDecoder(text_cfg, weights, comm=comm, prefix=prefix)
    runner_cls, extra_kw = VlmCausalLM, (extra if mt == "gemma3" else {})
    newline = next((n for n in ("image_newline", "model.image_newline") if weights.has_tensor(n)), None)
    if mt == "llava_next" and newline is not None and cfg.get("image_grid_pinpoints"):
        from .llava_next import LlavaNextCausalLM     # any-resolution tiling; without these weights: base view only

        runner_cls = LlavaNextCausalLM
        extra_kw = dict(image_newline=weights.get_tensor(newline), pinpoints=cfg.get("image_grid_pinpoints"))
    if mt == "idefics3":
        from .idefics3 import Idefics3CausalLM, processor_settings      # image splitting into tiles + global view

        longest, split = processor_settings(path, int(vis["image_size"]))
        runner_cls, extra_kw = Idefics3CausalLM, dict(longest_edge=longest, do_split=split)
    if mt == "gemma3" and hasattr(tokenizer, "convert_tokens_to_ids"):
        # the processor writes "\n\n<start_of_image>" ... "<end_of_image>\n\n" (reference: vlm_causal_lm.py:160-165)
        pad = list(tokenizer("\n\n", add_special_tokens=False)["input_ids"])
        if 0 < len(pad) <= 2:
            extra_kw = dict(extra_kw, image_pad_ids=pad)
    if mt == "paligemma":
        bos = getattr(tokenizer, "bos_token", None)
        if isinstance(bos, str) and bos:
            extra_kw = dict(extra_kw, text_wrap=(bos, "\n"))
    if mt == "idefics2":
        from .idefics2 import Idefics2CausalLM, processor_split_setting    # markers around images, optional 5-way split

        runner_cls, extra_kw = Idefics2CausalLM, dict(do_split=processor_split_setting(path))
    runner = runner_cls(model, tower, projector, tokenizer, dtype, device, rank, world, image_token, drop_cls,
                         scale, speculate=speculate, **extra_kw,
                         kv_cache_dtype=resolve_kv_dtype(kv_cache_dtype, dtype), max_prefill_tokens=max_prefill_tokens)
    weights.close()
    return runner
