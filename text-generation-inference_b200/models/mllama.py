"""Llama-3.2-Vision (``mllama``): a Llama decoder whose layers listed in ``cross_attention_layers`` attend to the
states of a tiled vision transformer instead of to the text.

Reference: ``models/mllama_causal_lm.py`` (batch with image payloads, cross states per request) and
``models/custom_modeling/mllama.py:622-886`` (cross-attention layer: normalised q / k per head, ``tanh`` gates on the
attention and MLP branches, rows of sequences without an image pass through unchanged), ``:407-620`` (vision
model), ``:913-1043`` (wiring).  Like the reference, every text row of a sequence sees all image tiles of that
sequence (the per-token tile mask of the original implementation is not applied); tiles that are only padding of
the aspect-ratio canvas are left out of the cross states.

Division of work here: the self-attention layers, MLPs, embeddings and head are the generic paged decoder
(``models/decoder.py``, architecture ``llama``); ``CrossAttentionLayer`` takes the place of a decoder layer; the
vision tower runs once per image through the ``transformers`` module (it is not on the decode path); keys and
values of the cross layers are projected once per sequence and kept on its ``Seq`` until it leaves the batch.
"""
from __future__ import annotations

import io
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .decoder import CausalDecoder, DenseMLP, Norm
from .flash_causal_lm import FlashCausalLM
from .layers import FastLinear
from .vlm_causal_lm import VlmCausalLMBatch


@dataclass
class CrossInfo:
    """Rows of a step that belong to sequences with images: ``rows`` indexes the ragged batch, ``segments`` are
    ``(begin, end, seq)`` ranges inside ``rows``."""

    rows: torch.Tensor
    segments: List[Tuple[int, int, object]]


def _head_rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class _NoCache:
    """Stands where a self-attention module would be: the cross layers write nothing into the paged KV cache."""

    k_scale = None
    v_scale = None


class CrossAttentionLayer:
    fusable_tp = False
    attn_in_quant = False
    mlp_in_quant = False

    def __init__(self, arch, cfg, dims, prefix: str, weights, idx: int, comm):
        from ..utils.quantization import DefaultWeightsLoader

        self.idx, self.dims, self.pg, self.comm = idx, dims, weights.process_group, comm
        self.eps = dims.eps
        self.head_dim = dims.head_dim
        self.num_heads, self.num_kv = dims.num_heads, dims.num_kv_heads          # per rank
        self.norm1 = Norm.load(arch, f"{prefix}.input_layernorm", weights, dims.eps)
        self.norm2 = Norm.load(arch, f"{prefix}.post_attention_layernorm", weights, dims.eps)
        p = f"{prefix}.cross_attn"
        with weights.use_loader(DefaultWeightsLoader()):
            self.q_proj = FastLinear(weights.get_sharded(f"{p}.q_proj.weight", dim=0))
            self.k_proj = FastLinear(weights.get_sharded(f"{p}.k_proj.weight", dim=0))
            self.v_proj = FastLinear(weights.get_sharded(f"{p}.v_proj.weight", dim=0))
            self.o_proj = FastLinear(weights.get_sharded(f"{p}.o_proj.weight", dim=1))
            self.q_norm = weights.get_tensor(f"{p}.q_norm.weight")
            self.k_norm = weights.get_tensor(f"{p}.k_norm.weight")
            self.attn_gate = weights.get_tensor(f"{prefix}.cross_attn_attn_gate").float().tanh().to(weights.dtype)
            self.mlp_gate = weights.get_tensor(f"{prefix}.cross_attn_mlp_gate").float().tanh().to(weights.dtype)
        self.mlp = DenseMLP(arch, cfg, dims, prefix, weights, comm, idx)
        self.attn = _NoCache()

    def cross_kv(self, seq) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[1, kv_heads, Nv, D]`` keys (normalised per head) and values of the sequence's image states."""
        cache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = seq.cross_kv
        if self.idx not in cache:
            states = seq.cross_states                                     # [Nv, hidden]
            k = self.k_proj(states).view(-1, self.num_kv, self.head_dim)
            v = self.v_proj(states).view(-1, self.num_kv, self.head_dim)
            k = _head_rms(k, self.k_norm, self.eps)
            cache[self.idx] = (k.transpose(0, 1).unsqueeze(0).contiguous(), v.transpose(0, 1).unsqueeze(0).contiguous())
        return cache[self.idx]

    def __call__(self, h, residual, meta, rotary, kv):
        normed, residual = self.norm1(h, residual)
        cross: Optional[CrossInfo] = getattr(meta, "cross", None)
        out = torch.zeros_like(normed)
        if cross is None or not cross.segments:
            return out, residual                # no image in this step: the layer is the identity
        x = normed.index_select(0, cross.rows)
        q = _head_rms(self.q_proj(x).view(-1, self.num_heads, self.head_dim), self.q_norm, self.eps)
        attn = torch.empty_like(q)
        rep = self.num_heads // self.num_kv
        for a, b, seq in cross.segments:
            k, v = self.cross_kv(seq)
            if rep > 1:
                k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1).unsqueeze(0), k, v)     # [1, heads, n, D]
            attn[a:b] = o.squeeze(0).transpose(0, 1)
        attn = self.o_proj(attn.reshape(-1, self.num_heads * self.head_dim))
        if self.pg.size() > 1:
            if self.comm is not None:
                attn = self.comm.all_reduce(attn)
            else:
                torch.distributed.all_reduce(attn, group=self.pg)
        attn = attn * self.attn_gate
        hidden = residual.index_select(0, cross.rows) + attn
        mlp_in, _ = self.norm2(hidden, None)
        delta = attn + self.mlp(mlp_in) * self.mlp_gate
        out.index_copy_(0, cross.rows, delta.to(out.dtype))
        return out, residual


class MllamaVision:
    """Tiled vision transformer + projector: images of one sequence -> ``[tiles * patches, hidden_text]``."""

    def __init__(self, cfg, weights, path, dtype, device):
        from transformers import MllamaConfig
        from transformers.models.mllama.image_processing_mllama import MllamaImageProcessor
        from transformers.models.mllama.modeling_mllama import MllamaVisionModel

        hf = MllamaConfig(**{k: v for k, v in cfg.to_dict().items() if k in ("vision_config", "text_config")})
        self.vcfg = hf.vision_config
        with torch.device("meta"):
            tower = MllamaVisionModel(self.vcfg)
        tower = tower.to_empty(device=device).to(dtype)
        state = {}
        for name, ref in tower.state_dict().items():
            t = weights.get_tensor(f"vision_model.{name}")
            state[name] = t.to(ref.dtype).reshape(ref.shape)
        tower.load_state_dict(state, strict=True)
        self.tower = tower.eval()
        self.proj_w = weights.get_tensor("multi_modal_projector.weight")
        self.proj_b = weights.get_tensor("multi_modal_projector.bias")
        self.dtype, self.device = dtype, device
        import json
        import os

        pp = os.path.join(str(path), "preprocessor_config.json")
        kw = {}
        if os.path.exists(pp):
            raw = json.load(open(pp))
            kw = {k: raw[k] for k in ("size", "max_image_tiles", "image_mean", "image_std", "do_rescale", "rescale_factor",
                                      "do_normalize", "do_pad", "do_resize", "do_convert_rgb", "resample") if k in raw}
        kw.setdefault("size", {"height": self.vcfg.image_size, "width": self.vcfg.image_size})
        kw.setdefault("max_image_tiles", self.vcfg.max_num_tiles)
        self.processor = MllamaImageProcessor(**kw)

    @torch.no_grad()
    def __call__(self, images: List[bytes]) -> torch.Tensor:
        from PIL import Image

        pil = [Image.open(io.BytesIO(b)).convert("RGB") for b in images]
        feats = self.processor(images=[pil], return_tensors="pt")
        mask = feats["aspect_ratio_mask"].to(self.device)                         # [1, images, max_tiles]
        out = self.tower(pixel_values=feats["pixel_values"].to(self.device, self.dtype),
                         aspect_ratio_ids=feats["aspect_ratio_ids"].to(self.device),
                         aspect_ratio_mask=mask).last_hidden_state                 # [1, images, tiles, patches, dim]
        states = F.linear(out.to(self.dtype), self.proj_w, self.proj_b)
        keep = mask.bool().view(-1)                                                # real tiles only
        return states.reshape(-1, states.shape[-2], states.shape[-1])[keep].reshape(-1, states.shape[-1])


class MllamaBatch(VlmCausalLMBatch):
    """One ``<|image|>`` token per image; the payload is the encoded image itself (tiling depends on its shape)."""

    @classmethod
    def image_payload(cls, data: bytes):
        return data, 1


class MllamaCausalLM(FlashCausalLM):
    def __init__(self, model: CausalDecoder, vision: MllamaVision, tokenizer, dtype, device, rank, world,
                 image_token_id: int, **kw):
        super().__init__(model, tokenizer, dtype, device, rank, world, **kw)
        self.vision = vision
        self.batch_cls = type("BoundMllamaBatch", (MllamaBatch,), dict(image_token_id=image_token_id))

    @property
    def batch_type(self):
        return self.batch_cls

    def graph_eligible(self, batch) -> bool:
        # the cross layers of a sequence with images run per sequence (ragged image lengths): eager steps
        return not any(getattr(s, "images", None) for s in batch.seqs)

    def build_meta(self, batch, counts):
        meta, row_owner = super().build_meta(batch, counts)
        rows: List[int] = []
        segments: List[Tuple[int, int, object]] = []
        t = 0
        for s, n in zip(batch.seqs, counts):
            if n > 0 and getattr(s, "images", None):
                if not hasattr(s, "cross_states"):
                    s.cross_states = self.vision([payload for _, payload, _ in s.images])
                    s.cross_kv = {}
                segments.append((len(rows), len(rows) + n, s))
                rows.extend(range(t, t + n))
            t += n
        if segments:
            meta.cross = CrossInfo(torch.tensor(rows, dtype=torch.long, device=self.device), segments)
        return meta, row_owner


def load_mllama(path, cfg, loader, process_group, rank, world, dtype, device, tokenizer, speculate, kv_cache_dtype,
                max_prefill_tokens):
    from . import resolve_kv_dtype
    from ..parallel.peer import make_comm
    from ..utils.weights import Weights, weight_files
    from .arch import ModelConfig

    # the language model is published under `language_model.model.*`, `model.language_model.*` or (recent
    # transformers) `model.language_model.model.*`
    renames = [("model.", "language_model.model."), ("model.", "model.language_model."),
               ("model.", "model.language_model.model."),
               ("lm_head", "language_model.lm_head"),
               ("vision_model.", "model.vision_model."), ("multi_modal_projector.", "model.multi_modal_projector.")]
    weights = Weights(weight_files(path), device, dtype, process_group=process_group, loader=loader, renames=renames)
    text = dict(cfg.text_config().to_dict())
    text["model_type"] = "llama"                    # the self-attention layers are Llama layers
    tcfg = ModelConfig(text)
    comm = make_comm(process_group, rank, world, device, tcfg.hidden_size, max_prefill_tokens or 4096) if world > 1 else None
    model = CausalDecoder(tcfg, weights, comm=comm)
    vision = MllamaVision(cfg, weights, path, dtype, device)
    image_token = int(cfg.get("image_token_index", cfg.get("image_token_id", 128256)))
    return MllamaCausalLM(model, vision, tokenizer, dtype, device, rank, world, image_token,
                          kv_cache_dtype=resolve_kv_dtype(kv_cache_dtype, dtype), speculate=speculate,
                          max_prefill_tokens=max_prefill_tokens)
