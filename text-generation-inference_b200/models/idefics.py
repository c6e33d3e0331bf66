"""Idefics (v1, 9B / 80B): a Llama-1 decoder with gated cross-attention blocks over CLIP image features
(optionally through a perceiver resampler).

Reference: ``models/idefics_causal_lm.py`` (padded batches that carry ``pixel_values`` and an
``image_attention_mask``; the image states are computed in the first forward and reused afterwards) over the
modelling code in ``models/custom_modeling/idefics_*.py``.  As in the reference this family is not on the paged
fast path: the ``transformers`` module runs per request with its own cache (``models/padded.py``); what this file
adds is the multimodal part of the batch — image chunks become ``<fake_token_around_image><image>
<fake_token_around_image>``, every text position attends to the most recent image before it (none after an
end-of-sequence token until the next image), a request without images gets one blank image that nothing attends
to, and decode steps pass the cached image states instead of pixels.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..proto import generate_v3 as pb  # noqa: F401  (message types of the batch)
from ..utils.tokens import NextTokenChooser, StoppingCriteria
from .padded import PaddedBatch, PaddedCausalLM, PaddedSeq
from .vlm_causal_lm import CLIP_MEAN, CLIP_STD, preprocess_image


def image_attention_rows(ids: List[int], image_token_id: int, eos_ids, num_images: int) -> torch.Tensor:
    """``[len(ids), num_images]``: position t sees image j when j is the last image at or before t and no
    end-of-sequence token lies between them."""
    mask = torch.zeros(len(ids), max(1, num_images), dtype=torch.long)
    current, closed = -1, False
    for t, tok in enumerate(ids):
        if tok == image_token_id:
            current += 1
            closed = False
        if current >= 0 and not closed and current < num_images:
            mask[t, current] = 1
        if tok in eos_ids:
            closed = True
    return mask


class IdeficsBatch(PaddedBatch):
    image_token_id = 32001
    fake_token_id = 32000
    image_size = 224

    @classmethod
    def from_pb(cls, batch_pb, tokenizer, dtype, device, speculate: int = 0) -> "IdeficsBatch":
        seqs, params = [], []
        for r in batch_pb.requests:
            ids: List[int] = []
            images: List[torch.Tensor] = []
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
                    images.append(preprocess_image(c.image.data, cls.image_size, CLIP_MEAN, CLIP_STD))
                    ids.extend([cls.fake_token_id, cls.image_token_id, cls.fake_token_id])
            if r.truncate and len(ids) > r.truncate:
                if images:
                    raise ValueError("truncation would cut through an image; raise `truncate` or shorten the prompt")
                ids = ids[-r.truncate:]
            s = PaddedSeq(r, ids, len(ids), StoppingCriteria.from_pb(r.stopping_parameters, tokenizer),
                          int(r.top_n_tokens), max(0, len(ids) - 5), len(ids))
            s.images = images
            s.image_states = None
            seqs.append(s)
            params.append(r.parameters)
        return cls(batch_pb.id, seqs, NextTokenChooser.from_pb(params, device, tokenizer), device)


class IdeficsCausalLM(PaddedCausalLM):
    def __init__(self, hf_model, tokenizer, dtype, device, rank=0, world_size=1, eos_token_ids=None):
        super().__init__(hf_model, tokenizer, dtype, device, rank, world_size, eos_token_ids)
        cfg = hf_model.config
        self.use_resampler = bool(getattr(cfg, "use_resampler", False))
        vocab = int(cfg.vocab_size)
        image_id = fake_id = None
        if hasattr(tokenizer, "convert_tokens_to_ids"):
            try:
                image_id = tokenizer.convert_tokens_to_ids("<image>")
                fake_id = tokenizer.convert_tokens_to_ids("<fake_token_around_image>")
            except Exception:  # noqa: BLE001
                image_id = fake_id = None
        unk = getattr(tokenizer, "unk_token_id", None)
        if image_id is None or image_id == unk or image_id < 0:
            fake_id, image_id = vocab, vocab + 1          # the two additional vocabulary entries
        self.eos_set = set(eos_token_ids or [])
        self.batch_cls = type("BoundIdeficsBatch", (IdeficsBatch,), dict(
            image_token_id=int(image_id), fake_token_id=int(fake_id), image_size=int(cfg.vision_config.image_size)))

    @property
    def batch_type(self):
        return self.batch_cls

    @torch.no_grad()
    def _step(self, s: PaddedSeq) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        dev = self.device
        n_img = len(s.images)
        rows = image_attention_rows(s.ids, self.batch_cls.image_token_id, self.eos_set, n_img).to(dev)
        if not s.prefilled:
            size = self.batch_cls.image_size
            pixels = (torch.stack(s.images) if n_img else torch.zeros(1, 3, size, size)).unsqueeze(0)
            ids = torch.tensor([s.ids], dtype=torch.long, device=dev)
            out = self.hf(input_ids=ids, pixel_values=pixels.to(dev, self.dtype), image_attention_mask=rows.unsqueeze(0),
                          use_cache=True)
            s.image_states = out.image_hidden_states
            s.prefilled = True
            prompt_logits = out.logits[0]
        else:
            ids = torch.tensor([[s.ids[-1]]], dtype=torch.long, device=dev)
            key = "perceiver_embeddings" if self.use_resampler else "image_encoder_embeddings"
            out = self.hf(input_ids=ids, past_key_values=s.cache, image_attention_mask=rows[-1:].unsqueeze(0),
                          use_cache=True, **{key: s.image_states})
            prompt_logits = None
        s.cache = out.past_key_values
        return out.logits[0, -1], prompt_logits


def load_idefics(path, cfg, process_group, rank: int, world: int, dtype, device, tokenizer):
    if world > 1:
        raise NotImplementedError("the Idefics runner is not sharded: run it on one GPU")
    import transformers

    hf_cfg = transformers.AutoConfig.from_pretrained(str(path))
    model = transformers.IdeficsForVisionText2Text.from_pretrained(str(path), torch_dtype=dtype).to(device)
    if not hasattr(tokenizer, "decode"):
        tokenizer = transformers.AutoTokenizer.from_pretrained(str(path))
    eos = getattr(hf_cfg, "eos_token_id", None)
    eos_ids = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else None)
    return IdeficsCausalLM(model, tokenizer, dtype, device, rank, world, eos_ids)
