"""Llama-3.2-Vision shape (mllama) on CPU against transformers: tiled vision tower, projector, cross-attention
layers with gates and per-head q / k norms, sequences with and without an image in one batch, greedy generation
through prefill and decode (cross keys / values cached per sequence) must agree."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _png, _request  # noqa: E402

IMG = 299


def _build(tmp):
    torch.manual_seed(0)
    vis = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_global_layers=2, attention_heads=4,
               image_size=28, patch_size=14, max_num_tiles=4, intermediate_layers_indices=[0, 1],
               vision_output_dim=96, supported_aspect_ratios=[[1, 1], [1, 2], [1, 3], [1, 4], [2, 1], [2, 2], [3, 1], [4, 1]])
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=IMG + 1 - 8, max_position_embeddings=512, cross_attention_layers=[1, 3], tie_word_embeddings=False,
               rope_scaling=None, rope_theta=10000.0, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    cfg = transformers.MllamaConfig(vision_config=vis, text_config=txt, image_token_index=IMG)
    hf = transformers.MllamaForConditionalGeneration(cfg).eval()
    with torch.no_grad():      # gates start at zero: open them so that the cross layers matter
        for name, p in hf.named_parameters():
            if name.endswith("_gate") or "gate_attn" in name or "gate_ffn" in name or name.endswith(".gate"):
                p.fill_(0.7)
    hf.save_pretrained(str(tmp), safe_serialization=True)
    (tmp / "preprocessor_config.json").write_text(json.dumps({
        "size": {"height": 28, "width": 28}, "max_image_tiles": 4, "image_mean": [0.5, 0.5, 0.5],
        "image_std": [0.5, 0.5, 0.5]}))
    return hf


def test_mllama_generation_matches_transformers(tmp_path):
    from transformers.models.mllama.image_processing_mllama import MllamaImageProcessor
    from PIL import Image
    import io

    hf = _build(tmp_path)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    png = _png(3)
    reqs = [
        _request(0, [("image", png), ("text", "abc def")], 5, range(1, 4)),
        _request(1, [("text", "no picture here")], 5, range(4, 7)),
    ]
    model.init_kv_cache(10)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=2), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    assert prompts[0].count(IMG) == 1 and prompts[1].count(IMG) == 0
    got = {0: [], 1: []}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)

    proc = MllamaImageProcessor(size={"height": 28, "width": 28}, max_image_tiles=4, image_mean=[0.5] * 3,
                                image_std=[0.5] * 3)
    feats = proc(images=[[Image.open(io.BytesIO(png)).convert("RGB")]], return_tensors="pt")
    ids = torch.tensor([prompts[0]])
    # every text row sees every real tile of the image (what the serving path implements)
    cam = feats["aspect_ratio_mask"][:, None, :, :].expand(1, ids.shape[1], -1, -1).clone()
    with torch.no_grad():
        ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=feats["pixel_values"],
                          aspect_ratio_ids=feats["aspect_ratio_ids"], aspect_ratio_mask=feats["aspect_ratio_mask"],
                          cross_attention_mask=cam, max_new_tokens=5, min_new_tokens=5, do_sample=False)
        ids1 = torch.tensor([prompts[1]])
        ref1 = hf.generate(input_ids=ids1, attention_mask=torch.ones_like(ids1), max_new_tokens=5, min_new_tokens=5,
                           do_sample=False)
    assert got[0][:5] == ref[0, ids.shape[1]:].tolist(), (got[0], ref[0, ids.shape[1]:].tolist())
    assert got[1][:5] == ref1[0, ids1.shape[1]:].tolist(), (got[1], ref1[0, ids1.shape[1]:].tolist())
