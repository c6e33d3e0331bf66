"""Idefics2 (perceiver resampler) and Idefics3 (pixel-shuffle connector) on CPU against transformers: the
global view of the image goes through the tower and the connector, lands on the placeholder rows, and
greedy generation must agree."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.vlm_causal_lm import SIGLIP_MEAN, SIGLIP_STD, preprocess_image  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _png, _request  # noqa: E402

VIS = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28,
           patch_size=7)
TXT = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           vocab_size=300, max_position_embeddings=512, tie_word_embeddings=False)


def _build(kind, tmp):
    torch.manual_seed(0)
    if kind == "idefics3":
        cfg = transformers.Idefics3Config(vision_config=VIS, text_config=dict(TXT, model_type="llama"),
                                          image_token_id=299, scale_factor=2)
        hf = transformers.Idefics3ForConditionalGeneration(cfg)
    else:
        cfg = transformers.Idefics2Config(
            vision_config=VIS, text_config=dict(TXT, model_type="mistral", sliding_window=None), image_token_id=299,
            perceiver_config=dict(resampler_n_latents=4, resampler_depth=2, resampler_n_heads=2, resampler_head_dim=16,
                                  num_key_value_heads=1, hidden_act="silu", hidden_size=64, rms_norm_eps=1e-6))
        hf = transformers.Idefics2ForConditionalGeneration(cfg)
    hf = hf.eval()
    hf.save_pretrained(str(tmp), safe_serialization=True)
    c = json.loads((tmp / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp / "config.json").write_text(json.dumps(c))
    return hf


@pytest.mark.parametrize("kind,tokens", [("idefics3", 4), ("idefics2", 4)])
def test_idefics_generation_matches_transformers(tmp_path, kind, tokens):
    hf = _build(kind, tmp_path)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert model.tokens_per_image == tokens
    png1, png2 = _png(1), _png(2)
    reqs = [
        _request(0, [("text", "ab"), ("image", png1), ("text", "cde")], 6, range(1, 4)),
        _request(1, [("image", png2), ("text", "xy"), ("image", png1)], 6, range(4, 8)),
    ]
    model.init_kv_cache(12)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=2), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    assert prompts[0].count(299) == tokens and prompts[1].count(299) == 2 * tokens
    got = {0: [], 1: []}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    images = {0: [png1], 1: [png2, png1]}
    for i in range(2):
        ids = torch.tensor([prompts[i]])
        px = torch.stack([preprocess_image(b, 28, SIGLIP_MEAN, SIGLIP_STD) for b in images[i]]).unsqueeze(0)
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=px,
                              pixel_attention_mask=torch.ones(1, px.shape[1], 28, 28, dtype=torch.long),
                              max_new_tokens=6, min_new_tokens=6, do_sample=False)
        assert got[i][:6] == ref[0, ids.shape[1]:].tolist(), (kind, i, got[i], ref[0, ids.shape[1]:].tolist())
