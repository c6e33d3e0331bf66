"""Idefics v1 shape on CPU against the transformers module driven step by step without a cache: gated
cross-attention over perceiver latents, the image attention rows (most recent image; nothing for a request without
images), decode on cached image states."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.idefics import image_attention_rows  # noqa: E402
from tgi_b200.models.vlm_causal_lm import CLIP_MEAN, CLIP_STD, preprocess_image  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _png, _request  # noqa: E402


def _build(tmp):
    torch.manual_seed(0)
    cfg = transformers.IdeficsConfig(
        vocab_size=300, additional_vocab_size=2, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
        num_attention_heads=4, cross_layer_interval=2, max_position_embeddings=256, use_resampler=True,
        vision_config=dict(embed_dim=32, image_size=28, patch_size=14, num_hidden_layers=2, num_attention_heads=4,
                           intermediate_size=64),
        perceiver_config=dict(use_resampler=True, resampler_n_latents=4, resampler_depth=2, resampler_n_heads=2,
                              resampler_head_dim=16),
        pad_token_id=0, bos_token_id=1, eos_token_id=2, tie_word_embeddings=False)
    hf = transformers.IdeficsForVisionText2Text(cfg).eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if "alpha_cross_attn" in name or "alpha_dense" in name:
                p.fill_(0.8)
    hf.save_pretrained(str(tmp), safe_serialization=True)
    return hf


def test_image_attention_rows():
    rows = image_attention_rows([5, 301, 7, 8, 2, 9, 301, 4], 301, {2}, 2)
    assert rows.tolist() == [[0, 0], [1, 0], [1, 0], [1, 0], [1, 0], [0, 0], [0, 1], [0, 1]]


def test_idefics_v1_generation_matches_transformers(tmp_path):
    hf = _build(tmp_path)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    png = _png(4)
    reqs = [_request(0, [("text", "ab"), ("image", png), ("text", "cd e")], 5, range(1, 3)),
            _request(1, [("text", "plain text")], 5, range(3, 5))]
    model.init_kv_cache(8)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=2), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    img_id = model.batch_type.image_token_id
    assert prompts[0].count(img_id) == 1 and prompts[1].count(img_id) == 0
    got = {0: [], 1: []}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    px = {0: preprocess_image(png, 28, CLIP_MEAN, CLIP_STD)[None, None], 1: torch.zeros(1, 1, 3, 28, 28)}
    for i in range(2):
        ids = list(prompts[i])
        out = []
        for _ in range(5):
            rows = image_attention_rows(ids, img_id, {2}, 1 if i == 0 else 0)
            with torch.no_grad():
                logits = hf(input_ids=torch.tensor([ids]), pixel_values=px[i], image_attention_mask=rows[None],
                            use_cache=False).logits
            tok = int(logits[0, -1].argmax())
            out.append(tok)
            ids.append(tok)
        assert got[i][:5] == out, (i, got[i], out)
