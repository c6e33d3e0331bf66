"""LLaVA-NeXT any-resolution images on CPU against transformers: best-resolution choice, tiling, un-padding of
the tile map, newline rows, and a prompt whose number of image rows depends on the image size."""
import io
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.llava_next import anyres_rows, anyres_views, select_best_resolution  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _request  # noqa: E402

PINS = [[28, 56], [56, 28], [56, 56], [84, 28], [28, 84]]


def _png(seed, h, w):
    from PIL import Image

    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 255, size=(h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


@pytest.fixture(scope="module")
def llava_next(tmp_path_factory):
    torch.manual_seed(0)
    vis = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                        image_size=28, patch_size=7)
    txt = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=300, max_position_embeddings=1024,
                                   tie_word_embeddings=False)
    cfg = transformers.LlavaNextConfig(vision_config=vis, text_config=txt, image_token_index=299, vision_feature_layer=-2,
                                       vision_feature_select_strategy="default", image_grid_pinpoints=PINS)
    hf = transformers.LlavaNextForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        hf.model.image_newline.normal_()
    d = tmp_path_factory.mktemp("llava_next")
    hf.save_pretrained(str(d), safe_serialization=True)
    return hf, d


def test_best_resolution_matches_transformers():
    from transformers.image_processing_utils import select_best_resolution as ref

    for size in [(40, 52), (52, 40), (100, 30), (30, 100), (56, 56), (500, 499), (13, 200)]:
        assert select_best_resolution(size, PINS) == tuple(ref(size, [tuple(p) for p in PINS])), size


def test_llava_next_generation_matches_transformers(llava_next):
    hf, d = llava_next
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"))
    assert type(model).__name__ == "LlavaNextCausalLM" and model.side == 4
    wide, tall, square = _png(1, 30, 100), _png(2, 70, 40), _png(3, 50, 50)
    reqs = [
        _request(0, [("text", "ab"), ("image", wide), ("text", "cde")], 5, range(1, 12)),
        _request(1, [("image", tall), ("text", "xy"), ("image", square)], 5, range(12, 30)),
    ]
    model.init_kv_cache(32)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=2), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    rows = {k: anyres_rows(sz, PINS, 28, 4) for k, sz in {"wide": (30, 100), "tall": (70, 40), "square": (50, 50)}.items()}
    assert prompts[0].count(299) == rows["wide"] and prompts[1].count(299) == rows["tall"] + rows["square"]
    assert len({rows["wide"], rows["tall"], rows["square"]}) > 1          # the count really depends on the image
    got = {0: [], 1: []}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    images = {0: [(wide, (30, 100))], 1: [(tall, (70, 40)), (square, (50, 50))]}
    for i in range(2):
        ids = torch.tensor([prompts[i]])
        views = [anyres_views(b, PINS, 28)[0] for b, _ in images[i]]
        n = max(v.shape[0] for v in views)
        px = torch.stack([torch.cat([v, torch.zeros(n - v.shape[0], *v.shape[1:])]) for v in views])
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=px,
                              image_sizes=torch.tensor([list(sz) for _, sz in images[i]]), max_new_tokens=5,
                              min_new_tokens=5, do_sample=False)
        assert got[i][:5] == ref[0, ids.shape[1]:].tolist(), (i, got[i], ref[0, ids.shape[1]:].tolist())


def test_unpadding_and_fit_match_transformers_on_many_sizes():
    import random

    from transformers.image_processing_utils import get_patch_output_size
    from transformers.models.llava_next.modeling_llava_next import unpad_image

    from tgi_b200.models.llava_next import _fit, unpadded_map

    rng = random.Random(0)
    pins = [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]]
    for _ in range(200):
        h, w = rng.randint(8, 2500), rng.randint(8, 2500)
        bh, bw = select_best_resolution((h, w), pins)
        img = np.zeros((h, w, 3), dtype=np.uint8)
        assert _fit((h, w), (bh, bw)) == tuple(get_patch_output_size(img, (bh, bw), "channels_last")), (h, w)
        mh, mw = bh // 336 * 24, bw // 336 * 24
        top, bottom, left, right = unpadded_map((h, w), (mh, mw))
        ref = unpad_image(torch.zeros(1, mh, mw), (h, w))
        assert (bottom - top, right - left) == tuple(ref.shape[1:]), (h, w)
        assert anyres_rows((h, w), pins, 336, 24) == 576 + ref.shape[1] * (ref.shape[2] + 1)
