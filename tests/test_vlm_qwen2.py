"""Qwen2-VL on CPU against transformers: dynamic-resolution patches, the vision tower with 2-D rotary
embedding and patch merger, 3-axis rotary positions in the language model, and decode steps that carry
the position offset left by the images."""
import io
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.qwen2_vl import Qwen2VlBatch, patchify, preprocess_qwen_image, smart_resize  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _request  # noqa: E402

IMG, START, END = 299, 298, 297


def _png(seed, h, w):
    from PIL import Image

    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 255, size=(h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def _build(kind, d):
    torch.manual_seed(0)
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=300, max_position_embeddings=512, tie_word_embeddings=False,
               rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    ids = dict(image_token_id=IMG, vision_start_token_id=START, vision_end_token_id=END, video_token_id=296)
    if kind == "qwen2_vl":
        vis = dict(depth=2, embed_dim=32, hidden_size=64, mlp_ratio=2, num_heads=2, patch_size=14, spatial_merge_size=2,
                   temporal_patch_size=2, in_channels=3)
        hf = transformers.Qwen2VLForConditionalGeneration(transformers.Qwen2VLConfig(vision_config=vis, text_config=txt, **ids))
    else:
        # windows of 2 x 2 merged patches, full attention only in block 1
        vis = dict(depth=3, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, patch_size=14,
                   spatial_merge_size=2, temporal_patch_size=2, in_channels=3, window_size=56, fullatt_block_indexes=[1])
        hf = transformers.Qwen2_5_VLForConditionalGeneration(
            transformers.Qwen2_5_VLConfig(vision_config=vis, text_config=txt, **ids))
    hf = hf.eval()
    hf.save_pretrained(str(d), safe_serialization=True)
    c = json.loads((d / "config.json").read_text())
    c["vision_config"]["min_pixels"], c["vision_config"]["max_pixels"] = 28 * 28, 28 * 28 * 16
    (d / "config.json").write_text(json.dumps(c))
    return hf


@pytest.fixture(scope="module")
def qwen(tmp_path_factory):
    d = tmp_path_factory.mktemp("qwen2vl")
    return _build("qwen2_vl", d), d


@pytest.fixture(scope="module")
def qwen25(tmp_path_factory):
    d = tmp_path_factory.mktemp("qwen25vl")
    return _build("qwen2_5_vl", d), d


def test_smart_resize_and_patch_order():
    assert smart_resize(40, 52, 28, 28 * 28, 28 * 28 * 16) == (28, 56)
    assert smart_resize(1000, 1000, 28, 56 * 56, 28 * 28 * 16) == (112, 112)
    px = torch.arange(3 * 28 * 56, dtype=torch.float32).view(3, 28, 56)
    patches, grid = patchify(px, 14, 2, 2)
    assert grid == (1, 2, 4) and patches.shape == (8, 3 * 2 * 14 * 14)
    # rows 0..3 are the 2x2 patches of the left merge block: (0,0) (0,1) (1,0) (1,1)
    p = patches.view(8, 3, 2, 14, 14)
    assert torch.equal(p[1, 0, 0], px[0, :14, 14:28]) and torch.equal(p[2, 0, 1], px[0, 14:28, :14])
    assert torch.equal(p[4, 2, 0], px[2, :14, 28:42])


def test_position_streams_match_transformers(qwen):
    hf, _ = qwen
    ids = [5, 6, START] + [IMG] * 2 + [END, 7, 8, START] + [IMG] * 4 + [END, 9]
    images = [(3, None, (1, 2, 4)), (9, None, (1, 4, 4))]
    pos, delta = Qwen2VlBatch.position_streams(len(ids), images, 2)
    grid = torch.tensor([[1, 2, 4], [1, 4, 4]])
    import inspect
    kw = {}
    if "mm_token_type_ids" in inspect.signature(hf.model.get_rope_index).parameters:
        tt = torch.tensor([[1 if t == IMG else 0 for t in ids]])
        kw["mm_token_type_ids"] = tt
    want, want_delta = hf.model.get_rope_index(torch.tensor([ids]), image_grid_thw=grid,
                                               attention_mask=torch.ones(1, len(ids), dtype=torch.long), **kw)
    assert torch.equal(torch.from_numpy(pos).long(), want[:, 0])
    assert delta == int(want_delta.view(-1)[0])


@pytest.mark.parametrize("chunk", [None, 5])
def test_qwen2_vl_generation_matches_transformers(qwen, chunk):
    hf, d = qwen
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"), max_prefill_tokens=chunk)
    png1, png2 = _png(1, 40, 52), _png(2, 60, 58)
    reqs = [
        _request(0, [("text", "ab"), ("image", png1), ("text", "cde")], 6, range(1, 4)),
        _request(1, [("image", png2), ("text", "xy"), ("image", png1)], 6, range(4, 8)),
        _request(2, [("text", "no image here")], 6, range(8, 11)),
    ]
    model.init_kv_cache(12)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=3), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    if chunk:
        batch.max_prefill_tokens = chunk
    prompts = [list(s.ids) for s in batch.seqs]
    assert prompts[0].count(IMG) == 2 and prompts[1].count(IMG) == 4 + 2 and prompts[0].count(START) == 1
    got = {i: [] for i in range(3)}
    steps = 0
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
        steps += 1
        assert steps < 100
    images = {0: [png1], 1: [png2, png1], 2: []}
    for i in range(3):
        ids = torch.tensor([prompts[i]])
        kw = {}
        if images[i]:
            pre = [preprocess_qwen_image(b, 14, 2, 2, 28 * 28, 28 * 28 * 16) for b in images[i]]
            kw["pixel_values"] = torch.cat([p for p, _ in pre])
            kw["image_grid_thw"] = torch.tensor([list(g) for _, g in pre])
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=6, min_new_tokens=6,
                              do_sample=False, **kw)
        assert got[i][:6] == ref[0, ids.shape[1]:].tolist(), (i, got[i], ref[0, ids.shape[1]:].tolist())


def test_qwen2_5_vl_generation_matches_transformers(qwen25):
    """Windowed vision tower (RMSNorm, gated MLP, window / full attention blocks, window reordering)."""
    hf, d = qwen25
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"))
    assert model.tower.v25 and model.tower.full_blocks == {1}
    png1, png2 = _png(1, 80, 110), _png(2, 60, 58)          # 84 x 112 (3 x 4 merged patches: ragged windows) and 56 x 56
    reqs = [
        _request(0, [("text", "ab"), ("image", png1), ("text", "cde")], 6, range(1, 4)),
        _request(1, [("image", png2), ("text", "xy"), ("image", png1)], 6, range(4, 8)),
    ]
    model.init_kv_cache(12)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=2), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    assert prompts[0].count(IMG) == 12 and prompts[1].count(IMG) == 4 + 12
    got = {0: [], 1: []}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    images = {0: [png1], 1: [png2, png1]}
    for i in range(2):
        ids = torch.tensor([prompts[i]])
        pre = [preprocess_qwen_image(b, 14, 2, 2, 28 * 28, 28 * 28 * 16) for b in images[i]]
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=6, min_new_tokens=6,
                              do_sample=False, pixel_values=torch.cat([p for p, _ in pre]),
                              image_grid_thw=torch.tensor([list(g) for _, g in pre]))
        assert got[i][:6] == ref[0, ids.shape[1]:].tolist(), (i, got[i], ref[0, ids.shape[1]:].tolist())


def test_smart_resize_matches_transformers_on_many_sizes():
    import random

    from transformers.models.qwen2_vl.image_processing_qwen2_vl import smart_resize as ref

    rng = random.Random(3)
    for _ in range(500):
        h, w = rng.randint(4, 5000), rng.randint(4, 5000)
        if max(h, w) / min(h, w) > 200:
            continue
        for lo, hi in [(56 * 56, 28 * 28 * 1280), (28 * 28, 28 * 28 * 16)]:
            assert smart_resize(h, w, 28, lo, hi) == tuple(ref(h, w, 28, lo, hi)), (h, w, lo, hi)
