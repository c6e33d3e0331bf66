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


def _image(w, h, seed=0):
    import io

    import numpy as np
    from PIL import Image

    rng = np.random.default_rng(seed)
    # smooth content: resampling filters of different libraries agree on it far better than on noise
    base = rng.integers(0, 255, size=(4, 4, 3), dtype=np.uint8)
    img = Image.fromarray(base).resize((w, h), Image.BICUBIC)
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return buf.getvalue(), img


@pytest.mark.parametrize("w,h", [(52, 40), (40, 52), (200, 90), (90, 200), (28, 28), (640, 480), (17, 300)])
def test_idefics3_tile_grid_matches_the_transformers_processor(w, h):
    """Resized size, grid and number of views against the image processor of transformers (tile 28, longest edge 112)."""
    from tgi_b200.models.idefics3 import split_views, tile_grid

    data, img = _image(w, h)
    proc = transformers.Idefics3ImageProcessor(size={"longest_edge": 112}, max_image_size={"longest_edge": 28},
                                               do_image_splitting=True)
    out = proc(images=[img], return_tensors="pt", return_row_col_info=True)
    rows, cols = int(out["rows"][0][0]), int(out["cols"][0][0])
    _, _, r, c = tile_grid(h, w, 112, 28)
    assert (r, c) == (rows, cols)
    sp = split_views(data, 112, 28)
    px = out["pixel_values"][0]
    assert tuple(sp.views.shape) == tuple(px.shape) == (rows * cols + 1 if rows else 1, 3, 28, 28)
    # same content up to the resampling filter's implementation
    assert (sp.views - px).abs().mean().item() < 0.08


def _marker_tokenizer(path, image_token="<image>"):
    """A character-level tokenizer with the Idefics3 marker tokens, saved as tokenizer.json."""
    from tokenizers import Regex, Tokenizer, models, pre_tokenizers

    chars = ["<unk>"] + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split(Regex("."), "isolated")
    # "." does not match a newline: split those as well
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(r"\n"), "isolated"),
                                                 pre_tokenizers.Split(Regex("."), "isolated")])
    specials = ["<fake_token_around_image>", "<global-img>", image_token] + [
        f"<row_{r}_col_{c}>" for r in range(1, 5) for c in range(1, 5)]
    tok.add_special_tokens(specials)
    tok.save(str(path / "tokenizer.json"))
    (path / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast",
                                                            "unk_token": "<unk>"}))
    return {s: tok.token_to_id(s) for s in specials}


def test_idefics3_split_image_generation_matches_transformers(tmp_path):
    """A 52 x 40 image with 28-pixel tiles and a longest edge of 56: a 2 x 2 grid plus the global view.  The prompt
    rows hold marker embeddings and tile features in the processor's order; greedy tokens equal those of
    transformers on the equivalent input ids and pixel values."""
    from tgi_b200.models.idefics3 import Idefics3CausalLM, expansion_length, split_views

    torch.manual_seed(0)
    ids_of = _marker_tokenizer(tmp_path)
    image_id = ids_of["<image>"]
    cfg = transformers.Idefics3Config(vision_config=VIS, text_config=dict(TXT, model_type="llama"),
                                      image_token_id=image_id, scale_factor=2)
    hf = transformers.Idefics3ForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    c = json.loads((tmp_path / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp_path / "config.json").write_text(json.dumps(c))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps(
        {"size": {"longest_edge": 56}, "max_image_size": {"longest_edge": 28}, "do_image_splitting": True}))
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert isinstance(model, Idefics3CausalLM) and model.markers is not None
    seq = model.tokens_per_image
    png = _png(1)
    sp = split_views(png, 56, 28)
    assert (sp.rows, sp.cols) == (2, 2) and sp.views.shape[0] == 5
    nl = model.tokenizer("\n", add_special_tokens=False)["input_ids"]
    nlnl = model.tokenizer("\n\n", add_special_tokens=False)["input_ids"]
    R = expansion_length(2, 2, seq, len(nl), len(nlnl))
    reqs = [_request(0, [("text", "ab"), ("image", png), ("text", "cde")], 6, range(1, 8))]
    model.init_kv_cache(12)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=1), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompt = list(batch.seqs[0].ids)
    assert prompt.count(image_id) == R and len(prompt) == 2 + R + 3
    got = []
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got.extend(g.tokens.token_ids)
    # the same prompt for transformers: real marker ids around runs of the image token
    fake, glob = ids_of["<fake_token_around_image>"], ids_of["<global-img>"]
    run = []
    for r in range(2):
        for col in range(2):
            run += [fake, ids_of[f"<row_{r + 1}_col_{col + 1}>"]] + [image_id] * seq
        run += nl if r == 0 else nlnl
    run += [fake, glob] + [image_id] * seq + [fake]
    assert len(run) == R
    text_a = model.tokenizer("ab", add_special_tokens=False)["input_ids"]
    text_b = model.tokenizer("cde", add_special_tokens=False)["input_ids"]
    ids = torch.tensor([text_a + run + text_b])
    px = sp.views.unsqueeze(0)
    with torch.no_grad():
        ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=px,
                          pixel_attention_mask=torch.ones(1, px.shape[1], 28, 28, dtype=torch.long),
                          max_new_tokens=6, min_new_tokens=6, do_sample=False)
    assert got[:6] == ref[0, ids.shape[1]:].tolist(), (got, ref[0, ids.shape[1]:].tolist())


@pytest.mark.parametrize("split", [False, True])
def test_idefics2_marker_layout_matches_transformers(tmp_path, split):
    """Marker tokens around the image rows and, with image splitting, the four quadrants before the whole image:
    greedy tokens equal those of transformers on the equivalent ids and pixel values; the router counts the same
    number of prompt rows."""
    from tgi_b200.models.idefics2 import Idefics2CausalLM, expansion_length, quadrants_and_whole

    torch.manual_seed(0)
    ids_of = _marker_tokenizer(tmp_path)
    image_id, fake = ids_of["<image>"], ids_of["<fake_token_around_image>"]
    cfg = transformers.Idefics2Config(
        vision_config=VIS, text_config=dict(TXT, model_type="mistral", sliding_window=None), image_token_id=image_id,
        perceiver_config=dict(resampler_n_latents=4, resampler_depth=2, resampler_n_heads=2, resampler_head_dim=16,
                              num_key_value_heads=1, hidden_act="silu", hidden_size=64, rms_norm_eps=1e-6))
    hf = transformers.Idefics2ForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    c = json.loads((tmp_path / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp_path / "config.json").write_text(json.dumps(c))
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"do_image_splitting": split}))
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert isinstance(model, Idefics2CausalLM) and model.fake_id == fake
    L = model.tokens_per_image
    views = 5 if split else 1
    R = expansion_length(views, L)
    png = _png(1)
    reqs = [_request(0, [("text", "ab"), ("image", png), ("text", "cde")], 6, range(1, 6))]
    model.init_kv_cache(8)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=1), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompt = list(batch.seqs[0].ids)
    assert prompt.count(image_id) == R and len(prompt) == 5 + R
    got = []
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got.extend(g.tokens.token_ids)
    run = [fake]
    for _ in range(views):
        run += [image_id] * L + [fake]
    text_a = model.tokenizer("ab", add_special_tokens=False)["input_ids"]
    text_b = model.tokenizer("cde", add_special_tokens=False)["input_ids"]
    ids = torch.tensor([text_a + run + text_b])
    parts = quadrants_and_whole(png) if split else [png]
    px = torch.stack([preprocess_image(p, 28, SIGLIP_MEAN, SIGLIP_STD) for p in parts]).unsqueeze(0)
    with torch.no_grad():
        ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=px,
                          pixel_attention_mask=torch.ones(1, px.shape[1], 28, 28, dtype=torch.long),
                          max_new_tokens=6, min_new_tokens=6, do_sample=False)
    assert got[:6] == ref[0, ids.shape[1]:].tolist(), (got, ref[0, ids.shape[1]:].tolist())
    # the router's count for the same image
    from tgi_b200.router.build import build

    build()
    from tgi_b200.router import _router_test as rt

    rcfg = dict(c, _idefics2={"split": split})
    assert rt.tokens_per_image(json.dumps(rcfg), 52, 40) == R
    assert rt.tokens_per_image(json.dumps(c), 52, 40) == L


def test_idefics2_adjacent_images_share_a_marker(tmp_path):
    """Two images without text between them: marker, rows, marker, rows, marker (the processor collapses the doubled
    marker); generation equals transformers on that prompt."""
    from tgi_b200.models.idefics2 import expansion_length

    torch.manual_seed(0)
    ids_of = _marker_tokenizer(tmp_path)
    image_id, fake = ids_of["<image>"], ids_of["<fake_token_around_image>"]
    cfg = transformers.Idefics2Config(
        vision_config=VIS, text_config=dict(TXT, model_type="mistral", sliding_window=None), image_token_id=image_id,
        perceiver_config=dict(resampler_n_latents=4, resampler_depth=2, resampler_n_heads=2, resampler_head_dim=16,
                              num_key_value_heads=1, hidden_act="silu", hidden_size=64, rms_norm_eps=1e-6))
    hf = transformers.Idefics2ForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    c = json.loads((tmp_path / "config.json").read_text())
    c["vision_config"] = dict(c["vision_config"], **VIS)
    (tmp_path / "config.json").write_text(json.dumps(c))
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    L = model.tokens_per_image
    png1, png2 = _png(1), _png(2)
    reqs = [_request(0, [("text", "ab"), ("image", png1), ("image", png2), ("text", "c")], 5, range(1, 6))]
    model.init_kv_cache(8)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=1), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompt = list(batch.seqs[0].ids)
    R = expansion_length(1, L)
    assert prompt.count(image_id) == 2 * R - 1
    got = []
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got.extend(g.tokens.token_ids)
    run = [fake] + [image_id] * L + [fake] + [image_id] * L + [fake]
    ids = torch.tensor([model.tokenizer("ab", add_special_tokens=False)["input_ids"] + run +
                        model.tokenizer("c", add_special_tokens=False)["input_ids"]])
    px = torch.stack([preprocess_image(p, 28, SIGLIP_MEAN, SIGLIP_STD) for p in (png1, png2)]).unsqueeze(0)
    with torch.no_grad():
        ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=px,
                          pixel_attention_mask=torch.ones(1, 2, 28, 28, dtype=torch.long),
                          max_new_tokens=5, min_new_tokens=5, do_sample=False)
    assert got[:5] == ref[0, ids.shape[1]:].tolist(), (got, ref[0, ids.shape[1]:].tolist())
