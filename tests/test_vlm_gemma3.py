"""Gemma-3 multimodal on CPU against transformers: SigLIP tower, average-pooled projector, and image rows that
attend to each other in both directions (also inside sliding-window layers) through the attention horizon."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.vlm_causal_lm import SIGLIP_MEAN, SIGLIP_STD, preprocess_image  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _png, _request  # noqa: E402

IMG, BOI, EOI = 299, 298, 297


@pytest.fixture(scope="module")
def gemma(tmp_path_factory):
    torch.manual_seed(0)
    vis = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=56,
               patch_size=14)
    txt = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
               head_dim=64, vocab_size=300, max_position_embeddings=512, sliding_window=6, sliding_window_pattern=2,
               query_pre_attn_scalar=64, tie_word_embeddings=True)
    cfg = transformers.Gemma3Config(vision_config=vis, text_config=txt, mm_tokens_per_image=4, image_token_index=IMG,
                                    boi_token_index=BOI, eoi_token_index=EOI)
    hf = transformers.Gemma3ForConditionalGeneration(cfg).eval()
    d = tmp_path_factory.mktemp("gemma3")
    hf.save_pretrained(str(d), safe_serialization=True)
    return hf, d


def test_gemma3_generation_matches_transformers(gemma):
    hf, d = gemma
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"))
    assert model.tokens_per_image == 4 and model.bidirectional_images and not model.support_chunking
    png1, png2 = _png(1), _png(2)
    reqs = [
        _request(0, [("text", "abcdefgh"), ("image", png1), ("text", "cde")], 6, range(1, 4)),
        _request(1, [("image", png2), ("text", "xy"), ("image", png1), ("text", "z")], 6, range(4, 8)),
        _request(2, [("text", "no image here")], 6, range(8, 11)),
    ]
    model.init_kv_cache(12)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=3), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompts = [list(s.ids) for s in batch.seqs]
    assert prompts[0].count(IMG) == 4 and prompts[0].count(BOI) == 1 and prompts[1].count(EOI) == 2
    got = {i: [] for i in range(3)}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    images = {0: [png1], 1: [png2, png1], 2: []}
    for i in range(3):
        ids = torch.tensor([prompts[i]])
        kw = {}
        if images[i]:
            kw["pixel_values"] = torch.stack([preprocess_image(b, 56, SIGLIP_MEAN, SIGLIP_STD) for b in images[i]])
            kw["token_type_ids"] = (ids == IMG).long()
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=6, min_new_tokens=6,
                              do_sample=False, **kw)
        assert got[i][:6] == ref[0, ids.shape[1]:].tolist(), (i, got[i], ref[0, ids.shape[1]:].tolist())


def test_horizon_changes_the_result(gemma):
    """The bidirectional rows matter: with plain causal attention the logits of an image prompt differ."""
    _, d = gemma
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"))
    req = _request(0, [("text", "ab"), ("image", _png(3)), ("text", "c")], 2, range(1, 4))
    model.init_kv_cache(6)
    outs = []
    for bidir in (True, False):
        model.bidirectional_images = bidir
        batch = model.batch_type.from_pb(pb.Batch(id=0, requests=[req], size=1), model.tokenizer, torch.float32,
                                         torch.device("cpu"), 0)
        counts = batch.plan_step()
        meta, _ = model.build_meta(batch, counts)
        assert (meta.attn_horizon is not None) == bidir
        outs.append(model.forward(meta).float())
    assert not torch.allclose(outs[0], outs[1], atol=1e-5)


def test_gemma3_image_runs_get_blank_lines_with_a_real_tokenizer(gemma, tmp_path):
    """With a Hugging Face tokenizer an image is "\\n\\n" + begin token + rows + end token + "\\n\\n", as the processor
    writes it; the router counts those tokens too."""
    import shutil

    from tokenizers import Regex, Tokenizer, models, pre_tokenizers

    _, d = gemma
    for f in d.iterdir():
        shutil.copy(f, tmp_path / f.name)
    chars = ["<unk>"] + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(r"\n"), "isolated"),
                                                 pre_tokenizers.Split(Regex("."), "isolated")])
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast",
                                                                "unk_token": "<unk>"}))
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    reqs = [_request(0, [("text", "ab"), ("image", _png(1)), ("text", "c")], 2, range(1, 4))]
    model.init_kv_cache(6)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=1), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    nl = tok.token_to_id("\n")
    a, b, c = (tok.token_to_id(x) for x in "abc")
    assert list(batch.seqs[0].ids) == [a, b, nl, nl, BOI] + [IMG] * 4 + [EOI, nl, nl, c]
    from tgi_b200.router.build import build

    build()
    from tgi_b200.router import _router_test as rt

    cfg = json.loads((tmp_path / "config.json").read_text())
    assert rt.tokens_per_image(json.dumps(dict(cfg, _gemma3={"pad": 2})), 52, 40) == 4 + 2 + 4
    assert rt.tokens_per_image(json.dumps(cfg), 52, 40) == 4 + 2
