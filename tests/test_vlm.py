"""LLaVA-style vision-language runner on CPU against transformers' own implementation: the image is
encoded by the CLIP tower, projected, scattered over the placeholder rows, and greedy generation
must agree; also with the prompt prefilled in chunks that cut through the image rows."""
import io
import json

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.vlm_causal_lm import CLIP_MEAN, CLIP_STD, preprocess_image  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402
from tgi_b200.utils.weights import save_safetensors  # noqa: E402


def _png(seed):
    from PIL import Image

    rng = np.random.default_rng(seed)
    img = Image.fromarray(rng.integers(0, 255, size=(40, 52, 3), dtype=np.uint8))
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return buf.getvalue()


def _hub_names(sd):
    out = {}
    for k, v in sd.items():
        if k.startswith("model.language_model."):
            k = "language_model.model." + k[len("model.language_model."):]
        elif k == "lm_head.weight":
            k = "language_model.lm_head.weight"
        elif k.startswith("model."):
            k = k[len("model."):]
        out[k] = v.detach().clone().contiguous()
    return out


@pytest.fixture(scope="module")
def llava(tmp_path_factory):
    torch.manual_seed(0)
    vis = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                        image_size=28, patch_size=14)
    txt = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=300, max_position_embeddings=512,
                                   tie_word_embeddings=False)
    cfg = transformers.LlavaConfig(vision_config=vis, text_config=txt, image_token_index=299, vision_feature_layer=-2,
                                   vision_feature_select_strategy="default")
    hf = transformers.LlavaForConditionalGeneration(cfg).eval()
    d = tmp_path_factory.mktemp("llava")
    save_safetensors(_hub_names(hf.state_dict()), d / "model.safetensors", {"format": "pt"})
    c = cfg.to_dict()
    c["model_type"] = "llava_next"
    (d / "config.json").write_text(json.dumps(c))
    return hf, d


def _request(i, chunks, n_new, blocks):
    r = pb.Request(id=i, inputs="")
    r.add_special_tokens = False
    for kind, val in chunks:
        c = r.input_chunks.chunks.add()
        if kind == "text":
            c.text = val
        else:
            c.image.data = val
            c.image.mimetype = "image/png"
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.blocks.extend(blocks)
    return r


@pytest.mark.parametrize("chunk", [None, 3])
def test_llava_generation_matches_transformers(llava, chunk):
    hf, d = llava
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"), max_prefill_tokens=chunk)
    assert model.tokens_per_image == 4
    png1, png2 = _png(1), _png(2)
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
    assert prompts[0].count(299) == 4 and prompts[1].count(299) == 8 and prompts[2].count(299) == 0
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
            kw["pixel_values"] = torch.stack([preprocess_image(b, 28, CLIP_MEAN, CLIP_STD) for b in images[i]])
        with torch.no_grad():
            ref = hf.generate(input_ids=ids, max_new_tokens=6, min_new_tokens=6, do_sample=False, **kw)
        # requests that finish early keep stepping until the router filters them out: compare 6 tokens
        assert got[i][:6] == ref[0, ids.shape[1]:].tolist(), (i, got[i], ref[0, ids.shape[1]:].tolist())
