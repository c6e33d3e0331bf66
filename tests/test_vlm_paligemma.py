"""PaliGemma on CPU against transformers: SigLIP tower + linear projector, image rows first, every text piece wrapped
as bos + text + newline when the tokenizer names a bos token."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.vlm_causal_lm import SIGLIP_MEAN, SIGLIP_STD, preprocess_image  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402

from test_vlm import _png, _request  # noqa: E402


def _build(tmp, image_id=299, vocab=300):
    torch.manual_seed(0)
    vis = transformers.SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                          image_size=28, patch_size=14, projection_dim=64)
    txt = transformers.GemmaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=1, head_dim=16, vocab_size=vocab, max_position_embeddings=512)
    cfg = transformers.PaliGemmaConfig(vision_config=vis, text_config=txt, image_token_index=image_id, projection_dim=64,
                                       hidden_size=64, vocab_size=vocab)
    hf = transformers.PaliGemmaForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp), safe_serialization=True)
    return hf


def _generate(model, chunks, n_new):
    reqs = [_request(0, chunks, n_new, range(1, 4))]
    model.init_kv_cache(8)
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=1), model.tokenizer, torch.float32,
                                     torch.device("cpu"), 0)
    prompt = list(batch.seqs[0].ids)
    got = []
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got.extend(g.tokens.token_ids)
    return prompt, got


def test_paligemma_generation_matches_transformers(tmp_path):
    hf = _build(tmp_path)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert model.tokens_per_image == 4
    png = _png(1)
    prompt, got = _generate(model, [("image", png), ("text", "what")], 5)
    assert prompt[:4] == [299] * 4
    ids = torch.tensor([prompt])
    px = preprocess_image(png, 28, SIGLIP_MEAN, SIGLIP_STD).unsqueeze(0)
    with torch.no_grad():
        seq = list(prompt)
        for _ in range(5):      # plain greedy decoding with the image-prefix mask of the model
            out = hf(input_ids=torch.tensor([seq]), pixel_values=px, attention_mask=torch.ones(1, len(seq), dtype=torch.long),
                     token_type_ids=torch.zeros(1, len(seq), dtype=torch.long))
            seq.append(int(out.logits[0, -1].argmax()))
    assert got[:5] == seq[len(prompt):], (got, seq[len(prompt):])
    assert ids.shape[1] == len(prompt)


def test_paligemma_text_pieces_are_wrapped_when_the_tokenizer_has_a_bos_token(tmp_path):
    from tokenizers import Regex, Tokenizer, models, pre_tokenizers

    chars = ["<unk>"] + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(r"\n"), "isolated"),
                                                 pre_tokenizers.Split(Regex("."), "isolated")])
    tok.add_special_tokens(["<bos>", "<image>"])
    tok.save(str(tmp_path / "tokenizer.json"))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "bos_token": "<bos>"}))
    _build(tmp_path, image_id=tok.token_to_id("<image>"))
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    prompt, got = _generate(model, [("image", _png(2)), ("text", "hi")], 2)
    image_id, bos, nl = tok.token_to_id("<image>"), tok.token_to_id("<bos>"), tok.token_to_id("\n")
    assert prompt == [image_id] * 4 + [bos, tok.token_to_id("h"), tok.token_to_id("i"), nl]
    assert len(got) == 2
