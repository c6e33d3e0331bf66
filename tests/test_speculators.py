"""Medusa (v1 / v2 layouts) and MLP-speculator heads on CPU: drafts come from the heads, and greedy
output with speculation is identical to greedy output without it."""
import json
import random

import pytest
import torch

from tgi_b200.models import get_model
from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch
from tgi_b200.proto import generate_v3 as pb
from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint
from tgi_b200.utils.weights import save_safetensors

CFG = dict(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=128, vocab=300, max_pos=512)


def _request(i, n_new, blocks):
    r = pb.Request(id=i, inputs="")
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.blocks.extend(blocks)
    return r


def _generate(model, prompts, n_new, speculate):
    cursor, reqs = 1, []
    for i, p in enumerate(prompts):
        nb = (len(p) + n_new + speculate + 15) // 16 + 1
        reqs.append(_request(i, n_new, range(cursor, cursor + nb)))
        cursor += nb
    model.init_kv_cache(cursor)
    batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts, model.tokenizer,
                                              torch.float32, torch.device("cpu"), speculate)
    toks = {i: [] for i in range(len(prompts))}
    steps = 0
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        steps += 1
        for g in gens:
            toks[g.request_id].extend(g.tokens.token_ids)
        assert steps < 200
    return {i: t[:n_new] for i, t in toks.items()}, steps


def _write_medusa(path, v2: bool, H=64, V=300, heads=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for h in range(heads):
        sd[f"{h}.0.linear.weight"] = torch.randn(H, H, generator=g) * 0.05
        sd[f"{h}.0.linear.bias"] = torch.randn(H, generator=g) * 0.05
        if not v2:
            sd[f"{h}.1.weight"] = torch.randn(V, H, generator=g) * 0.05
    save_safetensors(sd, path / "medusa_lm_head.safetensors", {"format": "pt"})
    (path / "config.json").write_text(json.dumps({"medusa_num_heads": heads, "medusa_num_layers": 1}))


def _write_mlp_speculator(path, H=64, V=300, n=3, inner=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for i in range(n):
        sd[f"speculator.emb.{i}.weight"] = torch.randn(V, inner, generator=g) * 0.05
        sd[f"speculator.proj.{i}.weight"] = torch.randn(inner, H if i == 0 else inner, generator=g) * 0.05
        sd[f"speculator.head.{i}.weight"] = torch.randn(V, inner, generator=g) * 0.05
        sd[f"speculator.ln.{i}.weight"] = torch.ones(inner)
        sd[f"speculator.ln.{i}.bias"] = torch.zeros(inner)
    save_safetensors(sd, path / "model.safetensors", {"format": "pt"})
    (path / "config.json").write_text(json.dumps({"model_type": "mlp_speculator", "n_predict": n, "emb_dim": H,
                                                  "inner_dim": inner, "tie_weights": False, "scale_input": True}))


@pytest.mark.parametrize("kind", ["medusa_v1", "medusa_v2", "mlp"])
def test_speculator_heads_keep_greedy_output(tmp_path, kind):
    base = tmp_path / "base"
    write_llama_checkpoint(base, llama_config(**CFG))
    rng = random.Random(1)
    prompts = [[rng.randrange(3, 300) for _ in range(n)] for n in (9, 23, 14)]
    plain = get_model(str(base), dtype="float32", device=torch.device("cpu"))
    want, plain_steps = _generate(plain, prompts, 12, 0)

    spec_dir = base / "speculator"
    spec_dir.mkdir()
    if kind == "mlp":
        _write_mlp_speculator(spec_dir)
    else:
        _write_medusa(spec_dir, v2=(kind == "medusa_v2"))
    model = get_model(str(base), dtype="float32", device=torch.device("cpu"))
    assert model.model.speculator is not None and model.speculate == 3
    got, steps = _generate(model, prompts, 12, model.speculate)
    assert got == want
    assert steps <= plain_steps
    # the head produces one draft per head for every sampled row
    hidden = torch.randn(5, 64)
    logits = torch.randn(5, 300)
    assert model.model.speculator(hidden, logits).shape == (5, 3, 300)


def test_ngram_speculation_keeps_greedy_output(tmp_path):
    base = tmp_path / "base"
    write_llama_checkpoint(base, llama_config(**CFG))
    prompts = [[5, 6, 7, 8] * 6, [9, 10, 11] * 5]
    model = get_model(str(base), dtype="float32", device=torch.device("cpu"))
    want, _ = _generate(model, prompts, 10, 0)
    model2 = get_model(str(base), dtype="float32", device=torch.device("cpu"), speculate=2)
    got, _ = _generate(model2, prompts, 10, 2)
    assert got == want
