"""Multi-LoRA on CPU: a mixed batch (base + two adapters) must reproduce, request by request, what
models with the adapters merged into their weights generate; adapter parsing and merge strategies."""
import json
import random

import pytest
import torch

from tgi_b200.models import get_model, get_model_with_lora_adapters
from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch
from tgi_b200.proto import generate_v3 as pb
from tgi_b200.utils import adapter as ad
from tgi_b200.utils.synthetic import llama_config, llama_state_dict, write_llama_checkpoint
from tgi_b200.utils.weights import save_safetensors

CFG = dict(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=128, vocab=300, max_pos=512)
TARGETS = {"q_proj": (64, 64), "k_proj": (32, 64), "v_proj": (32, 64), "o_proj": (64, 64),
           "gate_proj": (128, 64), "up_proj": (128, 64), "down_proj": (64, 128)}


def _write_adapter(path, seed, r=4, alpha=8.0):
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for li in range(2):
        for proj, (out_f, in_f) in TARGETS.items():
            mod = "self_attn" if proj in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{li}.{mod}.{proj}"
            sd[f"{base}.lora_A.weight"] = torch.randn(r, in_f, generator=g) * 0.2
            sd[f"{base}.lora_B.weight"] = torch.randn(out_f, r, generator=g) * 0.2
    path.mkdir(parents=True)
    save_safetensors(sd, path / "adapter_model.safetensors", {"format": "pt"})
    (path / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": alpha, "target_modules": list(TARGETS)}))
    return sd, alpha / r


def _merged_checkpoint(path, cfg, lora_sd, scale):
    sd = llama_state_dict(cfg)
    for li in range(2):
        for proj in TARGETS:
            mod = "self_attn" if proj in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            a = lora_sd[f"base_model.model.model.layers.{li}.{mod}.{proj}.lora_A.weight"]
            b = lora_sd[f"base_model.model.model.layers.{li}.{mod}.{proj}.lora_B.weight"]
            sd[f"model.layers.{li}.{mod}.{proj}.weight"] = sd[f"model.layers.{li}.{mod}.{proj}.weight"] + scale * (b @ a)
    path.mkdir(parents=True)
    (path / "config.json").write_text(json.dumps(cfg))
    save_safetensors(sd, path / "model.safetensors", {"format": "pt"})


def _request(i, n_new, blocks, adapter_id=None):
    r = pb.Request(id=i, inputs="")
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.blocks.extend(blocks)
    if adapter_id:
        r.adapter_id = adapter_id
    return r


def _generate(model, prompts, n_new, adapter_ids):
    cursor, reqs = 1, []
    for i, p in enumerate(prompts):
        nb = (len(p) + n_new + 15) // 16
        reqs.append(_request(i, n_new, range(cursor, cursor + nb), adapter_ids[i]))
        cursor += nb
    model.init_kv_cache(cursor)
    batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts, model.tokenizer,
                                              torch.float32, torch.device("cpu"))
    toks = {i: [] for i in range(len(prompts))}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            toks[g.request_id].extend(g.tokens.token_ids)
    return toks


def test_parse_lora_adapters():
    got = ad.parse_lora_adapters("a/b, c=/tmp/x ,d@rev1")
    assert [(p.adapter_id, p.path, p.revision) for p in got] == [("a/b", None, None), ("c", "/tmp/x", None), ("d", None, "rev1")]
    assert ad.parse_lora_adapters("") == []
    with pytest.raises(ValueError):
        ad.parse_lora_adapters("a,a")


def test_mixed_batch_matches_merged_models(tmp_path):
    cfg = llama_config(**CFG)
    base = tmp_path / "base"
    write_llama_checkpoint(base, cfg)
    sd1, s1 = _write_adapter(tmp_path / "ad1", 1)
    sd2, s2 = _write_adapter(tmp_path / "ad2", 2, r=8, alpha=4.0)
    _merged_checkpoint(tmp_path / "m1", cfg, sd1, s1)
    _merged_checkpoint(tmp_path / "m2", cfg, sd2, s2)
    rng = random.Random(0)
    prompts = [[rng.randrange(3, 300) for _ in range(n)] for n in (11, 19, 7, 15)]
    n_new = 8
    kw = dict(dtype="float32", device=torch.device("cpu"))
    want_base = _generate(get_model(str(base), **kw), prompts, n_new, [None] * 4)
    want_1 = _generate(get_model(str(tmp_path / "m1"), **kw), prompts, n_new, [None] * 4)
    want_2 = _generate(get_model(str(tmp_path / "m2"), **kw), prompts, n_new, [None] * 4)
    assert want_1 != want_base and want_2 != want_base      # the adapters do change the output

    adapters = ad.parse_lora_adapters(f"one={tmp_path / 'ad1'},two={tmp_path / 'ad2'}")
    model = get_model_with_lora_adapters(str(base), adapters, **kw)
    assert ad.ADAPTER_TO_INDEX["one"] == 1 and ad.ADAPTER_TO_INDEX["two"] == 2
    got = _generate(model, prompts, n_new, ["one", None, "two", "one"])
    assert got[0] == want_1[0] and got[1] == want_base[1] and got[2] == want_2[2] and got[3] == want_1[3]


def test_merge_strategies():
    def mk(seed):
        g = torch.Generator().manual_seed(seed)
        a = ad.LoraAdapter(f"a{seed}", ad.LoraConfig(4, 8.0, ["q_proj"]))
        a.layers[(0, "q_proj")] = ad.LoraLayer(torch.randn(4, 16, generator=g), torch.randn(16, 4, generator=g), 2.0)
        return a

    x, y = mk(1), mk(2)
    lin = ad.merge_adapters([x, y], [0.5, 0.5], "lin")
    torch.testing.assert_close(lin.layers[(0, "q_proj")].a, 0.5 * (x.layers[(0, "q_proj")].a + y.layers[(0, "q_proj")].a))
    ties = ad.merge_adapters([x, y], [1.0, 1.0], "ties", strategy="ties", density=0.5)
    assert (ties.layers[(0, "q_proj")].a == 0).float().mean() > 0.1
    dare = ad.merge_adapters([x, y], [1.0, 1.0], "dare", strategy="dare", density=0.5)
    assert dare.layers[(0, "q_proj")].a.shape == (4, 16)
