"""Tiny Llama on CPU, fp32: continuous batching with requests joining two per decode step; the
engine's logits must match a plain dense PyTorch forward to 1e-4 and greedy tokens must agree."""
import json
import random

import numpy as np
import pytest
import torch

from tgi_b200.models import get_model
from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch
from tgi_b200.proto import generate_v3 as pb
from tgi_b200.utils.synthetic import llama_config, llama_state_dict, reference_llama_forward


def make_request(i, n_new=32, blocks=None, **kw):
    r = pb.Request(id=i, inputs="", truncate=0, prefill_logprobs=False, top_n_tokens=0, **kw)
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    if blocks is not None:
        r.blocks.extend(blocks)
    return r


def greedy_reference(sd, cfg, prompt, n_new):
    ids = list(prompt)
    logits_trace = []
    for _ in range(n_new):
        lg = reference_llama_forward(sd, cfg, torch.tensor(ids))[-1]
        logits_trace.append(lg)
        ids.append(int(lg.argmax()))
    return ids[len(prompt):], logits_trace


def test_continuous_batching_matches_dense_forward(tiny_llama_dir, monkeypatch):
    cfg = llama_config()
    sd = llama_state_dict(cfg)
    model = get_model(tiny_llama_dir, dtype="float32", device=torch.device("cpu"))
    rng = random.Random(0)
    n_req, n_new = 8, 32
    prompts = [[rng.randrange(32000) for _ in range(rng.randint(16, 128))] for _ in range(n_req)]
    # router-style block allocation: disjoint block ranges per request
    cursor, blocks = 1, []
    for p in prompts:
        nb = (len(p) + n_new + 15) // 16
        blocks.append(list(range(cursor, cursor + nb)))
        cursor += nb
    model.init_kv_cache(cursor)

    captured = {}
    orig_forward = model.forward

    def spy(meta):
        out = orig_forward(meta)
        captured["logits"] = out.detach().clone()
        return out

    monkeypatch.setattr(model, "forward", spy)

    outputs = {i: [] for i in range(n_req)}
    first_logits = {}
    batch = None
    pending = list(range(n_req))
    step = 0
    while pending or batch is not None:
        if pending:
            new_ids = pending[:2]
            pending = pending[2:]
            bpb = pb.Batch(id=step, requests=[make_request(i, n_new, blocks[i]) for i in new_ids], size=len(new_ids))
            nb = FlashCausalLMBatch.from_tokenized(bpb, [prompts[i] for i in new_ids], model.tokenizer,
                                                   torch.float32, torch.device("cpu"))
            gens, nb, _ = model.generate_token(nb)
            for k, i in enumerate(new_ids):
                first_logits[i] = captured["logits"][k]
            for g in gens:
                outputs[g.request_id].extend(g.tokens.token_ids)
            batch = nb if batch is None else FlashCausalLMBatch.concatenate([batch, nb])
        gens, batch, _ = model.generate_token(batch)
        keep = []
        for g in gens:
            outputs[g.request_id].extend(g.tokens.token_ids)
            if g.generated_text is None:
                keep.append(g.request_id)
            else:
                assert g.generated_text.generated_tokens == n_new
        if batch is not None:
            batch = batch.filter(keep) if keep else None
        step += 1
        assert step < 200

    for i in range(n_req):
        want, trace = greedy_reference(sd, cfg, prompts[i], 3)
        assert outputs[i][:3] == want
        assert len(outputs[i]) == n_new
        torch.testing.assert_close(first_logits[i], trace[0], atol=1e-4, rtol=1e-4)


def test_chunked_prefill_and_prefix_cache_equal_full_prefill(tiny_llama_dir):
    model = get_model(tiny_llama_dir, dtype="float32", device=torch.device("cpu"))
    model.init_kv_cache(64)
    rng = random.Random(1)
    prompt = [rng.randrange(32000) for _ in range(70)]

    def run(req, budget=None):
        bpb = pb.Batch(id=0, requests=[req], size=1)
        b = FlashCausalLMBatch.from_tokenized(bpb, [prompt], model.tokenizer, torch.float32, torch.device("cpu"))
        b.max_prefill_tokens = budget
        toks = []
        while b is not None:
            gens, b, _ = model.generate_token(b)
            for g in gens:
                toks.extend(g.tokens.token_ids)
        return toks

    full = run(make_request(0, 6, list(range(1, 7))))
    chunked = run(make_request(1, 6, list(range(10, 16))), budget=16)
    assert chunked == full
    # prefix cache hit: blocks 1..4 (64 tokens) still hold the prompt's KV from the first run
    hit = make_request(2, 6, list(range(1, 5)) + [20, 21], cache_len=64)
    assert run(hit) == full
    # router-imposed first chunk
    first = make_request(3, 6, list(range(30, 36)), chunk_len=33)
    assert run(first, budget=40) == full
