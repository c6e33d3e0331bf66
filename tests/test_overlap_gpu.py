"""Decode overlap: the next step's graph replay is put on the stream before the text post-processing of the
current step.  Sequences of different lengths (so that steps with and without a finishing sequence alternate)
must produce the same tokens with the overlap on and off."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _generate(model, prompts, lengths, stop_at=None):
    from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch
    from tgi_b200.proto import generate_v3 as pb

    reqs, cursor = [], 1
    for i, (p, n) in enumerate(zip(prompts, lengths)):
        r = pb.Request(id=i, inputs="")
        r.parameters.temperature = 1.0
        r.parameters.top_p = 1.0
        r.parameters.typical_p = 1.0
        r.parameters.repetition_penalty = 1.0
        r.stopping_parameters.max_new_tokens = n
        r.stopping_parameters.ignore_eos_token = True
        if stop_at and i == 0:
            r.stopping_parameters.stop_sequences.append(stop_at)
        nb = (len(p) + n + 15) // 16
        r.blocks.extend(range(cursor, cursor + nb))
        cursor += nb
        reqs.append(r)
    batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts, model.tokenizer,
                                              torch.bfloat16, model.device)
    toks = {i: [] for i in range(len(prompts))}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        done = [g.request_id for g in gens if g.generated_text is not None]
        for g in gens:
            toks[g.request_id].extend(g.tokens.token_ids)
        if batch is not None and done:      # what the router does: drop finished sequences
            keep = [s.request.id for s in batch.seqs if s.request.id not in done]
            batch = batch.filter(keep) if keep else None
    return toks


def test_overlapped_decode_matches_plain_decode(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tgi_b200.models import get_model
    from tgi_b200.models.graphs import DecodeGraphs
    from tgi_b200.ops import cuda as K
    from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint

    cfg = llama_config(hidden=256, layers=2, heads=4, kv_heads=2, intermediate=512, vocab=300, max_pos=512)
    write_llama_checkpoint(tmp_path, cfg)
    model = get_model(str(tmp_path), dtype="bfloat16", device=torch.device("cuda"))
    rng = random.Random(1)
    prompts = [[rng.randrange(3, 300) for _ in range(n)] for n in (9, 17, 5, 12)]
    lengths = [6, 14, 10, 14]
    model.init_kv_cache(16)
    model.graphs = DecodeGraphs(model, 64, buckets=[1, 2, 4])
    model.graphs.capture_all()

    model.overlap_decode = False
    plain = _generate(model, prompts, lengths)
    assert model.overlap_hits == 0 and [len(plain[i]) for i in range(4)] == lengths
    model.overlap_decode = True
    over = _generate(model, prompts, lengths)
    assert over == plain
    assert model.overlap_hits >= 5          # steps between two finishes ran ahead of their post-processing
    # while a request with a stop string is in the batch (the first 6 steps) every step waits for its text
    hits = model.overlap_hits
    assert _generate(model, prompts, lengths, stop_at="\\x00never\\x00") == plain
    assert 0 < model.overlap_hits - hits < hits
    assert K.check_status() == 0
