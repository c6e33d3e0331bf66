"""Fallback runners over transformers modules (CPU): a GPT-2-style causal model, a T5-style
encoder/decoder and a Mamba state-space model, each checked against ``generate`` of transformers."""
import json

import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402


def _save(model, path, vocab):
    model.save_pretrained(str(path), safe_serialization=True)
    return path


def _request(i, text_ids, n_new):
    r = pb.Request(id=i, inputs="".join(chr(3 + t) for t in text_ids))
    r.add_special_tokens = False
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.prefill_logprobs = True
    return r


def _run(model, prompts, n_new):
    reqs = [_request(i, p, n_new) for i, p in enumerate(prompts)]
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=len(reqs)), model.tokenizer, model.dtype,
                                     model.device, 0)
    out = {i: [] for i in range(len(prompts))}
    first = True
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            out[g.request_id].extend(g.tokens.token_ids)
        if first and batch is not None and len(batch) > 1:
            # exercise filter + concatenate: split the batch and glue it back together
            a = batch.filter([0])
            b = batch.filter(list(range(1, len(prompts))))
            batch = type(batch).concatenate([a, b])
            first = False
    return out


@pytest.mark.parametrize("arch", ["bloom", "t5", "mamba"])
def test_fallback_runner_matches_transformers_generate(tmp_path, arch):
    torch.manual_seed(0)
    V = 300
    if arch == "bloom":
        cfg = transformers.BloomConfig(vocab_size=V, hidden_size=32, n_layer=2, n_head=4)
        hf = transformers.BloomForCausalLM(cfg)
    elif arch == "t5":
        cfg = transformers.T5Config(vocab_size=V, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4,
                                    decoder_start_token_id=0, pad_token_id=0, eos_token_id=1)
        hf = transformers.T5ForConditionalGeneration(cfg)
    else:
        cfg = transformers.MambaConfig(vocab_size=V, hidden_size=32, state_size=8, num_hidden_layers=2,
                                       pad_token_id=0, eos_token_id=1, bos_token_id=2)
        hf = transformers.MambaForCausalLM(cfg)
    hf = hf.eval()
    _save(hf, tmp_path, V)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert model.info.requires_padding and not model.support_chunking
    prompts = [[10, 20, 30, 40, 50], [7, 8, 9], [100, 90, 80, 70, 60, 50, 40]]
    n_new = 6
    got = _run(model, prompts, n_new)
    for i, p in enumerate(prompts):
        ids = torch.tensor([model.tokenizer("".join(chr(3 + t) for t in p))["input_ids"]])
        with torch.no_grad():
            ref = hf.generate(ids, max_new_tokens=n_new, min_new_tokens=n_new, do_sample=False)
        want = ref[0, (1 if arch == "t5" else ids.shape[1]):].tolist()
        assert got[i] == want[:n_new], (arch, i, got[i], want)


@pytest.mark.parametrize("arch", ["bloom", "opt"])
def test_fallback_runner_tensor_parallel(tmp_path, arch):
    """Two gloo ranks: column-parallel q / k / v and first MLP layer, row-parallel output projections, Bloom's ALiBi
    bias cut to the rank's heads; greedy tokens equal those of the unsharded transformers model."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    torch.manual_seed(0)
    V = 300
    if arch == "bloom":
        hf = transformers.BloomForCausalLM(transformers.BloomConfig(vocab_size=V, hidden_size=32, n_layer=2, n_head=4))
    else:
        hf = transformers.OPTForCausalLM(transformers.OPTConfig(
            vocab_size=V, hidden_size=32, ffn_dim=64, num_hidden_layers=2, num_attention_heads=4, word_embed_proj_dim=32,
            max_position_embeddings=64, pad_token_id=0, eos_token_id=1, bos_token_id=2))
    _save(hf.eval(), tmp_path, V)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", DIST_WORKER_DIR=str(tmp_path), PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29851 + (arch == "opt")), os.path.join(root, "tests", "dist_padded_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DIST_WORKER_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


def test_galactica_sequences_are_marked_character_by_character():
    from tgi_b200.models.padded import GALACTICA_SPLIT_MARKER as M, galactica_mark_sequences

    assert galactica_mark_sequences("plain text") == "plain text"
    got = galactica_mark_sequences("x [START_DNA]ACG[END_DNA] y [START_SMILES]C=O[END_SMILES]")
    assert got == f"x [START_DNA]{M}A{M}C{M}G{M}[END_DNA] y [START_SMILES]{M}C{M}={M}O{M}[END_SMILES]"
    # an unmatched or mismatched pair is left alone
    assert galactica_mark_sequences("[START_DNA]AC[END_AMINO]") == "[START_DNA]AC[END_AMINO]"


def test_galactica_checkpoints_get_their_batch_type(tmp_path):
    from tgi_b200.models.padded import GalacticaBatch

    torch.manual_seed(0)
    V = 300
    hf = transformers.OPTForCausalLM(transformers.OPTConfig(
        vocab_size=V, hidden_size=32, ffn_dim=64, num_hidden_layers=1, num_attention_heads=4, word_embed_proj_dim=32,
        max_position_embeddings=64, pad_token_id=0, eos_token_id=1, bos_token_id=2))
    d = tmp_path / "galactica-tiny"
    d.mkdir()
    _save(hf.eval(), d, V)
    model = get_model(str(d), dtype="float32", device=torch.device("cpu"))
    assert model.batch_type is GalacticaBatch
    got = _run(model, [[10, 20, 30]], 3)
    assert len(got[0]) == 3
