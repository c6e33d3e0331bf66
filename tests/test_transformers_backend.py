"""Transformers-backend runner (CPU): architectures without a native decoder run their own transformers
modules around the paged attention and keep the ragged batch; checked against ``generate`` of transformers."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.arch import ARCHS  # noqa: E402
from tgi_b200.models.flash_causal_lm import FlashCausalLM  # noqa: E402
from tgi_b200.models.transformers_backend import TransformersDecoder, supports  # noqa: E402

from tgi_b200.proto import generate_v3 as pb  # noqa: E402
from test_padded_runners import _request  # noqa: E402


def _run(model, prompts, n_new):
    reqs = [_request(i, p, n_new) for i, p in enumerate(prompts)]
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=len(reqs)), model.tokenizer, model.dtype,
                                     model.device)
    out = {i: [] for i in range(len(prompts))}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            if g.tokens is not None:
                out[g.request_id].extend(g.tokens.token_ids)
    return out


def _tiny(arch):
    V = 300
    common = dict(vocab_size=V, hidden_size=256, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=128, pad_token_id=0, eos_token_id=1, bos_token_id=2)
    if arch == "olmo2":
        return transformers.Olmo2ForCausalLM(transformers.Olmo2Config(**common))
    if arch == "glm":
        return transformers.GlmForCausalLM(transformers.GlmConfig(head_dim=64, partial_rotary_factor=0.5, **common))
    if arch == "llama4_text":      # the text decoder of Llama-4: interleaved MoE layers, q/k norm, rotary in pairs
        return transformers.Llama4ForCausalLM(transformers.Llama4TextConfig(
            vocab_size=V, hidden_size=64, intermediate_size=64, intermediate_size_mlp=128, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_local_experts=2, num_experts_per_tok=1,
            max_position_embeddings=128, pad_token_id=0, eos_token_id=1, bos_token_id=2, attention_chunk_size=64))
    return transformers.HeliumForCausalLM(transformers.HeliumConfig(head_dim=64, **common))


@pytest.mark.parametrize("arch", ["olmo2", "glm", "helium", "llama4_text"])
def test_transformers_backend_matches_generate(tmp_path, arch):
    assert arch not in ARCHS and supports({"model_type": arch})
    torch.manual_seed(0)
    hf = _tiny(arch).eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    model = get_model(str(tmp_path), dtype="float32", device=torch.device("cpu"))
    assert isinstance(model, FlashCausalLM) and isinstance(model.model, TransformersDecoder)
    assert not model.info.requires_padding and model.support_chunking
    prompts = [[10, 20, 30, 40, 50], [7, 8, 9], [100, 90, 80, 70, 60, 50, 40]]
    n_new = 6
    got = _run(model, prompts, n_new)
    for i, p in enumerate(prompts):
        seq = list(model.tokenizer("".join(chr(3 + t) for t in p))["input_ids"])
        n0 = len(seq)
        with torch.no_grad():      # plain greedy decoding (``generate`` would mask the end-of-sequence token)
            for _ in range(n_new):
                seq.append(int(hf(torch.tensor([seq])).logits[0, -1].argmax()))
        assert got[i] == seq[n0:], (arch, i)


@pytest.mark.parametrize("arch", ["olmo2", "glm", "helium"])
def test_transformers_backend_tensor_parallel(tmp_path, arch):
    """Two gloo ranks: helium shards the heads (column-parallel q / k / v), olmo2 gathers q / k / v for its norms over
    all heads, glm gathers its fused gate_up; all three must match the unsharded transformers model."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    torch.manual_seed(0)
    _tiny(arch).eval().save_pretrained(str(tmp_path), safe_serialization=True)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", DIST_WORKER_DIR=str(tmp_path), PYTHONPATH=root)
    port = 29831 + ["olmo2", "glm", "helium"].index(arch)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "tests", "dist_tfb_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DIST_WORKER_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


def test_unsupported_models_still_fall_back():
    assert not supports({"model_type": "stablelm"})
    assert not supports({"model_type": "no_such_model"})
