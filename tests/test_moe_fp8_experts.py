"""MoE checkpoints whose experts are stored in e4m3 (128 x 128 `weight_scale_inv` blocks, or one `weight_scale` per
tensor): the experts are dequantised with their scales at load and the model must reproduce the checkpoint whose
experts hold the dequantised values."""
import json

import pytest
import torch

from tgi_b200.models import get_model
from tgi_b200.utils.synthetic import llama_config, llama_state_dict
from tgi_b200.utils.weights import save_safetensors

FP8 = getattr(torch, "float8_e4m3fn", None)


def _logits(path, ids):
    from tgi_b200.models.decoder import ForwardMeta

    model = get_model(str(path), dtype="float32", device=torch.device("cpu"))
    model.init_kv_cache(8)
    T = len(ids)
    meta = ForwardMeta(input_ids=torch.tensor(ids, dtype=torch.int32), positions=torch.arange(T, dtype=torch.int32),
                       slots=torch.arange(16, 16 + T, dtype=torch.int32),
                       block_tables=torch.tensor([[1, 2, 3, 4]], dtype=torch.int32),
                       cu_seqlens_q=torch.tensor([0, T], dtype=torch.int32), kv_lens=torch.tensor([T], dtype=torch.int32),
                       max_q=T, max_kv=T)
    logits, _ = model.model.forward(meta, model.kv_cache)
    return logits.float()


@pytest.mark.skipif(FP8 is None, reason="no float8 dtype in this torch")
@pytest.mark.parametrize("scheme", ["block", "tensor"])
def test_fp8_experts_are_dequantised_with_their_scales(tmp_path, scheme):
    cfg = llama_config(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=96, vocab=300, max_pos=256,
                       model_type="mixtral", num_local_experts=4, num_experts_per_tok=2)
    sd = llama_state_dict(cfg, seed=3, std=0.05)
    blk = 32
    q_sd, deq_sd = {}, {}
    for name, w in sd.items():
        if ".experts." not in name:
            q_sd[name] = deq_sd[name] = w
            continue
        N, K = w.shape
        if scheme == "block":
            pad = torch.zeros(-(-N // blk) * blk, -(-K // blk) * blk)
            pad[:N, :K] = w
            amax = pad.view(pad.shape[0] // blk, blk, pad.shape[1] // blk, blk).abs().amax(dim=(1, 3)).clamp_min(1e-6)
            s = amax / 448.0
            s_el = s.repeat_interleave(blk, 0)[:N].repeat_interleave(blk, 1)[:, :K]
            q = (w / s_el).to(FP8)
            q_sd[name] = q
            q_sd[name.replace(".weight", ".weight_scale_inv")] = s
            deq_sd[name] = q.float() * s_el
        else:
            s = w.abs().max() / 448.0
            q = (w / s).to(FP8)
            q_sd[name] = q
            q_sd[name.replace(".weight", ".weight_scale")] = s.reshape(())
            deq_sd[name] = q.float() * s
    qdir, ddir = tmp_path / "q", tmp_path / "d"
    for d, state, extra in ((qdir, q_sd, True), (ddir, deq_sd, False)):
        d.mkdir()
        c = dict(cfg)
        if extra:
            c["quantization_config"] = {"quant_method": "fp8", "activation_scheme": "dynamic", "fmt": "e4m3",
                                        **({"weight_block_size": [blk, blk]} if scheme == "block" else {})}
        (d / "config.json").write_text(json.dumps(c))
        save_safetensors(state, d / "model.safetensors", {"format": "pt"})
    ids = [5, 17, 250, 33, 90, 12, 7]
    a, b = _logits(qdir, ids), _logits(ddir, ids)
    assert torch.allclose(a, b, atol=2e-4, rtol=1e-4), (a - b).abs().max()


def test_packed_integer_experts_are_dequantised_through_the_loader(tmp_path):
    """A GPTQ-packed expert projection (`qweight` / `qzeros` / `scales` / `g_idx`) loads as the dense matrix it
    encodes, whole or as a rank's slice."""
    from tgi_b200.models.decoder import _expert_weight
    from tgi_b200.utils.quantization import GPTQLoader, _pack_int32
    from tgi_b200.utils.weights import Weights, save_safetensors

    torch.manual_seed(0)
    N, K, G = 32, 128, 64
    q = torch.randint(0, 16, (K, N))
    zeros = torch.randint(1, 16, (K // G, N))
    scales = (torch.rand(K // G, N) * 0.02 + 0.001).to(torch.bfloat16)
    gi = torch.arange(K) // G
    dense = ((q.float() - zeros.float()[gi]) * scales.float()[gi]).t().contiguous()
    save_safetensors({"e.qweight": _pack_int32(q, 4, dim=0), "e.qzeros": _pack_int32(zeros - 1, 4, dim=1),
                      "e.scales": scales, "e.g_idx": gi.to(torch.int32)}, tmp_path / "model.safetensors", {"format": "pt"})
    w = Weights([tmp_path / "model.safetensors"], "cpu", torch.bfloat16, loader=GPTQLoader(4, G, False, "gptq"))
    got = _expert_weight(w, {}, "e")
    torch.testing.assert_close(got.float(), dense.to(torch.bfloat16).float(), atol=0, rtol=0)
    w.close()
