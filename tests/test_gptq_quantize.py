"""GPTQ calibration round trip on CPU: quantise a tiny Llama to 4 bits, load the result through the
GPTQ loader, and compare with the full-precision model; also the packing against the loader's unpacking."""
import json

import pytest
import torch

pytest.importorskip("transformers")

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.decoder import ForwardMeta  # noqa: E402
from tgi_b200.utils import gptq_quantize as gq  # noqa: E402
from tgi_b200.utils.quantization import GPTQWeight, dequantize_gptq  # noqa: E402
from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint  # noqa: E402


def test_pack_matches_loader_unpack():
    g = torch.Generator().manual_seed(0)
    out_f, in_f, gs = 16, 64, 32
    qint = torch.randint(0, 16, (out_f, in_f), generator=g, dtype=torch.int32)
    scales = torch.rand(in_f // gs, out_f, generator=g) * 0.1 + 0.01
    zeros = torch.randint(1, 16, (in_f // gs, out_f), generator=g, dtype=torch.int32)
    g_idx = (torch.arange(in_f) // gs).to(torch.int32)
    t = gq.pack(qint, scales, zeros, g_idx, 4)
    w = GPTQWeight(t["qweight"], t["qzeros"], t["scales"], t["g_idx"], 4, gs, False, False, torch.float32)
    deq = dequantize_gptq(w)
    gi = g_idx.long()
    want = (qint.float() - zeros.float()[gi].t()) * scales.half().float()[gi].t()
    torch.testing.assert_close(deq, want, atol=1e-3, rtol=1e-3)


def test_solver_beats_round_to_nearest():
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 48, bias=False)
    x = torch.randn(512, 64) @ torch.randn(64, 64) * 0.3          # correlated inputs
    ref = lin(x).detach()
    solver = gq.GPTQ(lin)
    solver.add_batch(x)
    w0 = lin.weight.data.clone()
    solver.fasterquant(bits=3, groupsize=32, act_order=True, percdamp=0.01, sym=False)
    err_gptq = (lin(x) - ref).pow(2).mean().item()
    q = gq._Quantizer(3, False)
    rtn = torch.zeros_like(w0)
    for c in range(0, 64, 32):
        q.find_params(w0[:, c:c + 32])
        rtn[:, c:c + 32] = q.quantize(w0[:, c:c + 32])[0]
    err_rtn = (x @ rtn.t() - ref).pow(2).mean().item()
    assert err_gptq < err_rtn


def test_quantize_cli_round_trip(tmp_path):
    cfg = llama_config(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=128, vocab=320, max_pos=256)
    src = tmp_path / "fp"
    write_llama_checkpoint(src, cfg, std=0.05)
    out = gq.quantize(str(src), str(tmp_path / "q4"), bits=4, groupsize=32, act_order=False, nsamples=8, seqlen=32,
                      device="cpu")
    qc = json.loads((out / "quantize_config.json").read_text())
    assert qc["bits"] == 4 and qc["group_size"] == 32 and qc["quant_method"] == "gptq"
    full = get_model(str(src), dtype="float32", device=torch.device("cpu"))
    quant = get_model(str(out), dtype="float32", device=torch.device("cpu"), quantize="gptq")
    ids = torch.arange(3, 27, dtype=torch.int32)
    outs = []
    for m in (full, quant):
        m.init_kv_cache(4)
        meta = ForwardMeta(input_ids=ids, positions=torch.arange(24, dtype=torch.int32),
                           slots=torch.arange(16, 40, dtype=torch.int32), block_tables=torch.tensor([[1, 2]], dtype=torch.int32),
                           cu_seqlens_q=torch.tensor([0, 24], dtype=torch.int32), kv_lens=torch.tensor([24], dtype=torch.int32),
                           max_q=24, max_kv=24)
        outs.append(m.forward(meta).float())
    rel = (outs[0] - outs[1]).norm() / outs[0].norm()
    assert rel < 0.2, f"4-bit model deviates by {rel:.3f}"
    assert rel > 0, "quantised checkpoint is identical to the original: nothing was quantised"
