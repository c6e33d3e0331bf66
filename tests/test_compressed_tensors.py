"""compressed-tensors pack-quantized int4 layers: loaded into the packed form the weight-only GEMM serves (GPTQ layout),
symmetric and with zero points, whole, column-fused and row-sharded."""
import torch

from tgi_b200.utils.quantization import CompressedTensorsLoader, GPTQWeight, _pack_int32, _unpack_int32
from tgi_b200.utils.weights import Weights, save_safetensors

CFG = {"format": "pack-quantized", "config_groups": {"group_0": {
    "targets": ["Linear"], "weights": {"num_bits": 4, "type": "int", "symmetric": True, "strategy": "group", "group_size": 64}}},
    "ignore": ["lm_head"]}


def _layer(N, K, G, asym, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (N, K), generator=g)
    scale = torch.rand(N, K // G, generator=g) * 0.02 + 0.001
    zp = torch.randint(5, 11, (N, K // G), generator=g) if asym else torch.full((N, K // G), 8)
    dense = (q.float() - zp.float().repeat_interleave(G, 1)) * scale.repeat_interleave(G, 1)
    t = {"weight_packed": _pack_int32(q, 4, dim=1), "weight_scale": scale.to(torch.bfloat16)}
    if asym:
        t["weight_zero_point"] = _pack_int32(zp, 4, dim=0)
    dense = (q.float() - zp.float().repeat_interleave(G, 1)) * scale.to(torch.bfloat16).float().repeat_interleave(G, 1)
    return t, dense


def test_pack_unpack_round_trip():
    v = torch.randint(0, 16, (16, 24))
    assert torch.equal(_unpack_int32(_pack_int32(v, 4, dim=0), 4, dim=0), v.to(torch.int32))
    assert torch.equal(_unpack_int32(_pack_int32(v, 4, dim=1), 4, dim=1), v.to(torch.int32))


def test_pack_quantized_layers_load_into_the_packed_form(tmp_path):
    layers = {"a": _layer(64, 128, 64, False, 0), "b": _layer(32, 128, 64, False, 1), "z": _layer(64, 128, 64, True, 2)}
    tensors = {f"{name}.{k}": v for name, (t, _) in layers.items() for k, v in t.items()}
    save_safetensors(tensors, tmp_path / "model.safetensors", {"format": "pt"})
    loader = CompressedTensorsLoader(CFG)
    w = Weights([tmp_path / "model.safetensors"], "cpu", torch.bfloat16, loader=loader)
    for name in ("a", "z"):
        got = loader.get_weights(w, name)
        assert isinstance(got, GPTQWeight) and got.bits == 4 and got.groupsize == 64
        torch.testing.assert_close(got.dequantize().float(), layers[name][1], atol=1e-6, rtol=1e-6)
    fused = loader.get_multi_weights_col(w, ["a", "b"], 0)
    assert isinstance(fused, GPTQWeight)
    torch.testing.assert_close(fused.dequantize().float(), torch.cat([layers["a"][1], layers["b"][1]]), atol=1e-6, rtol=1e-6)
    row = loader.get_weights_row(w, "a")
    torch.testing.assert_close(row.dequantize().float(), layers["a"][1], atol=1e-6, rtol=1e-6)
    lin = got.get_linear(None)           # CPU: the dequantised fallback of the packed linear
    x = torch.randn(3, 128).to(torch.bfloat16)
    torch.testing.assert_close(lin(x).float(), x.float() @ layers["z"][1].t(), atol=0.05, rtol=0.05)
    w.close()
