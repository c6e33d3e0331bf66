"""Fp8Linear on CPU: per-channel and per-tensor weight scales against the dequantised product."""
import pytest
import torch

from tgi_b200.models.layers import Fp8Linear


@pytest.mark.parametrize("per_channel", [True, False])
@pytest.mark.parametrize("with_out", [False, True])
def test_fp8_linear_scale_granularities(per_channel, with_out):
    torch.manual_seed(0)
    N, K, T = 256, 256, 5
    w = torch.randn(N, K) * 0.05
    scale = (w.abs().amax(1) / 448).clamp_min(1e-8) if per_channel else (w.abs().max() / 448).reshape(1)
    wq = (w / (scale[:, None] if per_channel else scale)).to(torch.float8_e4m3fn)
    bias = torch.randn(N).to(torch.bfloat16)
    lin = Fp8Linear(wq, scale, bias, torch.bfloat16)
    x = torch.randn(T, K).to(torch.bfloat16)
    want = x.float() @ (wq.float() * (scale[:, None] if per_channel else scale)).t() + bias.float()
    if with_out:
        out = torch.empty(T, N, dtype=torch.bfloat16)
        got = lin(x, out=out)
        assert got.data_ptr() == out.data_ptr()
    else:
        got = lin(x)
    assert got.dtype == torch.bfloat16
    # the activation is quantised to e4m3 per 128 values: a few percent of the output's scale
    torch.testing.assert_close(got.float(), want, atol=0.15, rtol=0.05)
