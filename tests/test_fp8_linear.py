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


def test_requantisation_to_power_of_two_block_scales():
    """The scale-factor MMA takes E8M0 scales: every block scale is rounded up to a power of two and the values are
    re-rounded to e4m3, so that the represented matrix moves by at most one e4m3 rounding step."""
    from tgi_b200.ops.cuda import requant_block_pow2

    torch.manual_seed(1)
    N, K = 300, 384                                   # a ragged last row block
    w = torch.randn(N, K) * 0.05
    nb, kb = (N + 127) // 128, K // 128
    scale = torch.empty(nb, kb)
    wq = torch.empty(N, K, dtype=torch.float8_e4m3fn)
    for i in range(nb):
        for j in range(kb):
            blk = w[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128]
            scale[i, j] = blk.abs().max() / 448
            wq[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128] = (blk / scale[i, j]).to(torch.float8_e4m3fn)
    scale[0, 0] = 0.25                                # already a power of two: must stay as it is
    wq2, s2 = requant_block_pow2(wq, scale)
    mant, _ = torch.frexp(s2)
    assert torch.all(mant == 0.5), "scales are powers of two"
    assert torch.all(s2 >= scale) and torch.all(s2 < 2 * scale) and s2[0, 0] == 0.25
    assert torch.equal(wq2[:128, :128].float(), wq[:128, :128].float())
    full = lambda q, s: q.float() * s.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)     # noqa: E731
    before, after = full(wq, scale), full(wq2, s2)
    # one e4m3 step is 2^-3 relative (2^-4 after rounding to nearest); values near zero fall into the subnormal grid
    err = (after - before).abs()
    assert torch.all(err <= before.abs() * 2.0 ** -4 + s2.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1) * 2.0 ** -10)
