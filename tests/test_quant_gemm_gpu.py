"""Weight-only quantised GEMM (4-bit GPTQ / AWQ layouts, int8 per-channel): the fused kernel against the
dequantised fp32 product, bit-equality of its operand with the whole-matrix dequantisation, the split-K path,
activation ordering, and the memory the packed layer keeps on the device."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def _gptq_layer(N, K, group, act_order=False, awq=False, seed=0):
    """A random 4-bit layer in checkpoint layout, plus its float matrix."""
    from tgi_b200.utils.quantization import GPTQWeight, _AWQ_ORDER

    g = torch.Generator().manual_seed(seed)
    G = K // group
    q = torch.randint(0, 16, (K, N), generator=g, dtype=torch.int32)
    zeros = torch.randint(1, 15, (G, N), generator=g, dtype=torch.int32)
    scales = (torch.rand(G, N, generator=g) * 0.02 + 0.002).to(torch.float16)
    g_idx = torch.arange(K) // group
    if act_order:
        g_idx = g_idx[torch.randperm(K, generator=g)]
    w = ((q.float() - zeros[g_idx].float()) * scales.float()[g_idx]).t().contiguous()      # [N, K]
    if awq:
        order = torch.tensor(_AWQ_ORDER)
        qw = torch.zeros(K, N // 8, dtype=torch.int32)
        qz = torch.zeros(G, N // 8, dtype=torch.int32)
        qv, zv = q.view(K, N // 8, 8)[:, :, order], zeros.view(G, N // 8, 8)[:, :, order]
        for j in range(8):
            qw |= qv[:, :, j] << (4 * j)
            qz |= zv[:, :, j] << (4 * j)
        return GPTQWeight(qw.to(dev()), qz.to(dev()), scales.to(dev()), None, 4, group, awq=True), w
    qw = torch.zeros(K // 8, N, dtype=torch.int32)
    for j in range(8):
        qw |= q[j::8] << (4 * j)
    qz = torch.zeros(G, N // 8, dtype=torch.int32)
    zm1 = zeros - 1                                   # GPTQ stores the zero point minus one
    for j in range(8):
        qz |= zm1[:, j::8] << (4 * j)
    return GPTQWeight(qw.to(dev()), qz.to(dev()), scales.to(dev()), g_idx.to(torch.int32).to(dev()), 4, group), w


@pytest.mark.parametrize("M", [1, 33, 128, 256, 300])
@pytest.mark.parametrize("N,K,group,act_order,awq", [(256, 512, 128, False, False), (1280, 4096, 128, False, False),
                                                     (384, 1024, 64, True, False), (512, 2048, 128, False, True),
                                                     (8192, 1024, 1024, False, False)])
def test_w4a16_matches_the_dequantised_product(M, N, K, group, act_order, awq):
    from tgi_b200.models.layers import PackedQuantLinear
    from tgi_b200.ops import cuda as Kc

    Kc.load()
    wt, w = _gptq_layer(N, K, group, act_order, awq, seed=N + K)
    lin = wt.get_linear(None)
    assert isinstance(lin, PackedQuantLinear) and lin.wq.dtype == torch.uint8 and tuple(lin.wq.shape) == (N, K // 2)
    torch.testing.assert_close(lin.weight.float().cpu(), w.to(torch.bfloat16).float(), atol=0, rtol=0)
    x = torch.randn(M, K, device=dev(), dtype=torch.bfloat16)
    got = lin(x)
    torch.cuda.synchronize()
    assert Kc.check_status(dev()) == 0, "a kernel wait timed out"
    # the op itself: tokens times the exact dequantised weights in fp32; the fused kernel rounds the weights to fp16
    # and the output to bf16, the large-step path rounds the weights to bf16
    want = x.float() @ w.float().to(dev()).t()
    torch.testing.assert_close(got.float(), want, atol=3e-2 * math.sqrt(K / 512), rtol=2e-2)


def test_int8_per_channel_and_bias_and_large_step():
    from tgi_b200.models.layers import PackedQuantLinear
    from tgi_b200.ops import cuda as Kc
    from tgi_b200.utils.quantization import Int8Weight

    torch.manual_seed(1)
    N, K = 768, 2048
    w = torch.randn(N, K, device=dev()) * 0.05
    bias = torch.randn(N, device=dev()).to(torch.bfloat16)
    lin = Int8Weight.quantize(w, torch.bfloat16).get_linear(bias)
    assert isinstance(lin, PackedQuantLinear) and lin.bits == 8 and lin.wq.dtype == torch.int8
    wd = lin.dequantize().float()
    for M in (5, 200, 700):          # 700 rows: dequantise to scratch + bf16 GEMM
        x = torch.randn(M, K, device=dev(), dtype=torch.bfloat16)
        got = lin(x)
        torch.cuda.synchronize()
        assert Kc.check_status(dev()) == 0
        torch.testing.assert_close(got.float(), x.float() @ wd.t() + bias.float(), atol=6e-2, rtol=2e-2)


def test_packed_layer_keeps_a_quarter_of_the_bf16_bytes():
    wt, _ = _gptq_layer(4096, 4096, 128)
    lin = wt.get_linear(None)
    held = lin.wq.numel() * lin.wq.element_size() + lin.scale.numel() * 2 + lin.zp.numel() * 2
    assert held < 0.3 * 4096 * 4096 * 2
    assert not hasattr(lin, "_dense")
