"""Sparse mixture-of-experts kernels (routing, grouping, grouped tcgen05 GEMMs, combine) against the PyTorch
fp32 oracle, including expert-parallel shares, experts without tokens, ragged sizes and CUDA-graph replay
with changing routing."""
import pytest
import torch

from tgi_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from tgi_b200.ops import cuda as K

    K.load()
    return K


def dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("T,E,k,renorm,dtype", [(1, 8, 2, True, torch.float32), (37, 8, 2, False, torch.bfloat16),
                                                (256, 64, 6, True, torch.float32), (5, 256, 8, True, torch.float32),
                                                (300, 60, 4, False, torch.float32)])
def test_topk_softmax(K, T, E, k, renorm, dtype):
    torch.manual_seed(T * E + k)
    logits = (torch.randn(T, E, device=dev()) * 3).to(dtype)
    w, ids = K.moe_topk_softmax(logits, k, renorm)
    rw, rids = ref.moe_topk_softmax(logits, k, renorm)
    assert ids.dtype == torch.int32 and torch.equal(ids.long(), rids)
    torch.testing.assert_close(w, rw, atol=1e-6, rtol=1e-5)


def _oracle(x, wgu, wd, w, ids, act, first):
    return ref.moe_experts(x.float(), wgu.float(), wd.float(), w.float(), ids.long(), act, first)


@pytest.mark.parametrize("T,E,k,H,I,first,e_local,act", [
    (1, 8, 2, 128, 64, 0, 8, "silu"),
    (7, 4, 2, 256, 96, 0, 4, "silu"),               # I not a multiple of the 128-column epilogue group
    (300, 8, 2, 512, 384, 0, 8, "silu"),            # some experts with more than one row tile
    (256, 8, 2, 1024, 1792, 0, 8, "gelu"),
    (129, 8, 2, 384, 200, 2, 3, "silu"),            # an expert-parallel share: experts 2..4 of 8, H and I ragged
    (64, 16, 4, 256, 128, 8, 8, "silu"),
    (513, 4, 1, 256, 256, 0, 4, "silu"),
])
def test_routed_experts_match_the_oracle(K, T, E, k, H, I, first, e_local, act):
    torch.manual_seed(T + E + H)
    d = dev()
    x = (torch.randn(T, H, device=d) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(e_local, 2 * I, H, device=d) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(e_local, H, I, device=d) * 0.05).to(torch.bfloat16)
    w, ids = K.moe_topk_softmax(torch.randn(T, E, device=d), k, True)
    got = K.moe_experts(x, wgu, wd, w, ids, act, first)
    torch.cuda.synchronize()
    assert K.check_status(d) == 0, "a kernel wait timed out"
    want = _oracle(x, wgu, wd, w, ids, act, first)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=3e-2)


def test_experts_without_tokens_and_all_tokens_on_one_expert(K):
    d = dev()
    torch.manual_seed(3)
    T, E, k, H, I = 200, 8, 2, 256, 128
    x = (torch.randn(T, H, device=d) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * I, H, device=d) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=d) * 0.05).to(torch.bfloat16)
    ids = torch.zeros(T, k, dtype=torch.int32, device=d)
    ids[:, 0], ids[:, 1] = 5, 1                     # experts 0, 2, 3, 4, 6, 7 get nothing
    w = torch.rand(T, k, device=d)
    got = K.moe_experts(x, wgu, wd, w, ids, "silu", 0)
    torch.testing.assert_close(got.float(), _oracle(x, wgu, wd, w, ids, "silu", 0), atol=2e-2, rtol=3e-2)
    # a rank whose experts receive nothing returns zeros
    got = K.moe_experts(x, wgu[:2].contiguous(), wd[:2].contiguous(), w, ids, "silu", 6)
    torch.cuda.synchronize()
    assert K.check_status(d) == 0
    assert float(got.float().abs().max()) == 0.0


def test_routed_experts_replay_in_a_cuda_graph_with_new_routing(K):
    d = dev()
    torch.manual_seed(11)
    T, E, k, H, I = 96, 8, 2, 256, 256
    x = (torch.randn(T, H, device=d) * 0.5).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * I, H, device=d) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=d) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, device=d)
    K.moe_experts(x, wgu, wd, *K.moe_topk_softmax(logits, k, True), "silu", 0)      # warm-up outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        w, ids = K.moe_topk_softmax(logits, k, True)
        out = K.moe_experts(x, wgu, wd, w, ids, "silu", 0)
    for seed in (1, 2):
        torch.manual_seed(seed)
        logits.copy_(torch.randn(T, E, device=d))
        x.copy_((torch.randn(T, H, device=d) * 0.5).to(torch.bfloat16))
        g.replay()
        torch.cuda.synchronize()
        assert K.check_status(d) == 0
        rw, rids = ref.moe_topk_softmax(logits, k, True)
        torch.testing.assert_close(out.float(), _oracle(x, wgu, wd, rw, rids, "silu", 0), atol=2e-2, rtol=3e-2)
