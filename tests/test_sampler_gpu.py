"""Fused sampler kernel against the sort-based PyTorch warpers: supports of top-k / top-p, argmax rows,
log-probabilities, distribution of the draws, and reproducibility per (seed, step)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_filtered(scores, temperature, top_k, top_p):
    from tgi_b200.utils.tokens import top_k_filter, top_p_filter

    x = scores.float() / temperature.view(-1, 1)
    x = top_k_filter(x, top_k)
    x = top_p_filter(x, top_p)
    return x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_supports_logprobs_and_greedy_rows(dtype):
    from tgi_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cuda").manual_seed(0)
    B, V = 64, 32003
    scores = (torch.randn(B, V, device=dev, generator=g) * 3).to(dtype)
    temperature = torch.rand(B, device=dev, generator=g) * 1.5 + 0.3
    top_k = torch.randint(0, 200, (B,), device=dev, generator=g, dtype=torch.int32)
    top_k[::5] = 0
    top_p = torch.rand(B, device=dev, generator=g) * 0.6 + 0.4
    top_p[::7] = 1.0
    do_sample = torch.ones(B, dtype=torch.uint8, device=dev)
    do_sample[::2] = 0
    seeds = torch.arange(B, device=dev, dtype=torch.int64) * 7919 + 13
    steps = torch.zeros(B, dtype=torch.int32, device=dev)
    want = _torch_filtered(scores, temperature, top_k, top_p)
    want_lp = torch.log_softmax(want, -1)
    for step in range(4):
        steps.fill_(step)
        ids, lps = ops.fused_sample(scores, temperature, top_k, top_p, do_sample, seeds, steps)
        torch.cuda.synchronize()
        # support check by value: with repeated values (bf16) the sort-based filter cuts through a group of
        # equal scores in sort order while the kernel keeps the whole group, so compare against the smallest
        # kept value instead of the exact index set
        x = scores.float() / temperature.view(-1, 1)
        picked = x.gather(1, ids.view(-1, 1)).view(-1)
        floor = torch.where(torch.isfinite(want), want, torch.full_like(want, float("inf"))).min(-1).values
        assert (picked >= floor - 1e-6).all(), "a sampled token lies outside the top-k / top-p support"
        ref_lp = torch.log_softmax(torch.where(x >= floor.view(-1, 1) - 1e-6, x, torch.full_like(x, -float("inf"))), -1)
        ref_lp = ref_lp.gather(1, ids.view(-1, 1)).view(-1)
        assert (lps - ref_lp).abs().max().item() < 3e-3
        greedy = do_sample == 0
        assert torch.equal(x.gather(1, ids.view(-1, 1)).view(-1)[greedy], x.max(-1).values[greedy])
    again, _ = ops.fused_sample(scores, temperature, top_k, top_p, do_sample, seeds, steps)
    assert torch.equal(again, ids), "same seed and step must reproduce the draw"
    steps.fill_(99)
    other, _ = ops.fused_sample(scores, temperature, top_k, top_p, do_sample, seeds, steps)
    assert (other != ids)[do_sample == 1].any()


def test_draws_follow_the_distribution():
    from tgi_b200 import ops

    dev = torch.device("cuda", 0)
    V, N = 40, 40000
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(V, device=dev, generator=g) * 1.5
    scores = logits.view(1, V).expand(N, V).contiguous()
    temperature = torch.full((N,), 0.8, device=dev)
    top_k = torch.full((N,), 12, dtype=torch.int32, device=dev)
    top_p = torch.full((N,), 0.9, device=dev)
    do_sample = torch.ones(N, dtype=torch.uint8, device=dev)
    seeds = torch.full((N,), 1234, dtype=torch.int64, device=dev)
    steps = torch.arange(N, dtype=torch.int32, device=dev)      # one request, N consecutive steps
    ids, _ = ops.fused_sample(scores, temperature, top_k, top_p, do_sample, seeds, steps)
    probs = torch.softmax(_torch_filtered(scores[:1], temperature[:1], top_k[:1], top_p[:1]), -1).view(-1)
    freq = torch.bincount(ids, minlength=V).float() / N
    assert (freq[probs == 0] == 0).all()
    # every kept token within 4 standard errors (plus a small absolute slack) of its probability
    se = torch.sqrt(probs * (1 - probs) / N)
    assert ((freq - probs).abs() <= 4 * se + 2e-3).all(), (freq, probs)


def test_chooser_uses_the_kernel_and_matches_filters():
    from tgi_b200.proto import generate_v3 as pb
    from tgi_b200.utils.tokens import NextTokenChooser

    dev = torch.device("cuda", 0)
    params = []
    for i in range(6):
        p = pb.NextTokenChooserParameters(temperature=(0.7 + 0.1 * i) if i else 1.0, top_k=20 if i % 2 else 0, top_p=0.9 if i % 3 else 1.0,
                                          typical_p=1.0, do_sample=i != 0, seed=100 + i, repetition_penalty=1.2 if i == 2 else 1.0,
                                          frequency_penalty=0.0, watermark=False)
        params.append(p)
    chooser = NextTokenChooser.from_pb(params, dev, None)
    g = torch.Generator(device="cuda").manual_seed(2)
    scores = (torch.randn(6, 5000, device=dev, generator=g) * 2).to(torch.bfloat16)
    history = torch.randint(0, 5000, (6, 9), device=dev, generator=g)
    ids, lps, all_lp, accepted, spec = chooser(history, scores, 0, None, None, need_logprobs=False)
    assert all_lp is None and spec is None and accepted.tolist() == [1] * 6
    warped = chooser.warp(history, scores.float().clone())
    assert torch.isfinite(warped.gather(1, ids.view(-1, 1))).all()
    assert warped[0, ids[0]].item() == warped[0].max().item()      # bf16 scores repeat: compare the value, not the index
    ref = torch.log_softmax(warped, -1).gather(1, ids.view(-1, 1)).view(-1)
    assert (lps - ref).abs().max().item() < 8e-2      # equal bf16 scores at the top-p boundary: the kernel keeps the whole group
    assert chooser.steps == [0, 1, 1, 1, 1, 1]


def test_penalties_kernel_matches_the_torch_warpers():
    from tgi_b200.ops import cuda as K
    from tgi_b200.utils.tokens import apply_frequency_penalty, apply_repetition_penalty

    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    B, V, L = 9, 3000, 57
    logits = (torch.randn(B, V, device=dev) * 4).to(torch.bfloat16)
    hist = torch.randint(0, V, (B, L), device=dev)
    hist[:, -7:] = 0                                  # padding zeros count as token 0, as in the reference
    rep = torch.rand(B, device=dev) * 0.6 + 1.0
    rep[0] = 1.0
    freq = torch.rand(B, device=dev) * 0.5
    freq[1] = 0.0
    got = K.penalties(logits, hist, rep, freq)
    want = apply_frequency_penalty(apply_repetition_penalty(logits.float(), hist, rep), hist, freq)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    # a vocabulary slice sees only its own ids
    lo, hi = 1000, 2200
    part = K.penalties(logits[:, lo:hi].contiguous(), hist, rep, freq, vocab_start=lo)
    torch.testing.assert_close(part, want[:, lo:hi], atol=1e-5, rtol=1e-5)
    assert torch.equal(K.penalties(logits, hist, None, None), logits.float())


def test_sharded_sampler_with_one_rank_equals_the_fused_sampler():
    """The vocabulary-parallel sampler run with a single rank (it exchanges its words with itself) must pick
    the same tokens and log-probabilities as the single-GPU kernel for the same seeds."""
    from tgi_b200.ops import cuda as K
    from tgi_b200.parallel.dist import FakeGroup
    from tgi_b200.parallel.peer import PeerComm

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    comm = PeerComm(FakeGroup(0, 1), 0, 1, dev, 64, 256)
    g = torch.Generator(device="cpu").manual_seed(17)
    for B, V in ((1, 300), (40, 5000), (300, 2048)):
        logits = (torch.randn(B, V, generator=g) * 3).to(torch.bfloat16).to(dev)
        temperature = torch.rand(B, generator=g) * 1.5 + 0.3
        top_k = torch.randint(0, 50, (B,), generator=g, dtype=torch.int32)
        top_k[::2] = 0
        top_p = torch.rand(B, generator=g) * 0.7 + 0.3
        top_p[::5] = 1.0
        do_sample = (torch.rand(B, generator=g) < 0.7).to(torch.uint8)
        seeds = torch.randint(0, 2 ** 40, (B,), generator=g, dtype=torch.int64)
        steps = torch.randint(0, 9, (B,), generator=g, dtype=torch.int32)
        want_ids, want_lp = K.fused_sample(logits, temperature, top_k, top_p, do_sample, seeds, steps)
        for _ in range(2):       # twice: the exchange counters keep counting across launches
            ids, lps = comm.sample(logits, 0, V, 1.0, temperature, top_k, top_p, do_sample, seeds, steps)
            torch.cuda.synchronize()
            assert comm.check() == 0
            assert (ids == want_ids).float().mean().item() >= 0.99
            ok = ids == want_ids
            assert (lps[ok] - want_lp[ok]).abs().max().item() < 2e-3
    comm.close()


def test_typical_p_support_matches_the_torch_filter():
    """Typical-p after top-k: every draw must lie in the set the sort-based filter keeps, the log-probability is
    the renormalised one over that set, and greedy rows take the best kept entry."""
    from tgi_b200 import ops
    from tgi_b200.utils.tokens import top_k_filter, typical_p_filter

    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cuda").manual_seed(3)
    B, V = 48, 5003
    scores = torch.randn(B, V, device=dev, generator=g) * 2.5
    temperature = torch.rand(B, device=dev, generator=g) + 0.5
    top_k = torch.randint(0, 400, (B,), device=dev, generator=g, dtype=torch.int32)
    top_k[::3] = 0
    typical = torch.rand(B, device=dev, generator=g) * 0.7 + 0.2
    typical[::6] = 1.0
    do_sample = torch.ones(B, dtype=torch.uint8, device=dev)
    do_sample[::4] = 0
    seeds = torch.arange(B, device=dev, dtype=torch.int64) + 100
    want = typical_p_filter(top_k_filter(scores / temperature.view(-1, 1), top_k), typical)
    want_lp = torch.log_softmax(want, -1)
    kept = torch.isfinite(want)
    assert (kept.sum(-1) < V).any() and (kept.sum(-1) > 1).any()
    for step in range(6):
        steps = torch.full((B,), step, dtype=torch.int32, device=dev)
        ids, lps = ops.fused_sample(scores, temperature, top_k, None, do_sample, seeds, steps, typical_p=typical)
        torch.cuda.synchronize()
        assert kept.gather(1, ids.view(-1, 1)).all(), "a draw lies outside the typical set"
        assert (lps - want_lp.gather(1, ids.view(-1, 1)).view(-1)).abs().max().item() < 3e-3
        greedy = do_sample == 0
        assert torch.equal(ids[greedy], want.argmax(-1)[greedy])
