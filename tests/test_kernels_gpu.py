"""Numerics of every sm_100a kernel against the plain PyTorch fp32 oracle (`ops/reference.py`)."""
import math

import pytest
import torch

from tgi_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def K():
    from tgi_b200.ops import cuda as K

    K.load()
    return K


@pytest.fixture(autouse=True)
def promote_path_by_default(K):
    """The kernel tests hand arbitrary (not power-of-two) block scales to the fp8 GEMM: they exercise the promotion
    path; the scale-factor MMA has its own test, which switches it on."""
    was = K.fp8_mx()
    K.set_fp8_mx(False)
    yield
    K.set_fp8_mx(was)


def dev():
    return torch.device("cuda", 0)


def no_kernel_error(K):
    torch.cuda.synchronize()
    assert K.check_status(dev()) == 0, "a kernel wait timed out"


@pytest.mark.parametrize("M,N,K_", [(1, 256, 512), (7, 384, 1024), (33, 1280, 4096), (64, 128, 64), (100, 512, 2048),
                                    (128, 4096, 4096), (200, 640, 8192), (256, 1024, 3584), (300, 768, 1024),
                                    (1000, 2048, 2048)])
def test_gemm_bf16(K, M, N, K_):
    torch.manual_seed(M * 131 + N)
    x = torch.randn(M, K_, device=dev(), dtype=torch.bfloat16)
    w = (torch.randn(N, K_, device=dev()) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device=dev(), dtype=torch.bfloat16)
    want = x.float() @ w.float().t() + b.float()
    for ctas in (None, 1, 37):
        got = K.gemm_bf16(x, w, b, max_ctas=ctas)
        no_kernel_error(K)
        torch.testing.assert_close(got.float(), want, atol=2e-2 * math.sqrt(K_ / 512), rtol=2e-2)


@pytest.mark.parametrize("M,N,K_", [(1, 256, 512), (16, 384, 1024), (48, 1280, 4096), (100, 512, 2048),
                                    (128, 4096, 4096), (256, 1024, 3584), (256, 2048, 8192), (513, 768, 1024),
                                    (256, 10240, 8192), (64, 8192, 28672)])
def test_gemm_fp8_block(K, M, N, K_):
    torch.manual_seed(M * 17 + N)
    x = torch.randn(M, K_, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(N, K_, device=dev()) * 0.05
    wq, ws = ref.fp8_quant_block_weight(w)
    xq, xs = K.fp8_quant_act(x)
    rq, rs = ref.fp8_quant_act(x)
    mismatch = (xq.view(torch.uint8) != rq.view(torch.uint8)).float().mean().item()
    assert mismatch < 3e-2, f"quantised bytes differ from the oracle in {mismatch:.4%} of the elements"
    torch.testing.assert_close(xs, rs, atol=1e-7, rtol=1e-5)
    # the GEMM is checked on the kernel's own quantised operands so that it is tested in isolation
    want = ref.gemm_fp8_block(xq, xs.contiguous(), wq, ws, torch.float32)
    for ctas in (None, 1, 37):
        got = K.gemm_fp8_block(xq, xs, wq, ws, max_ctas=ctas)
        no_kernel_error(K)
        torch.testing.assert_close(got.float(), want, atol=3e-2 * math.sqrt(K_ / 512), rtol=2e-2)


@pytest.mark.parametrize("M,N,K_", [(1, 256, 512), (16, 384, 1024), (100, 512, 2048), (128, 4096, 4096), (256, 1024, 3584),
                                    (256, 2048, 8192), (513, 768, 1024), (256, 10240, 8192), (64, 8192, 28672),
                                    (2048, 1280, 8192)])
def test_gemm_fp8_block_scaled_mma(K, M, N, K_):
    """Block-scaled fp8 on the scale-factor MMA: activation scales come out of the quantiser as powers of two,
    weights are requantised to power-of-two block scales, and the product must match the fp32 product of the
    dequantised operands (whole tiles, K splits and stream-K splits)."""
    torch.manual_seed(M * 13 + N)
    x = torch.randn(M, K_, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(N, K_, device=dev()) * 0.05
    wq0, ws0 = ref.fp8_quant_block_weight(w)
    K.set_fp8_mx(True)
    try:
        wq, ws = K.requant_block_pow2(wq0, ws0)
        assert (torch.frexp(ws)[0] == 0.5).all()
        xq, xs = K.fp8_quant_act(x)
        assert (torch.frexp(xs)[0] == 0.5).all(), "activation scales are not powers of two"
        # the power-of-two scale is at most twice the tight one: the row still uses at least half of the e4m3 range
        deq = xq.float().view(M, K_ // 128, 128) * xs.float().unsqueeze(-1)
        assert (deq.view(M, K_) - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
        want = ref.gemm_fp8_block(xq, xs.contiguous(), wq, ws, torch.float32)
        for ctas in (None, 1, 37):
            got = K.gemm_fp8_block(xq, xs, wq, ws, max_ctas=ctas)
            no_kernel_error(K)
            torch.testing.assert_close(got.float(), want, atol=3e-2 * math.sqrt(K_ / 512), rtol=2e-2)
    finally:
        K.set_fp8_mx(False)


@pytest.mark.parametrize("M,N,K_", [(129, 256, 256), (256, 256, 128), (256, 130 * 8, 512), (257, 7168, 8192),
                                    (512, 28672, 1024), (2048, 1280, 8192)])
def test_gemm_fp8_block_scaled_mma_on_cta_pairs(K, M, N, K_):
    """The scale-factor MMA on 256 x 256 pair tiles: each CTA writes the scale factors of its own tokens and of all
    256 weight rows into its TMEM."""
    torch.manual_seed(M + 3 * N + K_)
    x = torch.randn(M, K_, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(N, K_, device=dev()) * 0.05
    wq0, ws0 = ref.fp8_quant_block_weight(w)
    lib = K.load()
    K.set_fp8_mx(True)
    lib.tgi_gemm_set_mx_pairs(1)
    lib.tgi_gemm_set_pair_min_tiles(1)
    try:
        wq, ws = K.requant_block_pow2(wq0, ws0)
        xq, xs = K.fp8_quant_act(x)
        want = ref.gemm_fp8_block(xq, xs.contiguous(), wq, ws, torch.float32)
        for ctas in (None, 2, 38):
            got = K.gemm_fp8_block(xq, xs, wq, ws, max_ctas=ctas)
            no_kernel_error(K)
            assert lib.tgi_gemm_last_grid() % 2 == 0, "the launch did not use CTA pairs"
            torch.testing.assert_close(got.float(), want, atol=3e-2 * math.sqrt(K_ / 512), rtol=2e-2)
    finally:
        lib.tgi_gemm_set_pair_min_tiles(32)
        K.set_fp8_mx(False)


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("M,N,K_", [(129, 256, 256), (256, 256, 128), (256, 130 * 8, 512), (257, 7168, 8192),
                                    (512, 28672, 1024), (2048, 1280, 8192)])
def test_gemm_tile_configurations(K, pairs, M, N, K_):
    """More than 128 tokens: CTA pairs on 256 x 256 tiles (default) and single CTAs on 256 x 128 tiles must
    both match the oracle, for whole tiles, aligned K splits and stream-K splits, bf16 and block-scaled fp8."""
    torch.manual_seed(M + N + K_)
    x = torch.randn(M, K_, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(N, K_, device=dev()) * 0.05
    K.set_gemm_pairs(pairs)
    K.load().tgi_gemm_set_pair_min_tiles(1)      # small test shapes too
    try:
        wb = w.to(torch.bfloat16)
        want = x.float() @ wb.float().t()
        for ctas in (None, 2, 37, 74):
            got = K.gemm_bf16(x, wb, None, max_ctas=ctas)
            no_kernel_error(K)
            torch.testing.assert_close(got.float(), want, atol=2e-2 * math.sqrt(K_ / 512), rtol=2e-2)
        if K_ % 128 == 0 and N % 128 == 0:
            wq, ws = ref.fp8_quant_block_weight(w)
            xq, xs = K.fp8_quant_act(x)
            want8 = ref.gemm_fp8_block(xq, xs.contiguous(), wq, ws, torch.float32)
            for ctas in (None, 2, 37, 74):
                got = K.gemm_fp8_block(xq, xs, wq, ws, max_ctas=ctas)
                no_kernel_error(K)
                torch.testing.assert_close(got.float(), want8, atol=3e-2 * math.sqrt(K_ / 512), rtol=2e-2)
    finally:
        K.set_gemm_pairs(True)
        K.load().tgi_gemm_set_pair_min_tiles(32)


@pytest.mark.parametrize("T,H", [(1, 256), (5, 4096), (33, 8192), (4, 5120), (3, 16384)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm(K, T, H, with_res):
    torch.manual_seed(T + H)
    x = torch.randn(T, H, device=dev(), dtype=torch.bfloat16)
    r = torch.randn(T, H, device=dev(), dtype=torch.bfloat16) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device=dev())).to(torch.bfloat16)
    for off in (False, True):
        got, gres = K.rms_norm(x, r, w, 1e-5, off)
        want, wres = ref.rms_norm(x, r, w, 1e-5, off)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(gres.float(), wres.float(), atol=0, rtol=0)
    if H % 128 == 0:
        q, s, qres = K.rms_norm_quant(x, r, w, 1e-5, False)
        y, _ = ref.rms_norm(x, r, w, 1e-5, False)
        rq, rs = ref.fp8_quant_act(y)
        torch.testing.assert_close(s, rs, atol=1e-6, rtol=2e-2)
        deq = q.float() * s.repeat_interleave(128, dim=1)
        torch.testing.assert_close(deq, y.float(), atol=0.08, rtol=0.08)
    no_kernel_error(K)


def test_layer_norm(K):
    torch.manual_seed(0)
    x = torch.randn(9, 2048, device=dev(), dtype=torch.bfloat16)
    r = torch.randn(9, 2048, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(2048, device=dev(), dtype=torch.bfloat16)
    b = torch.randn(2048, device=dev(), dtype=torch.bfloat16)
    got, gres = K.layer_norm(x, r, w, b, 1e-5)
    want, wres = ref.layer_norm(x, r, w, b, 1e-5)
    torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(gres.float(), wres.float(), atol=0, rtol=0)


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh"])
def test_act_and_mul(K, act):
    torch.manual_seed(1)
    gu = torch.randn(37, 2 * 1792, device=dev(), dtype=torch.bfloat16)
    got = K.act_and_mul(gu, act)
    want = ref.act_and_mul(gu, act)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    q, s = K.act_and_mul_quant(gu, act)
    deq = q.float() * s.repeat_interleave(128, dim=1)
    torch.testing.assert_close(deq, want.float(), atol=0.1, rtol=0.08)


def test_act_and_mul_width_not_a_multiple_of_16(K):
    """An intermediate size of 8 (mod 16) takes the kernel instance with one 16-byte vector per thread."""
    torch.manual_seed(4)
    gu = torch.randn(5, 2 * 1800, device=dev(), dtype=torch.bfloat16)
    torch.testing.assert_close(K.act_and_mul(gu, "silu").float(), ref.act_and_mul(gu, "silu").float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("fp8_cache", [False, True])
@pytest.mark.parametrize("neox,rot", [(True, 128), (False, 128), (True, 64)])
def test_rope_and_cache(K, fp8_cache, neox, rot):
    torch.manual_seed(2)
    T, Hq, Hkv, D = 19, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev(), dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=dev(), dtype=torch.int32)
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    fr = torch.outer(torch.arange(512, dtype=torch.float32), inv)
    cos_sin = torch.cat([fr.cos(), fr.sin()], -1).to(dev())
    slots = torch.randperm(4 * 16, device=dev())[:T].to(torch.int32)
    dt = FP8 if fp8_cache else torch.bfloat16
    ks = torch.tensor([0.5, 2.0], device=dev()) if fp8_cache else None
    vs = torch.tensor([1.5, 0.25], device=dev()) if fp8_cache else None
    caches = []
    for impl in (K, ref):
        kc = torch.zeros(4, 16, Hkv, D, device=dev(), dtype=dt)
        vc = torch.zeros(4, 16, Hkv, D, device=dev(), dtype=dt)
        q = impl.rope_and_cache(qkv.clone(), pos, cos_sin, slots, kc, vc, Hq, Hkv, D, rot, neox, ks, vs)
        caches.append((q, kc, vc))
    (q1, k1, v1), (q2, k2, v2) = caches
    torch.testing.assert_close(q1.float(), q2.float(), atol=2e-2, rtol=2e-2)
    tol = dict(atol=0.13, rtol=0.13) if fp8_cache else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(k1.float(), k2.float(), **tol)
    torch.testing.assert_close(v1.float(), v2.float(), **tol)


def _attention_case(K, B, q_lens, kv_lens, Hq, Hkv, D, fp8, window=-1, softcap=0.0, nsplit=None, spans=None):
    torch.manual_seed(B * 7 + Hq)
    bs = 16
    nblocks = sum((l + bs - 1) // bs for l in kv_lens) + 2
    dt = FP8 if fp8 else torch.bfloat16
    kc = (torch.randn(nblocks, bs, Hkv, D, device=dev()) * (4.0 if fp8 else 1.0)).to(dt)
    vc = (torch.randn(nblocks, bs, Hkv, D, device=dev()) * (4.0 if fp8 else 1.0)).to(dt)
    maxb = max((l + bs - 1) // bs for l in kv_lens)
    perm = torch.randperm(nblocks - 1) + 1
    bt = torch.zeros(B, maxb, dtype=torch.int32)
    cur = 0
    for i, l in enumerate(kv_lens):
        nb = (l + bs - 1) // bs
        bt[i, :nb] = perm[cur:cur + nb].to(torch.int32)
        cur += nb
    bt = bt.to(dev())
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device=dev(), dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev())
    kl = torch.tensor(kv_lens, dtype=torch.int32, device=dev())
    ks = (torch.rand(Hkv, device=dev()) * 0.2 + 0.15) if fp8 else None
    vs = (torch.rand(Hkv, device=dev()) * 0.2 + 0.15) if fp8 else None
    scale = D ** -0.5
    horizon = None
    if spans is not None:
        # rows whose position falls in a span [a, b) of their sequence see the whole span
        hz, t = [], 0
        for (n, L), sp in zip(zip(q_lens, kv_lens), spans):
            for i in range(n):
                pos = L - n + i
                hz.append(next((b - 1 for a, b in sp if a <= pos < b), pos))
        horizon = torch.tensor(hz, dtype=torch.int32, device=dev())
    want = ref.paged_attention(q, kc, vc, bt, cu, kl, scale, window, softcap, ks, vs, horizon=horizon)
    got = K.paged_attention(q, kc, vc, bt, cu, kl, scale, window, softcap, ks, vs, max(q_lens), max(kv_lens),
                            nsplit=nsplit, horizon=horizon)
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 64), (8, 1, 128), (4, 2, 256)])
def test_paged_attention_prefill(K, fp8, Hq, Hkv, D):
    _attention_case(K, 3, [70, 1, 130], [70, 33, 200], Hq, Hkv, D, fp8)
    _attention_case(K, 2, [64, 17], [64, 400], Hq, Hkv, D, fp8, window=48)
    _attention_case(K, 2, [30, 65], [30, 65], Hq, Hkv, D, fp8, softcap=30.0)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (16, 2), (4, 4)])
def test_paged_attention_prefill_tensor_core_tiles(K, fp8, Hq, Hkv):
    """Head size 128 with pages of 16 tokens runs the tcgen05 kernel: several 128-row query tiles, several
    128-token KV tiles, chunked prefill behind a cached prefix, ragged tails, windows and soft-capping."""
    _attention_case(K, 3, [300, 129, 1000], [300, 500, 1000], Hq, Hkv, 128, fp8)
    _attention_case(K, 2, [128, 256], [128, 2048], Hq, Hkv, 128, fp8)
    _attention_case(K, 2, [513, 40], [700, 1100], Hq, Hkv, 128, fp8, window=200)
    _attention_case(K, 2, [260, 131], [260, 400], Hq, Hkv, 128, fp8, softcap=30.0)
    assert K.check_status() == 0


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 2, 256)])
def test_paged_attention_prefill_horizon(K, fp8, Hq, Hkv, D):
    """Image-style spans: rows inside a span attend to the whole span, also across 64-row tiles and with a window."""
    spans = [[(10, 30), (100, 170)], [(0, 5)], [(60, 130)]]
    _attention_case(K, 3, [200, 40, 130], [200, 40, 130], Hq, Hkv, D, fp8, spans=spans)
    _attention_case(K, 3, [200, 40, 130], [200, 40, 130], Hq, Hkv, D, fp8, window=48, spans=spans)
    _attention_case(K, 2, [100, 70], [150, 70], Hq, Hkv, D, fp8, spans=[[(60, 140)], [(3, 66)]])   # cached prefix


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 64), (32, 1, 128), (64, 8, 128), (4, 2, 256), (8, 1, 128)])
def test_paged_attention_decode(K, fp8, Hq, Hkv, D):
    _attention_case(K, 5, [1] * 5, [1, 17, 64, 250, 1000], Hq, Hkv, D, fp8)
    _attention_case(K, 3, [1] * 3, [300, 5, 129], Hq, Hkv, D, fp8, nsplit=1)
    _attention_case(K, 3, [1] * 3, [300, 5, 129], Hq, Hkv, D, fp8, nsplit=4)
    _attention_case(K, 2, [1, 1], [500, 90], Hq, Hkv, D, fp8, window=100)
    _attention_case(K, 3, [1] * 3, [77, 300, 32], Hq, Hkv, D, fp8, softcap=30.0)
    assert K.check_status() == 0


def test_embedding_and_argmax(K):
    torch.manual_seed(3)
    table = torch.randn(1000, 512, device=dev(), dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (77,), device=dev(), dtype=torch.int32)
    torch.testing.assert_close(K.embedding(ids, table), ref.embedding(ids, table))
    for dt in (torch.bfloat16, torch.float32):
        logits = torch.randn(9, 128256, device=dev(), dtype=dt) * 3
        ids1, lp1 = K.argmax_logprob(logits)
        ids2, lp2 = ref.argmax_logprob(logits)
        assert torch.equal(ids1, ids2)
        torch.testing.assert_close(lp1, lp2, atol=1e-3, rtol=1e-3)


def test_library_is_native():
    """The CUDA path must be the in-tree library, not a PyTorch fallback."""
    from tgi_b200 import ops
    from tgi_b200.ops import cuda as K

    assert K.lib_path().exists()
    x = torch.randn(4, 256, device=dev(), dtype=torch.bfloat16)
    assert ops.use_native(x)
    out, _ = ops.rms_norm(x, None, torch.ones(256, device=dev(), dtype=torch.bfloat16), 1e-5)
    assert out.shape == x.shape
    with open("/proc/self/maps") as f:
        assert "libtgi_b200_kernels.so" in f.read()


@pytest.mark.gpu
@pytest.mark.parametrize("layer,unit_offset,D", [(False, False, 128), (False, True, 256), (True, False, 128), (False, False, 64)])
def test_qk_norm_per_head(layer, unit_offset, D):
    """q / k heads of a fused qkv row normalised in place: RMSNorm with a weight shared by the heads (Qwen3,
    Gemma-3 with the unit offset) and bias-free LayerNorm with per-head weights (Cohere); v is left alone."""
    from tgi_b200.ops import cuda as K

    torch.manual_seed(5)
    T, nh, nkv = 37, 6, 2
    qkv = (torch.randn(T, (nh + 2 * nkv) * D, device="cuda") * 3).to(torch.bfloat16)
    qw = (torch.randn(nh, D, device="cuda") if layer else torch.randn(D, device="cuda")).to(torch.bfloat16)
    kw = (torch.randn(nkv, D, device="cuda") if layer else torch.randn(D, device="cuda")).to(torch.bfloat16)
    ref = qkv.clone().float().view(T, nh + 2 * nkv, D)
    for lo, hi, w in ((0, nh, qw), (nh, nh + nkv, kw)):
        x = ref[:, lo:hi]
        if layer:
            y = (x - x.mean(-1, keepdim=True)) * torch.rsqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-6) * w.float()
        else:
            y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * (w.float() + (1.0 if unit_offset else 0.0))
        ref[:, lo:hi] = y
    out = K.qk_norm(qkv.clone(), nh, nkv, D, qw, kw, 1e-6, unit_offset, layer=layer).float().view(T, nh + 2 * nkv, D)
    assert torch.equal(out[:, nh + nkv:], qkv.float().view(T, nh + 2 * nkv, D)[:, nh + nkv:])
    err = (out - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item(), err
