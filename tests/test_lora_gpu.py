"""Multi-adapter LoRA kernels (shrink / expand) against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tgi_b200.ops import cuda as K

    K.load()
    return K


@pytest.mark.parametrize("T,H,N", [(1, 256, 512), (37, 4096, 1536), (256, 8192, 1024)])
def test_lora_shrink_expand(K, T, H, N):
    dev = torch.device("cuda")
    torch.manual_seed(T)
    ranks = [0, 8, 16, 12, 0]            # adapter 0 is "none", adapter 4 does not target this projection
    A = [None] + [(torch.randn(r, H, device=dev) * 0.05).to(torch.bfloat16) if r else None for r in ranks[1:]]
    B = [None] + [(torch.randn(N, r, device=dev) * 0.05).to(torch.bfloat16) if r else None for r in ranks[1:]]
    scales = torch.tensor([0.0, 2.0, 0.5, 1.5, 1.0], device=dev)
    a_ptrs = torch.tensor([t.data_ptr() if t is not None else 0 for t in A], dtype=torch.int64, device=dev)
    b_ptrs = torch.tensor([t.data_ptr() if t is not None else 0 for t in B], dtype=torch.int64, device=dev)
    rk = torch.tensor(ranks, dtype=torch.int32, device=dev)
    tok = torch.randint(0, 5, (T,), device=dev, dtype=torch.int32)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    col0 = 128
    out = torch.randn(T, col0 + N + 64, device=dev, dtype=torch.bfloat16)
    want = out.float().clone()
    for t in range(T):
        a = int(tok[t])
        if ranks[a]:
            v = A[a].float() @ x[t].float()
            want[t, col0:col0 + N] += scales[a] * (B[a].float() @ v)
    v = K.lora_shrink(x, a_ptrs, rk, tok, 16)
    for t in range(T):
        a = int(tok[t])
        ref = torch.zeros(16, device=dev)
        if ranks[a]:
            ref[:ranks[a]] = A[a].float() @ x[t].float()
        torch.testing.assert_close(v[t], ref, atol=2e-2, rtol=2e-2)
    K.lora_expand(v, b_ptrs, rk, scales, tok, out, col0, N)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), want, atol=6e-2, rtol=3e-2)
    # columns outside [col0, col0 + N) are untouched
    assert torch.equal(out[:, :col0].float(), want[:, :col0]) and torch.equal(out[:, col0 + N:].float(), want[:, col0 + N:])


def test_lora_decode_under_cuda_graphs(K, tmp_path):
    """A mixed batch (base + two adapters) decodes through graphs that contain the LoRA kernels and must
    produce the tokens of the eager path; adapters must change the output."""
    import random

    from tgi_b200.models import get_model_with_lora_adapters
    from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch
    from tgi_b200.models.graphs import DecodeGraphs
    from tgi_b200.proto import generate_v3 as pb
    from tgi_b200.utils import adapter as ad
    from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint

    from test_lora import CFG, _request, _write_adapter

    dev = torch.device("cuda")
    cfg = llama_config(**CFG)
    base = tmp_path / "base"
    write_llama_checkpoint(base, cfg)
    _write_adapter(tmp_path / "ad1", 1)
    _write_adapter(tmp_path / "ad2", 2, r=8, alpha=4.0)
    adapters = ad.parse_lora_adapters(f"one={tmp_path / 'ad1'},two={tmp_path / 'ad2'}")
    model = get_model_with_lora_adapters(str(base), adapters, dtype="bfloat16", device=dev)
    rng = random.Random(0)
    prompts = [[rng.randrange(3, 300) for _ in range(n)] for n in (11, 19, 7)]
    n_new = 8

    def generate(adapter_ids, graphs):
        cursor, reqs = 1, []
        for i, p in enumerate(prompts):
            nb = (len(p) + n_new + 15) // 16
            reqs.append(_request(i, n_new, range(cursor, cursor + nb), adapter_ids[i]))
            cursor += nb
        if not model.kv_cache:
            model.init_kv_cache(cursor)
        if graphs and model.graphs is None:
            model.graphs = DecodeGraphs(model, 64, buckets=[4])
            model.graphs.capture_all()
        if not graphs:
            model.graphs = None
        batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts,
                                                  model.tokenizer, torch.bfloat16, dev)
        toks = {i: [] for i in range(len(prompts))}
        while batch is not None:
            gens, batch, _ = model.generate_token(batch)
            for g in gens:
                toks[g.request_id].extend(g.tokens.token_ids)
        return toks

    ids = ["one", None, "two"]
    eager = generate(ids, graphs=False)
    plain = generate([None] * 3, graphs=False)
    assert eager[1] == plain[1] and (eager[0] != plain[0] or eager[2] != plain[2])
    graphed = generate(ids, graphs=True)
    assert 4 in model.graphs.lora_buckets
    assert graphed == eager
    assert generate([None] * 3, graphs=True) == plain
    assert K.check_status() == 0
