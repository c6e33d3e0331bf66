"""Worker of the tensor-parallel engine test: run as N ranks by ``torch.distributed.run``.

Loads a small Llama checkpoint through the model registry twice in the same process: once with the
peer-memory collectives (fused reduce + residual + RMSNorm) and once with the process-group
collectives (``TGI_B200_COMM=nccl``).  Both must agree with each other and with a dense fp32 CPU
forward of the unsharded weights; decode through captured CUDA graphs must give the eager tokens.
Prints ``TP_WORKER_OK`` from rank 0.
"""
import os
import random
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.flash_causal_lm import FlashCausalLMBatch  # noqa: E402
from tgi_b200.models.graphs import DecodeGraphs  # noqa: E402
from tgi_b200.ops import cuda as K  # noqa: E402
from tgi_b200.parallel import dist as pdist  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402
from tgi_b200.utils.synthetic import (llama_config, llama_state_dict, reference_llama_forward,  # noqa: E402
                                      write_llama_checkpoint)


def request(i, n_new, blocks, sampled=False):
    r = pb.Request(id=i, inputs="")
    r.parameters.temperature = 0.7 if sampled else 1.0
    r.parameters.top_p = 0.9 if sampled else 1.0
    r.parameters.top_k = 50 if sampled else 0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.1 if sampled else 1.0
    if sampled:
        r.parameters.do_sample = True
        r.parameters.seed = 77 + i
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.blocks.extend(blocks)
    return r


def generate(runner, dev, prompts, n_new, sampled=False):
    cursor, reqs = 1, []
    for i, p in enumerate(prompts):
        nb = (len(p) + n_new + 15) // 16
        reqs.append(request(i, n_new, range(cursor, cursor + nb), sampled))
        cursor += nb
    if runner.num_blocks < cursor:
        runner.init_kv_cache(cursor)
    batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts,
                                              runner.tokenizer, torch.bfloat16, dev)
    toks = {i: [] for i in range(len(prompts))}
    first = {}
    orig = runner.forward

    def spy(meta):
        out = orig(meta)
        first.setdefault("logits", out.detach().float().clone())
        return out

    runner.forward = spy
    try:
        while batch is not None:
            gens, batch, _ = runner.generate_token(batch)
            for g in gens:
                toks[g.request_id].extend(g.tokens.token_ids)
    finally:
        runner.forward = orig
    return toks, first["logits"]


def main():
    group, rank, world = pdist.initialize_torch_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    path = os.environ["TP_WORKER_DIR"]
    cfg = llama_config(hidden=512, layers=3, heads=8, kv_heads=8 if world > 2 else 2, intermediate=1024, vocab=4096,
                       max_pos=1024)
    if os.environ.get("TP_WORKER_MODEL") == "mixtral":
        # sparse MoE: experts sliced over the ranks, or whole experts per rank with TGI_B200_MOE_PARALLEL=ep
        cfg = llama_config(hidden=512, layers=2, heads=8, kv_heads=8 if world > 2 else 2, intermediate=512, vocab=4096,
                           max_pos=1024, model_type="mixtral", num_local_experts=8, num_experts_per_tok=2)
    if rank == 0:
        write_llama_checkpoint(path, cfg, std=0.05)
    pdist.barrier(group)

    rng = random.Random(0)
    prompts = [[rng.randrange(3, 4096) for _ in range(n)] for n in (45, 100, 17, 33)]
    n_new = 6

    peer = get_model(path, dtype="bfloat16", max_prefill_tokens=512)
    assert peer.model.comm is not None, "peer-memory communicator was not created"
    toks_peer, logits_peer = generate(peer, dev, prompts, n_new)
    assert K.check_status(dev) == 0

    os.environ["TGI_B200_COMM"] = "nccl"
    base = get_model(path, dtype="bfloat16", max_prefill_tokens=512)
    assert base.model.comm is None
    toks_base, logits_base = generate(base, dev, prompts, n_new)
    os.environ.pop("TGI_B200_COMM")

    scale = logits_base.abs().max().item()
    diff = (logits_peer - logits_base).abs().max().item()
    assert diff <= 0.04 * scale, f"peer vs group collectives: {diff} (scale {scale})"

    sd = llama_state_dict(cfg, std=0.05)
    for i, p in enumerate(prompts if cfg["model_type"] == "llama" else []):   # the dense oracle covers Llama only
        want = reference_llama_forward(sd, cfg, torch.tensor(p))[-1]
        got = logits_peer[i].cpu()
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 0.02, f"prompt {i}: logits differ from the dense forward by {err}"

    # decode through captured graphs (peer kernels inside the graph) must reproduce the eager tokens
    peer.graphs = DecodeGraphs(peer, 256, buckets=[4])
    peer.graphs.capture_all()
    toks_graph, _ = generate(peer, dev, prompts, n_new)
    assert K.check_status(dev) == 0
    agree = sum(toks_graph[i] == toks_peer[i] for i in toks_peer)
    assert agree == len(prompts), (toks_graph, toks_peer)
    same = sum(toks_base[i][:2] == toks_peer[i][:2] for i in toks_peer)
    assert same >= len(prompts) - 1, (toks_base, toks_peer)

    # sampled requests (temperature, top-k, top-p, repetition penalty, seed): the decode graph leaves each rank its
    # slice of the logits and the ranks sample on the slices; the draw is a function of (seed, step) and must repeat
    taken = []
    orig_shard_sampler = peer._sample_on_shards

    def shard_sampler_spy(*a, **kw):
        out = orig_shard_sampler(*a, **kw)
        taken.append(out is not None)
        return out

    peer._sample_on_shards = shard_sampler_spy
    toks_s1, _ = generate(peer, dev, prompts, n_new, sampled=True)
    toks_s2, _ = generate(peer, dev, prompts, n_new, sampled=True)
    peer._sample_on_shards = orig_shard_sampler
    assert K.check_status(dev) == 0
    assert taken and all(taken), "sampled decode steps did not run on the vocabulary shards"
    assert toks_s1 == toks_s2, (toks_s1, toks_s2)
    # a rank reports the generations of the requests it owns (id % world == rank)
    assert all(len(v) == (n_new if i % world == rank else 0) and all(0 <= t < 4096 for t in v)
               for i, v in toks_s1.items()), toks_s1
    assert toks_s1 != toks_graph, "sampling with temperature produced the greedy tokens for every prompt"

    pdist.barrier(group)
    torch.cuda.synchronize()
    if rank == 0:
        print("TP_WORKER_OK", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
