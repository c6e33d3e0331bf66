"""CPU worker for the sharding tests (gloo, run by torch.distributed.run): loads a checkpoint as one
shard of a 2-rank group and checks its prefill logits and greedy tokens against the unsharded model."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.arch import ModelConfig  # noqa: E402
from tgi_b200.models.decoder import CausalDecoder  # noqa: E402
from tgi_b200.models.flash_causal_lm import FlashCausalLM, FlashCausalLMBatch  # noqa: E402
from tgi_b200.parallel import dist as pdist  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402
from tgi_b200.utils.tokenizer import ByteTokenizer  # noqa: E402
from tgi_b200.utils.weights import Weights, weight_files  # noqa: E402


def request(i, n_new, blocks):
    r = pb.Request(id=i, inputs="")
    r.parameters.temperature = 1.0
    r.parameters.top_p = 1.0
    r.parameters.typical_p = 1.0
    r.parameters.repetition_penalty = 1.0
    r.stopping_parameters.max_new_tokens = n_new
    r.stopping_parameters.ignore_eos_token = True
    r.blocks.extend(blocks)
    return r


def generate(runner, prompts, n_new):
    cursor, reqs = 1, []
    for i, p in enumerate(prompts):
        nb = (len(p) + n_new + 15) // 16
        reqs.append(request(i, n_new, range(cursor, cursor + nb)))
        cursor += nb
    runner.init_kv_cache(cursor)
    batch = FlashCausalLMBatch.from_tokenized(pb.Batch(id=0, requests=reqs, size=len(reqs)), prompts, runner.tokenizer,
                                              torch.float32, torch.device("cpu"))
    toks = {i: [] for i in range(len(prompts))}
    first = {}
    orig = runner.forward

    def spy(meta):
        out = orig(meta)
        first.setdefault("logits", out.detach().float().clone())
        return out

    runner.forward = spy
    while batch is not None:
        gens, batch, _ = runner.generate_token(batch)
        for g in gens:
            toks[g.request_id].extend(g.tokens.token_ids)
    runner.forward = orig
    return toks, first["logits"]


def main():
    path = os.environ["DIST_WORKER_DIR"]
    group, rank, world = pdist.initialize_torch_distributed()
    assert world == 2
    prompts = [[5, 17, 100, 42, 7, 9, 250, 31], [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23]]
    sharded = get_model(path, dtype="float32", device=torch.device("cpu"))
    toks, logits = generate(sharded, prompts, 6)
    # the same checkpoint unsharded, in this process
    cfg = ModelConfig.from_path(path)
    w = Weights(weight_files(path), torch.device("cpu"), torch.float32, process_group=pdist.FakeGroup(0, 1))
    single = FlashCausalLM(CausalDecoder(cfg, w), ByteTokenizer(cfg.get("vocab_size")), torch.float32, torch.device("cpu"))
    w.close()
    want_toks, want_logits = generate(single, prompts, 6)
    err = (logits - want_logits).abs().max().item()
    assert err < 2e-4, f"rank {rank}: sharded logits differ from the unsharded model by {err}"
    # every shard reports the generations of the requests it owns (request id modulo world size)
    for i, t in want_toks.items():
        if i % world == rank:
            assert toks[i] == t, (i, toks[i], t)
        else:
            assert toks[i] == []
    mode = os.environ.get("TGI_B200_MOE_PARALLEL", "tp")
    moe = getattr(sharded.model.layers[0], "mlp", None)
    if hasattr(moe, "expert_parallel"):
        assert (moe.expert_parallel is not None) == (mode == "ep"), "wrong MoE parallel mode"
    pdist.barrier(group)
    if rank == 0:
        print("DIST_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
