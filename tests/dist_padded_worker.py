"""CPU worker (gloo, two ranks, run by torch.distributed.run): the fallback runner with its transformers module
sharded by this package's plan (OPT, Bloom with its ALiBi bias cut to the rank's heads) must produce the greedy
tokens of the unsharded transformers model."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from test_padded_runners import _request  # noqa: E402
from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.padded import PaddedCausalLM  # noqa: E402
from tgi_b200.models.transformers_backend import ShardedLinear  # noqa: E402
from tgi_b200.parallel import dist as pdist  # noqa: E402
from tgi_b200.proto import generate_v3 as pb  # noqa: E402


def main():
    import transformers

    path = os.environ["DIST_WORKER_DIR"]
    group, rank, world = pdist.initialize_torch_distributed()
    assert world == 2
    model = get_model(path, dtype="float32", device=torch.device("cpu"))
    assert isinstance(model, PaddedCausalLM)
    assert sum(isinstance(m, ShardedLinear) for m in model.hf.modules()) >= 2 * 4
    prompts = [[10, 20, 30, 40, 50], [7, 8, 9], [100, 90, 80, 70, 60, 50, 40]]
    n_new = 6
    reqs = [_request(i, p, n_new) for i, p in enumerate(prompts)]
    batch = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs, size=len(reqs)), model.tokenizer, model.dtype,
                                     model.device, 0)
    got = {i: [] for i in range(len(prompts))}
    while batch is not None:
        gens, batch, _ = model.generate_token(batch)
        for g in gens:
            got[g.request_id].extend(g.tokens.token_ids)
    hf = transformers.AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.float32).eval()
    for i, p in enumerate(prompts):
        ids = list(model.tokenizer("".join(chr(3 + t) for t in p))["input_ids"])
        n0 = len(ids)
        with torch.no_grad():
            for _ in range(n_new):
                ids.append(int(hf(torch.tensor([ids])).logits[0, -1].argmax()))
        if i % world == rank:
            assert got[i] == ids[n0:], (i, got[i], ids[n0:])
        else:
            assert got[i] == []
    pdist.barrier(group)
    if rank == 0:
        print("DIST_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
