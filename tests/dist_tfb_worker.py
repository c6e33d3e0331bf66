"""CPU worker (gloo, two ranks, run by torch.distributed.run): a model type without a native decoder runs its
transformers modules tensor parallel around the paged attention and must reproduce the unsharded transformers model
(first-step logits to 2e-4, same greedy tokens)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from dist_cpu_worker import generate  # noqa: E402
from tgi_b200.models import get_model  # noqa: E402
from tgi_b200.models.transformers_backend import ShardedLinear, TransformersDecoder  # noqa: E402
from tgi_b200.parallel import dist as pdist  # noqa: E402


def main():
    import transformers

    path = os.environ["DIST_WORKER_DIR"]
    group, rank, world = pdist.initialize_torch_distributed()
    assert world == 2
    prompts = [[5, 17, 100, 42, 7, 9, 250, 31], [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23]]
    n_new = 6
    sharded = get_model(path, dtype="float32", device=torch.device("cpu"))
    assert isinstance(sharded.model, TransformersDecoder)
    n_sharded = sum(isinstance(m, ShardedLinear) for m in sharded.model.hf.modules())
    assert n_sharded >= 2 * 4, "the plan was not applied"
    toks, logits = generate(sharded, prompts, n_new)
    hf = transformers.AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        want_first = torch.cat([hf(torch.tensor([p])).logits[0, -1:] for p in prompts])
    err = (logits - want_first).abs().max().item()
    assert err < 2e-4, f"rank {rank}: sharded logits differ from the unsharded model by {err}"
    for i, p in enumerate(prompts):
        ids = list(p)          # plain greedy decoding (``generate`` would mask the end-of-sequence token)
        with torch.no_grad():
            for _ in range(n_new):
                ids.append(int(hf(torch.tensor([ids])).logits[0, -1].argmax()))
        if i % world == rank:
            assert toks[i] == ids[len(p):], (i, toks[i], ids[len(p):])
        else:
            assert toks[i] == []
    pdist.barrier(group)
    if rank == 0:
        print("DIST_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
