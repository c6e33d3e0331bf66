"""Two gloo ranks on CPU: tensor-parallel Llama, and Mixtral-style MoE with experts tensor-parallel
and expert-parallel, must reproduce the unsharded model (logits to 2e-4, same greedy tokens)."""
import os
import subprocess
import sys

import pytest

from tgi_b200.utils.synthetic import llama_config, write_llama_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(path, port, extra_env):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", DIST_WORKER_DIR=str(path), PYTHONPATH=ROOT, **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "dist_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DIST_WORKER_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


def test_tensor_parallel_llama(tmp_path):
    write_llama_checkpoint(tmp_path, llama_config(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=128, vocab=300,
                                                  max_pos=256))
    _run(tmp_path, 29811, {})


@pytest.mark.parametrize("mode", ["tp", "ep"])
def test_mixtral_experts_tp_and_ep(tmp_path, mode):
    write_llama_checkpoint(tmp_path, llama_config(hidden=64, layers=2, heads=4, kv_heads=2, intermediate=96, vocab=300,
                                                  max_pos=256, model_type="mixtral", num_local_experts=4,
                                                  num_experts_per_tok=2))
    _run(tmp_path, 29812 + (mode == "ep"), {"TGI_B200_MOE_PARALLEL": mode})


def test_pin_cpu_threads_splits_the_cores():
    import os

    import torch

    from tgi_b200.parallel.dist import pin_cpu_threads

    before = os.sched_getaffinity(0)
    threads = torch.get_num_threads()
    try:
        cpus = sorted(before)
        if len(cpus) >= 2:
            a = pin_cpu_threads(0, 2, cpus)
            assert os.sched_getaffinity(0) == set(a) and len(a) == len(cpus) // 2
            b = pin_cpu_threads(1, 2, cpus)
            assert not set(a) & set(b)
        # more shards than cores: nothing is pinned
        assert pin_cpu_threads(0, len(cpus) + 1, cpus) == cpus
    finally:
        os.sched_setaffinity(0, before)
        torch.set_num_threads(threads)
