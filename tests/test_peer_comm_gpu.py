"""Peer-memory collectives: single-rank math on one GPU, and the real exchange on two or more GPUs.

The multi-GPU part runs ``tests/peer_worker.py`` as child processes (one rank per GPU) with NVLS
switched off in NCCL, which is only used there to exchange the IPC handles and for barriers.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_reduce_norm_matches_oracle():
    from tgi_b200.ops import reference as ref
    from tgi_b200.parallel.dist import FakeGroup
    from tgi_b200.parallel.peer import PeerComm

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    H, T = 2048, 37
    comm = PeerComm(FakeGroup(0, 1), 0, 1, dev, 64, H)
    g = torch.Generator(device="cuda").manual_seed(3)
    w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
    x1 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    x2 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    comm.partial(T).copy_(x1)
    y1 = comm.reduce_norm(T, w, 1e-5, 0.0, quant=False, first=True).clone()
    n1, r1 = ref.rms_norm(x1, None, w, 1e-5)
    assert torch.equal(comm.residual[:T], r1)
    assert (y1.float() - n1.float()).abs().max().item() <= 2e-2
    comm.partial(T).copy_(x2)
    xq, xs = comm.reduce_norm(T, w, 1e-5, 0.0, quant=True)
    n2, r2 = ref.rms_norm(x2, r1, w, 1e-5)
    torch.cuda.synchronize()
    assert comm.check() == 0
    assert torch.equal(comm.residual[:T], r2)
    deq = (xq.float().view(T, H // 128, 128) * xs.float().unsqueeze(-1)).view(T, H)
    assert (deq - n2.float()).abs().max().item() <= 0.07 * n2.float().abs().max().item()
    comm.close()


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_collectives_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "peer_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PEER_WORKER_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


@pytest.mark.multigpu
@pytest.mark.parametrize("world,model", [(2, "llama"), (2, "mixtral"), (2, "mixtral-ep"), (4, "mixtral"), (8, "llama"),
                                         (8, "mixtral"), (8, "mixtral-ep")])
def test_tensor_parallel_engine_on_peer_memory(world, model, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    # prefill steps of 16 tokens or more use the pushing GEMM epilogue, smaller (decode) steps pull
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", TP_WORKER_DIR=str(tmp_path / "ckpt"),
               TGI_B200_PUSH_MIN_TOKENS="16", TP_WORKER_MODEL=model.split("-")[0],
               TGI_B200_MOE_PARALLEL="ep" if model.endswith("-ep") else "tp")
    env.pop("TGI_B200_COMM", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + world), os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
