"""Collective microbenchmark: peer-memory kernels against the process group's all-reduce.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m tgi_b200.parallel.bench_peer --tokens 256 --hidden 8192

Times, per call and as the maximum over ranks (CUDA events around a captured graph of ``--iters``
calls, so launch overhead is the replay's, as in the decode step):

* ``nccl_all_reduce``      ``dist.all_reduce`` of a bf16 ``[T, H]`` tensor
* ``nccl_ar_plus_norm``    the same followed by the stand-alone residual-add + RMSNorm + fp8 quant kernel
* ``peer_all_reduce``      ``PeerComm.all_reduce`` (copy in, reduce kernel, copy out)
* ``peer_reduce_norm``     ``PeerComm.reduce_norm(quant=True)``: reduce-scatter, residual, RMSNorm, fp8 quant,
                           all-gather in one kernel, input already in the peer heap

and prints one JSON line per row on rank 0.  The roofline column is the NVLink time of the bytes a
rank must move (pull ``(N-1)/N`` of the bf16 matrix, push ``(N-1)/N`` of the result) at the
measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .. import ops
from . import dist as pdist
from .peer import PeerComm

NVLINK_GBS = 770.0


def timed(fn, iters: int, group) -> float:
    """Seconds per call: ``iters`` calls captured in one graph, replayed 5 times, best replay, max over ranks."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier(group=group)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    best = float("inf")
    for _ in range(5):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3 / iters)
    t = torch.tensor([best], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    group, rank, world = pdist.initialize_torch_distributed()
    dev = torch.device("cuda", torch.cuda.current_device())
    T, H = args.tokens, args.hidden
    comm = PeerComm(group, rank, world, dev, T, H)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    res = torch.randn(T, H, device=dev).to(torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    comm.partial(T).copy_(x)
    comm.reduce_norm(T, w, 1e-5, 0.0, quant=True, first=True)

    def nccl_ar():
        dist.all_reduce(x, group=group)

    def nccl_ar_norm():
        dist.all_reduce(x, group=group)
        ops.rms_norm_quant(x, res, w, 1e-5)

    rows = {
        "nccl_all_reduce": timed(nccl_ar, args.iters, group),
        "nccl_ar_plus_norm": timed(nccl_ar_norm, args.iters, group),
        "peer_all_reduce": timed(lambda: comm.all_reduce(x), args.iters, group),
        "peer_reduce_norm": timed(lambda: comm.reduce_norm(T, w, 1e-5, 0.0, quant=True), args.iters, group),
    }
    status = comm.check()
    link_bytes = T * H * 2 * (world - 1) / world
    roof = link_bytes / (NVLINK_GBS * 1e9)
    if rank == 0:
        for name, t in rows.items():
            print(json.dumps({"op": name, "world": world, "tokens": T, "hidden": H, "us": round(t * 1e6, 2),
                              "nvlink_roofline_us": round(roof * 1e6, 2),
                              "frac_of_roofline": round(roof / t, 3), "kernel_status": status}), flush=True)
    dist.barrier(group=group)
    torch.cuda.synchronize()
    import os
    import sys

    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
