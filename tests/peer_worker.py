"""Worker of the multi-GPU peer-memory tests: run as N ranks by ``torch.distributed.run``.

Every rank builds its own partial sums from a seed that depends on the rank, so each rank can also
rebuild what the other ranks hold and compute the expected result locally in fp32.
Prints ``PEER_WORKER_OK`` on success (rank 0) and exits non-zero on any mismatch.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tgi_b200.ops import cuda as K  # noqa: E402
from tgi_b200.ops import reference as ref  # noqa: E402
from tgi_b200.parallel import dist as pdist  # noqa: E402
from tgi_b200.parallel.peer import PeerComm  # noqa: E402


def partial_of(rank: int, T: int, H: int, salt: int, device):
    g = torch.Generator(device="cpu").manual_seed(1000 * salt + rank)
    return (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16).to(device)


def main():
    group, rank, world = pdist.initialize_torch_distributed()
    device = torch.device("cuda", torch.cuda.current_device())
    H = int(os.environ.get("PEER_H", "1024"))
    max_T = 96
    comm = PeerComm(group, rank, world, device, max_T, H)
    g = torch.Generator(device="cpu").manual_seed(7)
    weight = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(device)
    eps = 1e-5
    salt = 0

    def expected_sum(T):
        acc = torch.zeros(T, H, dtype=torch.float32, device=device)
        for r in range(world):
            acc += partial_of(r, T, H, salt, device).float()
        return acc.to(torch.bfloat16)

    # ---- plain all-reduce, several shapes, repeated calls ------------------------------------
    for T in (1, 5, 16, 96):
        for _ in range(2):
            salt += 1
            t = partial_of(rank, T, H, salt, device).clone()
            comm.all_reduce(t)
            torch.cuda.synchronize()
            assert comm.check() == 0
            exp = expected_sum(T)
            assert torch.equal(t, exp), f"all_reduce mismatch T={T} rank={rank}: {(t.float()-exp.float()).abs().max()}"

    # ---- fused reduce + residual + RMSNorm (+ quant), a chain of three calls -----------------
    for T in (3, 64):
        rows_per = (T + world - 1) // world
        row0 = rank * rows_per
        res_ref = None
        for step, quant in enumerate((False, True, True)):
            salt += 1
            comm.partial(T).copy_(partial_of(rank, T, H, salt, device))
            out = comm.reduce_norm(T, weight, eps, 0.0, quant=quant, first=(step == 0))
            torch.cuda.synchronize()
            assert comm.check() == 0
            summed = expected_sum(T)
            normed, res_ref = ref.rms_norm(summed, res_ref, weight, eps, False)
            mine = slice(row0, min(T, row0 + rows_per))
            n_mine = max(0, mine.stop - mine.start)
            if n_mine > 0:
                assert torch.equal(comm.residual[:n_mine], res_ref[mine]), f"residual mismatch T={T} step={step}"
            if not quant:
                err = (out.float() - normed.float()).abs().max().item()
                assert err <= 2e-2, f"norm mismatch {err}"
            else:
                xq, xs = out
                deq = (xq.float().view(T, H // 128, 128) * xs.float().unsqueeze(-1)).view(T, H)
                err = (deq - normed.float()).abs().max().item()
                assert err <= 0.07 * normed.float().abs().max().item() + 1e-3, f"quant norm mismatch {err}"
                # every rank must hold bit-identical gathered data
                chk = torch.stack([xq.view(torch.uint8).float().sum(), xs.float().sum()])
                gathered = [torch.empty_like(chk) for _ in range(world)]
                torch.distributed.all_gather(gathered, chk, group=group)
                for o in gathered:
                    assert torch.equal(o, gathered[0]), "gathered rows differ between ranks"

    # ---- row-parallel GEMM whose epilogue pushes its rows to their owners, then the fused reduction ----
    from tgi_b200 import ops

    for T, Kd in ((5, 256), (64, 512), (96, 1024)):
        for rep in range(2):
            salt += 1
            xs_all, ws_all = [], []
            for r in range(world):
                g = torch.Generator(device="cpu").manual_seed(9000 * salt + r)
                xs_all.append((torch.randn(T, Kd, generator=g) * 0.5).to(torch.bfloat16).to(device))
                ws_all.append((torch.randn(H, Kd, generator=g) * 0.05).to(torch.bfloat16).to(device))
            dst = comm.push_target(T)
            ops.linear(xs_all[rank], ws_all[rank], None, out=dst)
            assert dst.used
            out = comm.reduce_norm(T, weight, eps, 0.0, quant=False, first=True, source=dst)
            torch.cuda.synchronize()
            assert comm.check() == 0
            acc = torch.zeros(T, H, dtype=torch.float32, device=device)
            for r in range(world):
                acc += (xs_all[r].float() @ ws_all[r].float().t()).to(torch.bfloat16).float()
            want, _ = ref.rms_norm(acc.to(torch.bfloat16), None, weight, eps, False)
            err = (out.float() - want.float()).abs().max().item()
            assert err <= 3e-2, f"pushed GEMM + reduce mismatch T={T} K={Kd}: {err}"

    # ---- vocabulary-parallel greedy sampling --------------------------------------------------
    for B, Vl in ((1, 500), (37, 2003), (256, 1024)):
        salt += 1
        shards = []
        for r in range(world):
            g = torch.Generator(device="cpu").manual_seed(5000 * salt + r)
            shards.append((torch.randn(B, Vl, generator=g) * 3).to(torch.bfloat16))
        full = torch.cat(shards, dim=1).to(device).float() * 0.5
        ids, lps = comm.argmax(shards[rank].to(device), rank * Vl, 0.5)
        torch.cuda.synchronize()
        assert comm.check() == 0
        want_ids = full.argmax(-1)
        want_lp = torch.log_softmax(full, -1).gather(1, want_ids.view(-1, 1)).view(-1)
        assert torch.equal(ids, want_ids), f"argmax ids differ B={B}"
        assert (lps - want_lp).abs().max().item() < 2e-3, f"argmax logprobs differ {(lps - want_lp).abs().max()}"

    # ---- vocabulary-parallel sampling: same tokens as the single-GPU fused sampler on the full logits ------
    from tgi_b200.ops import cuda as K

    for B, Vl, use_pen in ((1, 512, False), (33, 2003, False), (64, 1024, True), (256, 1024, False)):
        salt += 1
        g = torch.Generator(device="cpu").manual_seed(9000 + salt)
        full_bf = (torch.randn(B, Vl * world, generator=g) * 3).to(torch.bfloat16)
        temperature = torch.rand(B, generator=g) * 1.5 + 0.3
        top_k = torch.randint(0, 60, (B,), generator=g, dtype=torch.int32)
        top_k[::3] = 0
        top_p = torch.rand(B, generator=g) * 0.7 + 0.3
        top_p[1::4] = 1.0
        do_sample = (torch.rand(B, generator=g) < 0.8).to(torch.uint8)
        seeds = torch.randint(0, 2 ** 40, (B,), generator=g, dtype=torch.int64)
        steps = torch.randint(0, 50, (B,), generator=g, dtype=torch.int32)
        hist = torch.randint(0, Vl * world, (B, 40), generator=g, dtype=torch.int64)
        rep = torch.rand(B, generator=g) * 0.5 + 1.0
        freq = torch.rand(B, generator=g) * 0.4
        full_dev = full_bf.to(device)
        local = full_dev[:, rank * Vl:(rank + 1) * Vl].contiguous()
        if use_pen:
            ref_scores = K.penalties(full_dev, hist, rep.to(device), freq.to(device), 0, 0.5)
            want_ids, want_lp = K.fused_sample(ref_scores, temperature, top_k, top_p, do_sample, seeds, steps)
            loc_scores = K.penalties(local, hist, rep.to(device), freq.to(device), rank * Vl, 0.5)
            assert torch.equal(loc_scores, ref_scores[:, rank * Vl:(rank + 1) * Vl]), "penalties on a slice differ"
            ids, lps = comm.sample(loc_scores, rank * Vl, Vl * world, 1.0, temperature, top_k, top_p, do_sample, seeds, steps)
        else:
            want_ids, want_lp = K.fused_sample(full_dev.float() * 0.5, temperature, top_k, top_p, do_sample, seeds, steps)
            ids, lps = comm.sample(local, rank * Vl, Vl * world, 0.5, temperature, top_k, top_p, do_sample, seeds, steps)
        torch.cuda.synchronize()
        assert comm.check() == 0
        same = (ids == want_ids).float().mean().item()
        assert same >= 0.99, f"sharded sampling differs from the single-GPU sampler: B={B} agree={same}"
        ok = ids == want_ids
        assert (lps[ok] - want_lp[ok]).abs().max().item() < 2e-3
        # every rank must hold the same ids
        gathered = [torch.empty_like(ids) for _ in range(world)]
        torch.distributed.all_gather(gathered, ids, group=group)
        assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree on the sampled ids"

    # ---- CUDA graph replay: the call counters live in device memory ----------------------------
    T = 32
    salt += 1
    src = partial_of(rank, T, H, salt, device)
    exp = expected_sum(T)
    res = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):   # warm-up on the capture stream
            t = src.clone()
            comm.all_reduce(t)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    pdist.barrier(group)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        t = src.clone()
        comm.all_reduce(t)
        comm.all_reduce(t.zero_().add_(src))
        res.copy_(t)
    for _ in range(3):
        res.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert comm.check() == 0
        assert torch.equal(res, exp), "graph replay mismatch"

    pdist.barrier(group)
    comm.close()
    if rank == 0:
        print("PEER_WORKER_OK", flush=True)


if __name__ == "__main__":
    main()
