"""Per-kernel timings on the shapes of one decoder layer, with roofline fractions.

    python -m tgi_b200.ops.bench_kernels --model llama70b --tp 1 --batch 256 --ctx 1280 [--fp8 1]

Every kernel is timed with CUDA events on the launching stream after warm-up; between timed
launches a buffer larger than L2 is overwritten so that no launch starts with its inputs cached.
Achieved bandwidth / FLOP rate is reported against the measured copy bandwidth and cuBLAS bf16 rate
of ``MEASURED_PEAKS.json`` when that file is present next to the repository root (fallback:
6.65 TB/s and 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch

from . import cuda as K
from . import reference as ref

FP8 = torch.float8_e4m3fn
SHAPES = {
    "llama70b": dict(hidden=8192, heads=64, kv_heads=8, head_dim=128, inter=28672, vocab=128256),
    "llama8b": dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, inter=14336, vocab=128256),
}


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class Timer:
    def __init__(self, dev, iters=10, warmup=3, plain=False):
        self.dev, self.iters, self.warmup, self.plain = dev, iters, warmup, plain
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # 256 MB > 126 MB L2

    def _graph(self, fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(self.iters):
                self.flush.zero_()
                if fn is not None:
                    fn()
        return g

    def _time(self, g):
        g.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        return best

    def __call__(self, fn):
        """Seconds per launch of ``fn``: (flush + fn) x iters replayed from a CUDA graph, minus the
        flushes alone, so neither host launch overhead nor the flush is in the number."""
        fn()
        torch.cuda.synchronize()
        code = K.check_status(self.dev)
        if code != 0:  # a wait timed out inside a kernel: stop before spending time on a broken kernel
            raise SystemExit(f"kernel reported error status {code}; aborting the benchmark")
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        if self.plain:  # direct launches (what a profiler attaches to); includes host launch overhead
            total = 0.0
            for _ in range(self.iters):
                self.flush.zero_()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                total += s.elapsed_time(e)
            return total / self.iters * 1e-3
        if not hasattr(self, "_flush_ms"):
            self._flush_ms = self._time(self._graph(None))
        ms = self._time(self._graph(fn))
        return max(ms - self._flush_ms, 1e-6) / self.iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama70b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1280)
    ap.add_argument("--fp8", type=int, default=1)
    ap.add_argument("--prefill", type=int, default=0, help="also time prefill attention with this many tokens per sequence")
    ap.add_argument("--only", default="")
    ap.add_argument("--nsplit", type=int, default=0, help="KV splits of the decode attention (0: the library's choice)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--plain", action="store_true", help="time direct launches instead of graph replays")
    ap.add_argument("--promote", action="store_true",
                    help="fp8 GEMMs with per-K-block promotion instead of the block-scaled MMA (TGI_B200_FP8_MX=0)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    K.load()
    K.set_fp8_mx(not args.promote)
    s = SHAPES[args.model]
    H, D = s["hidden"], s["head_dim"]
    hq, hkv, I = s["heads"] // args.tp, max(1, s["kv_heads"] // args.tp), s["inter"] // args.tp
    M = args.batch
    bw, flops_peak, src = peaks()
    timer = Timer(dev, args.iters, args.warmup, args.plain)
    rows = []

    def report(name, t, bytes_, flops=0.0):
        r = dict(kernel=name, us=round(t * 1e6, 2), gbs=round(bytes_ / t / 1e9, 1), frac_hbm=round(bytes_ / t / bw, 3))
        if flops:
            r["tflops"] = round(flops / t / 1e12, 1)
            r["frac_bf16_peak"] = round(flops / t / flops_peak, 3)
            r["roofline_us"] = round(max(bytes_ / bw, flops / (flops_peak * (2 if args.fp8 else 1))) * 1e6, 2)
        else:
            r["roofline_us"] = round(bytes_ / bw * 1e6, 2)
        r["of"] = src
        rows.append(r)
        print(json.dumps(r), flush=True)

    def want(name):
        return not args.only or args.only in name

    gemms = {"qkv": ((hq + 2 * hkv) * D, H), "o": (H, hq * D), "gate_up": (2 * I, H), "down": (H, I)}
    for name, (N, Kd) in gemms.items():
        if not want("gemm_" + name):
            continue
        x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02
        if args.fp8:
            wq = w.to(FP8)
            ws = torch.rand((N + 127) // 128, Kd // 128, device=dev) + 0.5
            if K.fp8_mx():
                wq, ws = K.requant_block_pow2(wq, ws)
            xq, xs = K.fp8_quant_act(x)
            t = timer(lambda: K.gemm_fp8_block(xq, xs, wq, ws))
            report(f"gemm_fp8_{name}[{M}x{N}x{Kd}]", t, N * Kd + M * Kd + 2 * M * N, 2.0 * M * N * Kd)
        else:
            t = timer(lambda: K.gemm_bf16(x, w))
            report(f"gemm_bf16_{name}[{M}x{N}x{Kd}]", t, 2 * (N * Kd + M * Kd + M * N), 2.0 * M * N * Kd)
        del x, w
    if want("lm_head"):
        V = s["vocab"] // args.tp
        x = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
        w = torch.randn(V, H, device=dev, dtype=torch.bfloat16) * 0.02
        t = timer(lambda: K.gemm_bf16(x, w))
        report(f"gemm_bf16_lm_head[{M}x{V}x{H}]", t, 2 * (V * H + M * H + M * V), 2.0 * M * V * H)
        logits = K.gemm_bf16(x, w)
        t = timer(lambda: K.argmax_logprob(logits))
        report(f"argmax_logprob[{M}x{V}]", t, 2 * M * V)
        del x, w, logits
    if want("norm"):
        x = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
        r = torch.randn(M, H, device=dev, dtype=torch.bfloat16)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        t = timer(lambda: K.rms_norm_quant(x, r, w, 1e-5))
        report(f"rms_norm_quant[{M}x{H}]", t, M * H * (2 + 2 + 2 + 1))
        t = timer(lambda: K.rms_norm(x, r, w, 1e-5))
        report(f"rms_norm[{M}x{H}]", t, M * H * 8)
    if want("act"):
        gu = torch.randn(M, 2 * I, device=dev, dtype=torch.bfloat16)
        t = timer(lambda: K.act_and_mul_quant(gu))
        report(f"act_mul_quant[{M}x{I}]", t, M * I * 5)
    if want("sample"):
        V = s["vocab"] // args.tp
        logits = torch.randn(M, V, device=dev, dtype=torch.bfloat16) * 3
        temp = torch.full((M,), 0.7, device=dev)
        top_p = torch.full((M,), 0.9, device=dev)
        top_k = torch.full((M,), 40, device=dev, dtype=torch.int32)
        ds = torch.ones(M, device=dev, dtype=torch.uint8)
        seeds = torch.arange(M, device=dev, dtype=torch.int64)
        steps = torch.zeros(M, device=dev, dtype=torch.int32)
        t = timer(lambda: K.fused_sample(logits, temp, top_k, top_p, ds, seeds, steps))
        report(f"fused_sample[{M}x{V} T,top-k,top-p]", t, 2 * M * V)
        hist = torch.randint(0, V, (M, args.ctx), device=dev, dtype=torch.int64)
        rep = torch.full((M,), 1.1, device=dev)
        t = timer(lambda: K.penalties(logits, hist, rep, None))
        report(f"penalties[{M}x{V}, history {args.ctx}]", t, M * V * (2 + 4) + M * args.ctx * 8)
        del logits, hist
    if want("moe"):
        # Mixtral-8x7B experts: 8 experts of [2 x 14336, 4096] / [4096, 14336], top-2 routing
        E, Hm, Im, topk = 8, 4096, 14336 // args.tp, 2
        x = torch.randn(M, Hm, device=dev, dtype=torch.bfloat16)
        wgu = torch.randn(E, 2 * Im, Hm, device=dev, dtype=torch.bfloat16) * 0.02
        wd = torch.randn(E, Hm, Im, device=dev, dtype=torch.bfloat16) * 0.02
        router = torch.randn(M, E, device=dev, dtype=torch.bfloat16)
        wts, ids = K.moe_topk_softmax(router, topk)
        t = timer(lambda: K.moe_experts(x, wgu, wd, wts, ids, "silu"))
        touched = min(E, M * topk)
        report(f"moe_experts[{M} tokens, {E} experts top-{topk}, I={Im}]", t, 2 * touched * 3 * Im * Hm, 2.0 * M * topk * 3 * Im * Hm)
        t = timer(lambda: K.moe_topk_softmax(router, topk))
        report(f"moe_topk_softmax[{M}x{E}]", t, M * E * 2 + M * topk * 8)
        del x, wgu, wd
    if want("wq"):
        # 4-bit weights, group 128 (GPTQ / AWQ after the canonical repack): the gate_up projection
        N4, K4, group = 2 * I, H, 128
        x = torch.randn(M, K4, device=dev, dtype=torch.bfloat16)
        wq = torch.randint(0, 256, (N4, K4 // 2), device=dev, dtype=torch.uint8)
        sc = (torch.rand(K4 // group, N4, device=dev) * 0.01 + 0.005).to(torch.float16)
        zp = torch.full((K4 // group, N4), 8.0, device=dev, dtype=torch.float16)
        for m in sorted({min(M, 16), M}):
            xm = x[:m].contiguous()
            t = timer(lambda: K.gemm_wq(xm, wq, sc, zp, group, 4))
            report(f"gemm_wq4[{m}x{N4}x{K4}]", t, N4 * K4 // 2 + 4 * (K4 // group) * N4 + 2 * m * (K4 + N4), 2.0 * m * N4 * K4)
        del x, wq, sc, zp
    bs = 16
    nb_seq = math.ceil((args.ctx + 1) / bs)
    nblocks = M * nb_seq + 1
    kv_dt = FP8 if args.fp8 else torch.bfloat16
    if want("rope") or want("attn"):
        kc = torch.empty(nblocks, bs, hkv, D, device=dev, dtype=torch.uint8 if args.fp8 else torch.bfloat16)
        vc = torch.empty_like(kc)
        if args.fp8:
            kc.random_(0, 120)
            vc.random_(0, 120)
            kc, vc = kc.view(FP8), vc.view(FP8)
        else:
            kc.normal_()
            vc.normal_()
        bt = (torch.arange(M * nb_seq, device=dev, dtype=torch.int32) + 1).view(M, nb_seq)
        ksc = torch.full((hkv,), 0.05, device=dev) if args.fp8 else None
    if want("rope"):
        qkv = torch.randn(M, (hq + 2 * hkv) * D, device=dev, dtype=torch.bfloat16)
        pos = torch.full((M,), args.ctx, device=dev, dtype=torch.int32)
        slots = (bt[:, args.ctx // bs] * bs + args.ctx % bs).to(torch.int32)
        cs = torch.randn(args.ctx + 8, D, device=dev)
        t = timer(lambda: K.rope_and_cache(qkv, pos, cs, slots, kc, vc, hq, hkv, D, D, True, ksc, ksc))
        report(f"rope_and_cache[{M}x{hq}+2x{hkv}]", t, M * (hq + 2 * hkv) * D * 2 + M * hq * D * 2)
    if want("attn"):
        q = torch.randn(M, hq, D, device=dev, dtype=torch.bfloat16)
        cu = torch.arange(M + 1, device=dev, dtype=torch.int32)
        kl = torch.full((M,), args.ctx + 1, device=dev, dtype=torch.int32)
        eb = 1 if args.fp8 else 2
        t = timer(lambda: K.paged_attention(q, kc, vc, bt, cu, kl, D ** -0.5, -1, 0.0, ksc, ksc, 1, args.ctx + 1,
                                              nsplit=args.nsplit or None))
        kv_bytes = M * (args.ctx + 1) * hkv * D * 2 * eb
        report(f"attn_decode[{M}x{hq}/{hkv} ctx={args.ctx}]", t, kv_bytes + 4 * M * hq * D,
               4.0 * M * hq * D * (args.ctx + 1))
        if args.prefill:
            P = args.prefill
            nseq = max(1, min(M, 8192 // P))
            qp = torch.randn(nseq * P, hq, D, device=dev, dtype=torch.bfloat16)
            cup = (torch.arange(nseq + 1, device=dev, dtype=torch.int32) * P)
            klp = torch.full((nseq,), P, device=dev, dtype=torch.int32)
            t = timer(lambda: K.paged_attention(qp, kc, vc, bt[:nseq], cup, klp, D ** -0.5, -1, 0.0, ksc, ksc, P, P))
            report(f"attn_prefill[{nseq}x{P} {hq}/{hkv}]", t, nseq * P * (hkv * D * 2 * eb + 4 * hq * D),
                   4.0 * nseq * hq * D * P * P / 2)
    torch.cuda.synchronize()
    status = K.check_status(dev)
    print(json.dumps({"kernel_status": status}))


if __name__ == "__main__":
    main()
