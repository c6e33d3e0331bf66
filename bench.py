#!/usr/bin/env python
"""Serving benchmark: decode throughput of a Llama-3-70B-shape model in block-scaled fp8.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N ...             # the unmodified reference shard (baseline/_ref)

Workload (the headline configuration): Llama-3-70B shape (80 layers, hidden 8192, 64/8 heads,
intermediate 28672, vocab 128256), weights e4m3 with 128x128 block scales quantised from seeded
N(0, 0.02) values, activations quantised per token in 1x128 groups, fp8 KV cache with per-head
scales, tensor parallel over the N GPUs.  `--concurrency` requests (default 256) with
`--prompt-len` random-token prompts (default 1024) are prefilled through the engine (that phase gives
the TTFT figures); a *step* is then one decode iteration of the whole running batch, i.e. it emits
`concurrency` output tokens at a context that sits in the middle of the 512-token generation.

Reported numbers:
  value        output tokens/s of K decode steps replayed from the captured CUDA graph, timed with
               CUDA events (max over ranks).
  e2e.value    the same K steps driven through the shard's public API (`generate_token`, the call
               behind the Decode RPC): every step copies its inputs from pinned host memory, runs
               the step, samples, reads the new tokens back and does the host bookkeeping.
Weights (>= 8.75 GB per rank) and KV pages read by every step are far larger than the 126 MB L2, so
consecutive timed steps cannot hit in L2 (`l2: inputs larger than L2`).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "output tok/s (decode, Llama-3-70B-shape block-fp8, TP=N)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="llama70b-fp8", choices=["llama70b-fp8", "llama8b-bf16", "mixtral-bf16", "tiny"])
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--prefill-chunk", type=int, default=8192, help="tokens per prefill forward")
    ap.add_argument("--fast-setup", action="store_true",
                    help="development only: fill the KV cache with random values instead of running prefill")
    ap.add_argument("--layers", type=int, default=0, help="development only: override the layer count")
    ap.add_argument("--moe-skew", type=float, default=0.0,
                    help="MoE models: add this bias to the router logits of experts 0 and 1 (load-imbalance case)")
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "nucleus"],
                    help="nucleus = temperature 0.7, top-p 0.9, repetition penalty 1.1 on every request")
    return ap.parse_args()


def reference_main(args):
    """Runs the unmodified reference shard (``baseline/_ref``) on the same workload and prints the same JSON
    line with ``impl: reference``; if any step of that attempt fails, the line says ``unavailable`` with the
    exception of the attempt."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    try:
        if args.model not in ("llama70b-fp8", "llama8b-bf16", "tiny"):
            raise RuntimeError(f"no reference arm for --model {args.model}")
        from baseline import reference_arm

        rec = reference_arm.run(args, ClockSampler)
    except BaseException as err:  # noqa: BLE001 - report whatever stopped the attempt
        if isinstance(err, KeyboardInterrupt):
            raise
        import traceback

        traceback.print_exc()
        msg = f"{type(err).__name__}: {err}".replace("\n", " ")[:600]
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": msg}), flush=True)
        sys.stdout.flush()
        os._exit(0)
    if rank == 0:
        C = args.concurrency
        out = {
            "metric": METRIC if args.model == "llama70b-fp8" else f"output tok/s (decode, {args.model}, TP=N)",
            "value": round(rec["value"], 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(rec["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 (block-scaled weights+activations, fp8 KV)" if args.model != "llama8b-bf16" else "bf16",
            "data": "synthetic: random-token prompts, random-init N(0,0.02) weights", "impl": "reference",
            "config": {"model": args.model if not args.layers else f"{args.model}-{args.layers}L", "global_batch": C,
                       "seq_len": rec["reference"]["context_at_timed_steps"], "nominal_prompt_len": args.prompt_len,
                       "output_len": args.output_len, "parallelism": f"tp{world}",
                       "collectives": "none (one GPU)" if world == 1 else "nccl", "l2": "inputs larger than L2",
                       "timed": "CUDA events around K calls of generate_token, max over ranks"},
            "e2e": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in rec["e2e"].items()},
            "clocks": rec["clocks"], "reference": rec["reference"], "reference_shims": rec["reference_shims"],
        }
        print(json.dumps(out), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)   # same reason as in main(): no communicator tear-down with live CUDA graphs


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._halt = threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(float(parts[0]))
                    self.max_mhz = float(parts[1])
                    for n, v in zip(names, parts[2:6]):
                        if v.lower().startswith("active"):
                            self.reasons.add(n)
            except Exception:
                pass
            self._halt.wait(0.2)

    def stop(self):
        self._halt.set()
        self.join(timeout=3)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def model_config(args):
    from tgi_b200.utils import synthetic as syn

    if args.model == "llama70b-fp8":
        cfg, fp8, kv_fp8 = syn.llama3_70b_config(), True, True
    elif args.model == "llama8b-bf16":
        cfg, fp8, kv_fp8 = syn.llama3_8b_config(), False, False
    elif args.model == "mixtral-bf16":
        # Mixtral-8x7B shape; with N > 1 the experts are placed whole on the ranks (expert parallel), attention
        # stays tensor parallel
        cfg, fp8, kv_fp8 = syn.mixtral_8x7b_config(), False, False
    else:
        cfg = syn.llama_config(hidden=1024, layers=4, heads=8, kv_heads=2, intermediate=2048, vocab=32000, max_pos=8192)
        cfg["quantization_config"] = {"quant_method": "fp8", "weight_block_size": [128, 128]}
        fp8, kv_fp8 = True, True
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    # long-context runs: the rotary table must cover every position that will be generated
    cfg["max_position_embeddings"] = max(int(cfg["max_position_embeddings"]), args.prompt_len + args.output_len + 8)
    return cfg, fp8, kv_fp8


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_main(args)

    import numpy as np
    import torch

    from tgi_b200.models.arch import ModelConfig
    from tgi_b200.models.decoder import CausalDecoder
    from tgi_b200.models.flash_causal_lm import BLOCK_SIZE, FlashCausalLM, FlashCausalLMBatch
    from tgi_b200.models.graphs import DecodeGraphs
    from tgi_b200.ops import cuda as K
    from tgi_b200.parallel.dist import initialize_torch_distributed
    from tgi_b200.proto import generate_v3 as pb
    from tgi_b200.utils.quantization import DefaultWeightsLoader, Fp8Loader
    from tgi_b200.utils.synthetic import SyntheticWeights
    from tgi_b200.utils.tokenizer import ByteTokenizer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("--gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    pg, rank, world = initialize_torch_distributed()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    K.load()
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg, fp8, kv_fp8 = model_config(args)
    weights = SyntheticWeights(cfg, dev, torch.bfloat16, process_group=pg, fp8_block=fp8)
    weights.weights_loader = Fp8Loader(weight_block_size=[128, 128]) if fp8 else DefaultWeightsLoader()
    t0 = time.time()
    from tgi_b200.parallel.peer import make_comm

    comm = make_comm(pg, rank, world, dev, cfg["hidden_size"], max(args.prefill_chunk, args.concurrency))
    model = CausalDecoder(ModelConfig(cfg), weights, comm=comm)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    C, P, O = args.concurrency, args.prompt_len, args.output_len
    # decode context: centred in the generation so K steps see the average KV length of the run
    start_ctx = P + max(0, (O - args.steps - args.warmup) // 2)
    max_total = P + O
    runner = FlashCausalLM(model, ByteTokenizer(cfg["vocab_size"]), torch.bfloat16, dev, rank, world,
                           kv_cache_dtype=torch.float8_e4m3fn if kv_fp8 else torch.bfloat16)
    blocks_per_seq = math.ceil(max_total / BLOCK_SIZE)
    runner.init_kv_cache(1 + C * blocks_per_seq)
    if args.moe_skew:
        for layer in model.layers:
            router = getattr(layer.mlp, "router", None)
            if router is not None:
                bias = torch.zeros(router.weight.shape[0], dtype=router.weight.dtype, device=dev)
                bias[:2] = args.moe_skew
                router.bias = bias
    if kv_fp8:
        for layer in model.layers:
            layer.attn.k_scale = torch.full((model.dims.num_kv_heads,), 0.05, device=dev)
            layer.attn.v_scale = torch.full((model.dims.num_kv_heads,), 0.05, device=dev)

    rng = np.random.default_rng(1234)       # same seed on every rank: identical prompts everywhere
    vocab = cfg["vocab_size"]
    prompts = [rng.integers(3, vocab, size=start_ctx).tolist() for _ in range(C)]

    def make_request(i):
        r = pb.Request(id=i, inputs="")
        nucleus = args.sampling == "nucleus"
        r.parameters.temperature = 0.7 if nucleus else 1.0
        r.parameters.top_p = 0.9 if nucleus else 1.0
        r.parameters.typical_p = 1.0
        r.parameters.repetition_penalty = 1.1 if nucleus else 1.0
        if nucleus:
            r.parameters.do_sample = True
            r.parameters.seed = 1000 + i
        r.stopping_parameters.max_new_tokens = O
        r.stopping_parameters.ignore_eos_token = True
        r.blocks.extend(range(1 + i * blocks_per_seq, 1 + (i + 1) * blocks_per_seq))
        return r

    # ---- prefill phase (real prefill through the engine; gives TTFT) ------------------------------
    per_batch = max(1, args.prefill_chunk // start_ctx)
    batches, ttft_ms, prefill_tokens = [], [], 0
    barrier()
    t_prefill0 = time.time()
    if args.fast_setup:
        for k, v in runner.kv_cache:
            k.view(torch.uint8).random_(0, 120) if kv_fp8 else k.normal_()
            v.view(torch.uint8).random_(0, 120) if kv_fp8 else v.normal_()
        bpb = pb.Batch(id=0, requests=[make_request(i) for i in range(C)], size=C)
        batch = FlashCausalLMBatch.from_tokenized(bpb, prompts, runner.tokenizer, torch.bfloat16, dev)
        for s in batch.seqs:                  # pretend the prompt is cached and one token was sampled
            s.cache_len, s.prefilling = s.prompt_len, False
            s.ids.append(int(rng.integers(3, vocab)))
    else:
        for lo in range(0, C, per_batch):
            ids = list(range(lo, min(C, lo + per_batch)))
            bpb = pb.Batch(id=lo, requests=[make_request(i) for i in ids], size=len(ids))
            b = FlashCausalLMBatch.from_tokenized(bpb, [prompts[i] for i in ids], runner.tokenizer, torch.bfloat16, dev)
            t_b = time.time()
            _, b, _ = runner.generate_token(b)
            torch.cuda.synchronize()
            ttft_ms.append((time.time() - t_b) * 1e3)          # one prefill step: prompt in, first token out
            prefill_tokens += sum(len(prompts[i]) for i in ids)
            batches.append(b)
        batch = FlashCausalLMBatch.concatenate(batches)
    barrier()
    prefill_s = time.time() - t_prefill0
    assert K.check_status(dev) == 0, "a kernel wait timed out during prefill"

    # ---- capture the decode graph for this batch size -------------------------------------------
    runner.graphs = DecodeGraphs(runner, max_total, buckets=[C])
    runner.graphs.capture_all()
    bucket = runner.graphs.buckets[C]

    # count kernel launches of one eager decode step (the graph replays exactly these)
    K.LAUNCHES = 0
    counts = batch.plan_step()
    meta, _ = runner.build_meta(batch, counts)
    # the eager step re-writes the KV of the current position with identical values: harmless
    runner.forward(meta)
    torch.cuda.synchronize()
    launches_per_step = K.LAUNCHES

    # ---- e2e: K steps through the public API (warm-up first) ------------------------------------
    def api_step(b):
        gens, nb, _ = runner.generate_token(b)
        return nb

    for _ in range(args.warmup):
        batch = api_step(batch)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_api0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        batch = api_step(batch)
    e1.record()
    barrier()
    api_s = time.perf_counter() - t_api0
    api_dev_ms = e0.elapsed_time(e1)
    h2d_bytes = bucket.total * 4
    d2h_bytes = 2 * C * 4

    # ---- device-timed graph replays -------------------------------------------------------------
    for _ in range(args.warmup):
        bucket.graph.replay()
    barrier()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(args.steps):
        bucket.graph.replay()
    g1.record()
    barrier()
    graph_ms = g0.elapsed_time(g1)
    clocks = sampler.stop() if rank == 0 else {}
    status = K.check_status(dev)

    vals = torch.tensor([graph_ms, api_s * 1e3, api_dev_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    graph_ms, api_ms, api_dev_ms = vals.tolist()
    if rank == 0:
        ms_per_step = graph_ms / args.steps
        value = C * args.steps / (graph_ms / 1e3)
        e2e_value = C * args.steps / (api_ms / 1e3)
        ttft_sorted = sorted(ttft_ms)
        out = {
            "metric": METRIC if args.model == "llama70b-fp8" else f"output tok/s (decode, {args.model}, TP=N)", "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (block-scaled weights+activations, fp8 KV)"
            if fp8 else "bf16", "data": "synthetic: random-token prompts, random-init N(0,0.02) weights",
            "impl": "b200",
            "config": {"model": args.model if not args.layers else f"{args.model}-{args.layers}L",
                       "global_batch": C, "seq_len": start_ctx + args.warmup, "prompt_len": start_ctx,
                       "nominal_prompt_len": P, "output_len": O,
                       "parallelism": f"tp{world}", "collectives": "none (one GPU)" if world == 1 else ("nccl" if comm is None else "peer-memory kernels"), "block_size": BLOCK_SIZE, "l2": "inputs larger than L2",
                       "timed": "CUDA events around K graph replays, max over ranks",
                       "setup": "fast-setup (random KV, development)" if args.fast_setup else "real prefill",
                       **({"fp8_gemm": "tcgen05 block-scaled MMA, power-of-two block scales (weights requantised at load)"
                           if K.fp8_mx() else "per-K-block promotion, checkpoint scales"} if fp8 else {}),
                       **({"moe_skew": args.moe_skew} if args.moe_skew else {}),
                       **({"sampling": "T=0.7 top-p=0.9 rep=1.1"} if args.sampling == "nucleus" else {})},
            "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "ms_per_step": round(api_ms / args.steps, 4),
                    "device_ms_per_step": round(api_dev_ms / args.steps, 4),
                    "api": "FlashCausalLM.generate_token (Decode RPC body)"},
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks,
            "itl_ms_p50": round(api_ms / args.steps, 4),
            # time of one prefill step (a batch of whole prompts up to --prefill-chunk tokens): what a request waits
            # for its first token when it is scheduled at once; served TTFT percentiles come from client/load_test.py
            "prefill_step_ms_p50": round(ttft_sorted[len(ttft_sorted) // 2], 2) if ttft_sorted else None,
            "prefill_all_s": round(prefill_s, 2),
            "prefill_tok_s": round(prefill_tokens / prefill_s, 1) if prefill_tokens else None,
            "load_s": round(load_s, 1), "kernel_status": status,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group whose collectives
        # were captured into still-alive CUDA graphs can block forever.  All results are printed and
        # every rank has passed the barrier, so a hard exit loses nothing.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
