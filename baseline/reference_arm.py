"""Reference arm of ``bench.py``: the unmodified text-generation-inference shard from ``baseline/_ref``
(`pip install --no-deps --target baseline/_ref` of the reference's ``server/`` project), driven
through its own public entry points on the same synthetic workload as the engine's arm.

What runs: ``text_generation_server.models.get_model_with_lora_adapters`` builds the stock
``FlashCausalLM`` / ``FlashLlamaForCausalLM`` from a safetensors directory in ``/dev/shm``;
``model.warmup`` sizes the KV cache and captures the reference's own CUDA graphs;
``FlashCausalLMBatch.from_pb`` / ``concatenate`` / ``model.generate_token`` are the calls behind its
Prefill and Decode RPCs (``server/text_generation_server/server.py:152-226``).  None of the engine's
models, kernels or runtime is imported: the only module taken from ``tgi_b200`` is
``proto/generate_v3.py``, a pure-protobuf description of ``proto/v3/generate.proto`` that stands in
for the ``generate_pb2`` files which the reference's Makefile generates with protoc.

What is substituted (every item is listed in the JSON line under ``reference_shims``): see
``baseline/ref_shims/README.md``.  The kernel modules are resolved by the reference's own
local-module-first loader (``utils/kernels.py:9-19``).
"""
from __future__ import annotations

import json
import math
import os
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "ref_shims")

SHIM_NOTES = [
    "pb.generate_pb2(_grpc): built at run time from the descriptor table in tgi_b200/proto/generate_v3.py (protoc is not in the image)",
    "rotary: local module, one Triton kernel with the contract of flash-attn csrc/rotary apply_rotary",
    "dropout_layer_norm: local module, RMSNorm(+residual) via vllm _custom_ops.fused_add_rms_norm / rms_norm",
    "quantization: local module re-exporting vllm _custom_ops (scaled_fp8_quant, cutlass_scaled_mm, ...)",
    "moe_kernels.fp8_utils: local module re-exporting vllm's Triton w8a8 block-scaled GEMM and per_token_group_quant_fp8",
    "paged_attention, moe: local modules re-exporting vllm ops (import only unless ATTENTION=paged / a MoE model)",
    "peft, punica_sgmv, accelerate.init_empty_weights, kernels, grpc_interceptor, grpc_reflection, outlines: import stand-ins off the forward path",
    "transformers 5: image_utils.VideoInput aliased from video_utils (import of the qwen2.5-vl model file)",
    "checkpoint: attention projections and the first/last layer use per-channel fp8 scales, middle MLPs 128x128 block scales (the reference's Llama loader drops the block size in its no_fp8 scopes)",
    "flashinfer 0.6: BatchPrefillWithPagedKVCacheWrapper.plan accepts the reference's keyword head_dim (renamed head_dim_qk upstream)",
]


# ---------------------------------------------------------------------------------------------------
# environment and shims
# ---------------------------------------------------------------------------------------------------
def _pb2_modules():
    """``text_generation_server.pb.generate_pb2`` and ``generate_pb2_grpc`` without protoc."""
    from google.protobuf.internal import enum_type_wrapper

    from tgi_b200.proto import generate_v3 as g

    pb2 = types.ModuleType("text_generation_server.pb.generate_pb2")
    for name in g._MESSAGES:
        setattr(pb2, name, g.message_class(name))
    for ename in ("GrammarType", "FinishReason"):
        wrapper = enum_type_wrapper.EnumTypeWrapper(getattr(g, ename))
        setattr(pb2, ename, wrapper)
        for vname, number in g._ENUMS[ename]:
            setattr(pb2, vname, number)
    pb2.DESCRIPTOR = g._file_desc

    grpc_mod = types.ModuleType("text_generation_server.pb.generate_pb2_grpc")

    class TextGenerationServiceServicer:   # base class of the reference's servicer
        pass

    def add_TextGenerationServiceServicer_to_server(servicer, server):
        raise RuntimeError("the benchmark does not start the gRPC server")

    grpc_mod.TextGenerationServiceServicer = TextGenerationServiceServicer
    grpc_mod.add_TextGenerationServiceServicer_to_server = add_TextGenerationServiceServicer_to_server
    pkg = types.ModuleType("text_generation_server.pb")
    pkg.__path__ = []
    pkg.generate_pb2 = pb2
    pkg.generate_pb2_grpc = grpc_mod
    return pkg, pb2, grpc_mod


def install(attention: str, cuda_graphs: str):
    """Puts the reference and the stand-in modules on the path and sets the environment the reference's
    launcher would set for a CUDA deployment (``launcher/src/main.rs``: ATTENTION, PREFIX_CACHING,
    CUDA_GRAPHS default 1,2,4,8,16,32)."""
    if not os.path.isdir(os.path.join(REF, "text_generation_server")):
        raise RuntimeError("baseline/_ref/text_generation_server is missing (the reference was not installed)")
    os.environ["ATTENTION"] = attention
    os.environ["PREFIX_CACHING"] = "1" if attention in ("flashinfer", "flashdecoding") else "0"
    os.environ["CUDA_GRAPHS"] = cuda_graphs
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    # transformers probes optional packages by name and caches the answer: ask before the stand-ins
    # named accelerate / peft / kernels become importable, so that it keeps treating them as absent
    from transformers.utils import import_utils as _tiu

    for probe in ("is_accelerate_available", "is_peft_available", "is_kernels_available"):
        fn = getattr(_tiu, probe, None)
        if fn is not None:
            fn()
    for p in (SHIMS, REF):
        if p not in sys.path:
            sys.path.insert(0, p)
    pkg, pb2, grpc_mod = _pb2_modules()
    sys.modules["text_generation_server.pb"] = pkg
    sys.modules["text_generation_server.pb.generate_pb2"] = pb2
    sys.modules["text_generation_server.pb.generate_pb2_grpc"] = grpc_mod
    if attention == "flashinfer":
        _adapt_flashinfer()
    _adapt_transformers()
    return pb2


def _adapt_transformers():
    """The reference pins transformers 4.x; names that moved since are aliased at their old place so that
    its model registry (one try-block over every model file, ``models/__init__.py:83-190``) imports."""
    import transformers.image_utils as iu

    if not hasattr(iu, "VideoInput"):
        try:
            from transformers.video_utils import VideoInput

            iu.VideoInput = VideoInput
        except ImportError:
            pass


def _adapt_flashinfer():
    """flashinfer renamed ``head_dim`` of the paged-prefill ``plan`` to ``head_dim_qk`` after the
    version the reference pins (0.2.0.post2); accept the old keyword."""
    import inspect

    import flashinfer

    cls = flashinfer.BatchPrefillWithPagedKVCacheWrapper
    params = inspect.signature(cls.plan).parameters
    if "head_dim" in params or getattr(cls.plan, "_accepts_head_dim", False):
        return
    inner = cls.plan

    def plan(self, *args, head_dim=None, **kwargs):
        if head_dim is not None:
            kwargs["head_dim_qk"] = head_dim
        return inner(self, *args, **kwargs)

    plan._accepts_head_dim = True
    cls.plan = plan


# ---------------------------------------------------------------------------------------------------
# synthetic checkpoint (HF layout) and tokenizer
# ---------------------------------------------------------------------------------------------------
MODELS = {
    # name: (hidden, layers, heads, kv_heads, intermediate, vocab, block fp8 weights, kv cache dtype)
    "llama70b-fp8": dict(hidden=8192, layers=80, heads=64, kv_heads=8, inter=28672, vocab=128256, fp8=True,
                         kv="fp8_e4m3fn"),
    "llama8b-bf16": dict(hidden=4096, layers=32, heads=32, kv_heads=8, inter=14336, vocab=128256, fp8=False, kv=None),
    "tiny": dict(hidden=1024, layers=4, heads=8, kv_heads=2, inter=2048, vocab=32000, fp8=True, kv="fp8_e4m3fn"),
}


def checkpoint_bytes(m) -> int:
    per_layer = m["hidden"] * (m["heads"] + 2 * m["kv_heads"]) * (m["hidden"] // m["heads"]) + m["hidden"] * m["hidden"] \
        + 3 * m["hidden"] * m["inter"]
    body = per_layer * m["layers"] * (1 if m["fp8"] else 2)
    return body + 2 * m["vocab"] * m["hidden"] * 2


def write_checkpoint(path: str, m: dict, max_pos: int, device, all_block: bool = False):
    """config.json, tokenizer files and one safetensors file per layer.  Weights are N(0, 0.02) in bf16;
    with ``fp8`` the linear layers are stored as e4m3, the MLPs with one fp32 ``weight_scale_inv`` per 128x128
    block (the DeepSeek-style format the reference reads in ``layers/fp8.py:187-396``), the tensors the
    reference's Llama cannot read in that format with per-channel scales (see below); ``all_block`` stores every
    linear layer in the block format (a checkpoint for engines that read it everywhere)."""
    import torch
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    H, L, nh, nkv, I, V = m["hidden"], m["layers"], m["heads"], m["kv_heads"], m["inter"], m["vocab"]
    D = H // nh
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=H, num_hidden_layers=L,
               num_attention_heads=nh, num_key_value_heads=nkv, intermediate_size=I, vocab_size=V, rms_norm_eps=1e-5,
               rope_theta=500000.0, max_position_embeddings=max_pos, hidden_act="silu", tie_word_embeddings=False,
               torch_dtype="bfloat16", bos_token_id=1, eos_token_id=2)
    if m["fp8"]:
        cfg["quantization_config"] = {"quant_method": "fp8", "activation_scheme": "dynamic", "fmt": "e4m3",
                                      "weight_block_size": [128, 128]}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    _write_tokenizer(path, V)
    gen = torch.Generator(device=device).manual_seed(0)

    def rnd(*shape):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def linear(out, name, rows, cols, block):
        w = rnd(rows, cols)
        if not m["fp8"]:
            out[name + ".weight"] = w.cpu()
            return
        if block:
            blocks = w.float().reshape(rows // 128, 128, cols // 128, 128)
            scale = blocks.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-12) / 448.0
            q = (blocks / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(rows, cols)
            out[name + ".weight_scale_inv"] = scale.reshape(rows // 128, cols // 128).float().cpu()
        else:
            scale = w.float().abs().amax(dim=1, keepdim=True).clamp(min=1e-12) / 448.0
            q = (w.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
            out[name + ".weight_scale"] = scale.float().cpu()
        out[name + ".weight"] = q.cpu()

    weight_map = {}

    def flush(tensors, fname):
        save_file(tensors, os.path.join(path, fname))
        for k in tensors:
            weight_map[k] = fname

    flush({"model.embed_tokens.weight": rnd(V, H).cpu(), "model.norm.weight": torch.ones(H, dtype=torch.bfloat16),
           "lm_head.weight": rnd(V, H).cpu()}, "model-embed.safetensors")
    for layer in range(L):
        p = f"model.layers.{layer}"
        t = {p + ".input_layernorm.weight": torch.ones(H, dtype=torch.bfloat16),
             p + ".post_attention_layernorm.weight": torch.ones(H, dtype=torch.bfloat16)}
        # The reference's Llama builds the attention projections of every layer, and the whole first and last
        # layer, inside its `no_fp8` scope, whose loader has no block size (`flash_llama_modeling.py:124-134,
        # 411, 514, 549`): those tensors can only be read as fp8 with a per-output-channel `weight_scale`.
        # All weights stay e4m3 either way, so the bytes a decode step streams are those of the block format.
        mlp_block = all_block or 0 < layer < L - 1
        linear(t, p + ".self_attn.q_proj", nh * D, H, all_block)
        linear(t, p + ".self_attn.k_proj", nkv * D, H, all_block)
        linear(t, p + ".self_attn.v_proj", nkv * D, H, all_block)
        linear(t, p + ".self_attn.o_proj", H, nh * D, all_block)
        linear(t, p + ".mlp.gate_proj", I, H, mlp_block)
        linear(t, p + ".mlp.up_proj", I, H, mlp_block)
        linear(t, p + ".mlp.down_proj", H, I, mlp_block)
        flush(t, f"model-{layer:05d}.safetensors")
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)


def _write_tokenizer(path: str, vocab: int):
    """A word-level tokenizer whose token ``i`` (from 3 up) is the text ``t<i>``: prompts are written as such words so
    that the reference, which tokenises the request text itself, sees exactly the intended random ids."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    words = {f"t{i}": i for i in range(3, vocab)}
    words.update({"<unk>": 0, "<s>": 1, "</s>": 2})
    tok = Tokenizer(models.WordLevel(words, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "model_max_length": 1 << 20, "bos_token": "<s>",
                   "eos_token": "</s>", "unk_token": "<unk>"}, f)


# ---------------------------------------------------------------------------------------------------
# the run
# ---------------------------------------------------------------------------------------------------
def run(args, sampler_factory):
    """Returns the JSON record of the reference arm (raises on any failure; the caller turns the
    exception text into the ``unavailable`` line)."""
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: the reference's flash models only run on a GPU")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m = dict(MODELS[args.model])
    if args.layers:
        m["layers"] = args.layers
    attention = os.environ.get("TGI_REF_ATTENTION", "flashinfer")
    if m["kv"] is not None and attention != "flashinfer":
        raise RuntimeError("an fp8 KV cache needs ATTENTION=flashinfer in the reference")
    pb2 = install(attention, os.environ.get("TGI_REF_CUDA_GRAPHS", "1,2,4,8,16,32"))
    torch.cuda.set_device(rank % torch.cuda.device_count())
    device = torch.device("cuda", torch.cuda.current_device())

    C, P, O = args.concurrency, args.prompt_len, args.output_len
    max_pos = max(8192, P + O + 8)
    ckpt = os.path.join("/dev/shm", f"tgi_ref_{args.model}_{m['layers']}L")
    marker = os.path.join(ckpt, ".complete")
    if rank == 0 and not os.path.exists(marker):
        need = checkpoint_bytes(m)
        st = os.statvfs("/dev/shm")
        avail = st.f_bavail * st.f_frsize
        if avail < need * 1.15:
            raise RuntimeError(f"/dev/shm has {avail / 1e9:.0f} GB free, the synthetic checkpoint needs {need / 1e9:.0f} GB")
        write_checkpoint(ckpt, m, max_pos, device)
        torch.cuda.empty_cache()
        open(marker, "w").close()
    deadline = time.time() + 1800
    while not os.path.exists(marker):
        if time.time() > deadline:
            raise RuntimeError("timed out waiting for rank 0 to write the synthetic checkpoint")
        time.sleep(0.5)

    from text_generation_server.models import get_model_with_lora_adapters
    from text_generation_server.models.flash_causal_lm import FlashCausalLMBatch
    from text_generation_server.models.globals import BLOCK_SIZE
    from text_generation_server.utils.speculate import set_speculate

    from text_generation_server.utils.prefill_chunking import set_max_prefill_tokens

    set_speculate(0)
    t_load = time.time()
    model = get_model_with_lora_adapters(
        ckpt, [], None, world > 1, None, None, "bfloat16", m["kv"], False, max_input_tokens=P, adapter_to_index={})
    load_s = time.time() - t_load

    rng = np.random.default_rng(1234)

    def request(rid, n_tokens, max_new, blocks):
        ids = rng.integers(3, m["vocab"], size=n_tokens)
        text = " ".join(f"t{i}" for i in ids)
        slots = [s for b in blocks for s in range(b * BLOCK_SIZE, (b + 1) * BLOCK_SIZE)]
        return pb2.Request(
            id=rid, inputs=text, input_chunks=pb2.Input(chunks=[pb2.InputChunk(text=text)]), truncate=n_tokens,
            add_special_tokens=False, prefill_logprobs=False, top_n_tokens=0,
            parameters=pb2.NextTokenChooserParameters(temperature=1.0, top_k=0, top_p=1.0, typical_p=1.0, do_sample=False,
                                                      seed=0, repetition_penalty=1.0, frequency_penalty=0.0, watermark=False),
            stopping_parameters=pb2.StoppingCriteriaParameters(max_new_tokens=max_new, ignore_eos_token=True),
            blocks=blocks, slots=slots, cache_len=0)

    # The workload of the engine's arm: every request arrives with its context already at the middle of the
    # 512-token generation (prompt of `start_ctx` random tokens), so the K timed decode steps see the average
    # KV length of the run.  Blocks are handed out as the reference's router would (P + O tokens per request).
    start_ctx = P + max(0, (O - args.steps - args.warmup) // 2)
    blocks_per_req = math.ceil((P + O) / BLOCK_SIZE)

    # warmup, as the router does at start-up: one batch of max_batch_prefill_tokens tokens
    prefill_tokens = max(args.prefill_chunk, start_ctx)
    group = max(1, prefill_tokens // start_ctx)
    warm = pb2.Batch(id=0, size=group, max_tokens=group * (P + O), max_blocks=blocks_per_req, requests=[
        request(i, start_ctx, 2, []) for i in range(group)])
    set_max_prefill_tokens(prefill_tokens)   # first statement of the reference's Warmup RPC (server.py:100-101)
    warm_batch = FlashCausalLMBatch.from_pb(warm, model.tokenizer, model.dtype, model.device)
    max_supported, _, _ = model.warmup(warm_batch, start_ctx, P + O)
    if max_supported < C * (P + O):
        raise RuntimeError(f"the reference's KV cache holds {max_supported} tokens, the workload needs {C * (P + O)}")

    # prefill the running batch in groups of max_batch_prefill_tokens, as its router would admit them
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    batches, next_block, rid = [], 1, 0
    torch.cuda.synchronize()
    ev[0].record()
    while rid < C:
        n = min(group, C - rid)
        reqs = []
        for _ in range(n):
            reqs.append(request(rid, start_ctx, O, list(range(next_block, next_block + blocks_per_req))))
            next_block += blocks_per_req
            rid += 1
        pbatch = pb2.Batch(id=len(batches) + 1, size=n, max_tokens=n * (P + O), max_blocks=blocks_per_req, requests=reqs)
        b = FlashCausalLMBatch.from_pb(pbatch, model.tokenizer, model.dtype, model.device)
        _, nb, _ = model.generate_token(b)
        batches.append(nb)
    ev[1].record()
    torch.cuda.synchronize()
    prefill_ms = ev[0].elapsed_time(ev[1])
    batch = FlashCausalLMBatch.concatenate(batches) if len(batches) > 1 else batches[0]
    del batches

    for _ in range(args.warmup):
        _, batch, _ = model.generate_token(batch)
    ctx = start_ctx + args.warmup

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = sampler_factory(torch.cuda.current_device())
    barrier()
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    n_tokens = 0
    for _ in range(args.steps):
        gens, batch, _ = model.generate_token(batch)
        n_tokens += len(gens)
    stop.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if rank == 0 else {}
    dev_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([dev_ms, wall_ms], device=device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dev_ms, wall_ms = t.tolist()
    # every rank returns only the generations with id % world == rank; the step emits C tokens in total
    tokens_per_step = C
    return {
        "impl": "reference",
        "value": tokens_per_step * args.steps / (dev_ms * 1e-3),
        "ms_per_step": dev_ms / args.steps,
        "e2e": {"value": tokens_per_step * args.steps / (wall_ms * 1e-3), "unit": "tok/s",
                "api": "text_generation_server FlashCausalLM.generate_token",
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "ms_per_step": wall_ms / args.steps},
        "clocks": clocks,
        "reference": {"attention": attention, "cuda_graphs": os.environ["CUDA_GRAPHS"], "block_size": int(BLOCK_SIZE),
                      "kv_cache_dtype": m["kv"] or "bfloat16", "context_at_timed_steps": ctx, "load_s": round(load_s, 1),
                      "prefill_ms": round(prefill_ms, 1), "prefill_tok_s": round(C * start_ctx / (prefill_ms * 1e-3), 1),
                      "kv_cache_tokens": int(max_supported)},
        "reference_shims": SHIM_NOTES,
    }
