"""Any ``transformers`` decoder-only model on the paged KV cache and the paged attention kernels.

Reference: ``models/transformers_flash_causal_lm.py:20-84`` (an attention function registered in
``ALL_ATTENTION_FUNCTIONS`` that stores K/V into the paged cache and calls the engine's attention) and
``:96-290`` (the runner).  It is the middle link of the dispatch chain: architectures with a native
decoder (``models/arch.py``) run there; a model type that is unknown here but whose ``transformers``
implementation goes through the attention interface runs its own modules (norms, MLPs, rotary
embedding, whatever they are) around this attention, and keeps continuous batching, prefix caching,
chunked prefill and CUDA-graph decode; everything else falls back to the padded runners.

The model sees one ragged "sequence" ``[1, T]`` that holds the tokens of every request of the step,
with per-token ``position_ids``.  The attention function ignores the mask ``transformers`` would build
and uses the step's block tables and sequence lengths instead; they reach it through a context
variable set around the forward call, so no assumption is made about how a model forwards keyword
arguments to its layers.
"""
from __future__ import annotations

import contextvars
from typing import List, Optional, Tuple

import torch

from .. import ops
from .arch import ModelDims
from .decoder import ForwardMeta

ATTN_NAME = "tgi_b200_paged"

# (ForwardMeta, kv_cache) of the forward pass in flight
_STEP: contextvars.ContextVar = contextvars.ContextVar("tgi_b200_step", default=None)


def store_kv(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slots: torch.Tensor):
    """Scatter ``[T, Hkv, D]`` keys/values into ``[blocks, block_size, Hkv, D]`` pages; slot -1 is a pad row."""
    kc = k_cache.view(-1, k_cache.shape[-2], k_cache.shape[-1])
    vc = v_cache.view(-1, v_cache.shape[-2], v_cache.shape[-1])
    # pad rows are redirected to slot 0 (block 0 is reserved: no sequence ever reads it)
    idx = slots.long().clamp_min(0)
    kc.index_copy_(0, idx, key.to(kc.dtype))
    vc.index_copy_(0, idx, value.to(vc.dtype))


def paged_attention_forward(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0,
                            sliding_window=None, softcap=None, **kwargs):
    """``transformers`` attention interface: query ``[1, H, T, D]``, key/value ``[1, Hkv, T, D]`` (already
    rotated) -> ``[1, T, H, D]``."""
    step = _STEP.get()
    if step is None:
        raise RuntimeError(f"attention implementation {ATTN_NAME!r} was called outside TransformersDecoder.forward")
    meta, kv_cache = step
    k_cache, v_cache = kv_cache[module.layer_idx]
    q = query[0].transpose(0, 1).contiguous()
    k = key[0].transpose(0, 1).contiguous()
    v = value[0].transpose(0, 1).contiguous()
    store_kv(k, v, k_cache, v_cache, meta.slots)
    D = q.shape[-1]
    window = int(sliding_window) if sliding_window else -1
    out = ops.paged_attention(q, k_cache, v_cache, meta.block_tables, meta.cu_seqlens_q, meta.kv_lens,
                              float(scaling if scaling is not None else D ** -0.5), window,
                              float(softcap or 0.0), None, None, meta.max_q, meta.max_kv)
    return out.view(1, q.shape[0], q.shape[1], D), None


_registered = False


def register():
    """Make ``attn_implementation="tgi_b200_paged"`` known to ``transformers`` (idempotent)."""
    global _registered
    if _registered:
        return
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, flash_attention_mask

    AttentionInterface.register(ATTN_NAME, paged_attention_forward)
    # no dense mask: causality and sequence boundaries come from the block tables
    AttentionMaskInterface.register(ATTN_NAME, flash_attention_mask)
    _registered = True


class ShardedLinear(torch.nn.Module):
    """One rank's part of a ``torch.nn.Linear`` under tensor parallelism.

    The styles are those of the ``base_model_tp_plan`` a ``transformers`` config carries
    (``integrations/tensor_parallel.py`` in that library): ``colwise`` keeps a contiguous slice of the output
    features (for q / k / v that is a contiguous range of heads) and returns it; ``colwise_gather_output`` returns the
    full output (models that normalise q or k over all heads, or split a fused gate_up themselves); ``rowwise``
    multiplies the rank's slice of the input features and sums the partial outputs over the ranks;
    ``rowwise_split_input`` receives the full input and cuts its own slice first.  The bias of a row-parallel layer is
    added once, after the sum.
    """

    STYLES = ("colwise", "colwise_gather_output", "rowwise", "rowwise_split_input")

    def __init__(self, linear: torch.nn.Linear, style: str, rank: int, world: int, group):
        super().__init__()
        if style not in self.STYLES:
            raise NotImplementedError(f"tensor-parallel style {style!r}")
        out_f, in_f = linear.weight.shape
        self.style, self.rank, self.world, self.group = style, rank, world, group
        if style.startswith("colwise"):
            if out_f % world:
                raise ValueError(f"{out_f} output features cannot be split over {world} ranks")
            per = out_f // world
            w = linear.weight.detach()[rank * per:(rank + 1) * per]
            b = None if linear.bias is None else linear.bias.detach()[rank * per:(rank + 1) * per]
        else:
            if in_f % world:
                raise ValueError(f"{in_f} input features cannot be split over {world} ranks")
            per = in_f // world
            w = linear.weight.detach()[:, rank * per:(rank + 1) * per]
            b = None if linear.bias is None else linear.bias.detach()
        self.per = per
        self.weight = torch.nn.Parameter(w.clone().contiguous(), requires_grad=False)
        self.bias = None if b is None else torch.nn.Parameter(b.clone().contiguous(), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..parallel import dist as pdist

        if self.style == "colwise":
            return torch.nn.functional.linear(x, self.weight, self.bias)
        if self.style == "colwise_gather_output":
            y = torch.nn.functional.linear(x, self.weight, self.bias)
            rows = y.reshape(-1, y.shape[-1]).contiguous()
            parts = torch.empty(self.world * rows.shape[0], rows.shape[1], dtype=y.dtype, device=y.device)
            pdist.all_gather_into(parts, rows, self.group)      # rank-major blocks of rows
            full = parts.view(self.world, rows.shape[0], rows.shape[1]).transpose(0, 1)
            return full.reshape(*y.shape[:-1], self.world * y.shape[-1])
        if self.style == "rowwise_split_input":
            x = x[..., self.rank * self.per:(self.rank + 1) * self.per]
        y = torch.nn.functional.linear(x, self.weight)
        y = pdist.all_reduce(y.contiguous(), self.group)
        return y if self.bias is None else y + self.bias


def shard_model(hf_model, rank: int, world: int, group, plan: Optional[dict] = None, head_attrs=()) -> dict:
    """Replace the linear layers named by the config's ``base_model_tp_plan`` with this rank's part.  Returns
    ``{"heads_sharded": bool, "kv_sharded": bool}``: whether the attention of a layer sees a slice of the heads (q / k
    column-parallel without a gather) or all of them.  Reference: ``models/transformers_flash_causal_lm.py:137-150``
    loads with ``tp_plan="auto"``, which applies the same plan through DTensor hooks.  ``plan`` overrides the config's
    (model types whose config carries none); ``head_attrs`` names integer attributes of an attention module (its head
    count) that are divided by the number of ranks when its q projection is column parallel, for modelling code that
    reshapes with a stored head count instead of ``-1``."""
    import re

    cfg = hf_model.config.get_text_config() if hasattr(hf_model.config, "get_text_config") else hf_model.config
    plan = dict(plan or getattr(cfg, "base_model_tp_plan", None) or {})
    if not plan:
        raise NotImplementedError(f"model type {cfg.model_type!r} carries no tensor-parallel plan")
    body = getattr(hf_model, hf_model.base_model_prefix, None) or hf_model.model
    rules = [(re.compile("^" + re.escape(k).replace(r"\*", r"\d+") + "$"), v) for k, v in plan.items()]
    info = {"heads_sharded": False, "kv_sharded": False}
    todo = []
    for name, mod in body.named_modules():
        for rx, style in rules:
            if rx.match(name):
                if not isinstance(mod, torch.nn.Linear):
                    raise NotImplementedError(f"tensor-parallel plan names {name} ({type(mod).__name__}), not a Linear")
                todo.append((name, mod, style))
                break
    if not todo:
        raise NotImplementedError("the tensor-parallel plan matches no module")
    for name, mod, style in todo:
        parent_name, _, leaf = name.rpartition(".")
        parent = body.get_submodule(parent_name) if parent_name else body
        setattr(parent, leaf, ShardedLinear(mod, style, rank, world, group))
        if style == "colwise" and leaf in ("q_proj", "qkv_proj", "query_key_value"):
            info["heads_sharded"] = True
            for attr in head_attrs:
                n = getattr(parent, attr, None)
                if isinstance(n, int):
                    if n % world:
                        raise ValueError(f"{n} heads cannot be split over {world} ranks")
                    setattr(parent, attr, n // world)
        if style == "colwise" and leaf in ("k_proj", "qkv_proj", "query_key_value"):
            info["kv_sharded"] = True
    return info


class TransformersDecoder:
    """Adapter with the interface ``FlashCausalLM`` expects from a decoder (``dims``, ``forward``)."""

    comm = None
    speculator = None
    supports_local_head = False

    def __init__(self, hf_model, device, dtype, world: int = 1, heads_sharded: bool = False, kv_sharded: bool = False):
        self.hf = hf_model.eval()
        cfg = hf_model.config.get_text_config() if hasattr(hf_model.config, "get_text_config") else hf_model.config
        total_heads = int(cfg.num_attention_heads)
        head_dim = int(getattr(cfg, "head_dim", None) or cfg.hidden_size // total_heads)
        total_kv = int(getattr(cfg, "num_key_value_heads", None) or total_heads)
        if (heads_sharded and total_heads % world) or (kv_sharded and total_kv % world):
            raise ValueError(f"{total_heads} / {total_kv} heads cannot be split over {world} ranks")
        # the heads this rank's attention sees: a slice when q / k are column parallel, else all of them
        heads = total_heads // world if heads_sharded else total_heads
        kv = total_kv // world if kv_sharded else total_kv
        layers = int(cfg.num_hidden_layers)
        window = getattr(cfg, "sliding_window", None)
        layer_types = getattr(cfg, "layer_types", None)
        if layer_types:
            windows = [int(window) if (t == "sliding_attention" and window) else -1 for t in layer_types]
        else:
            windows = [int(window) if window and getattr(cfg, "use_sliding_window", True) else -1] * layers
        supported = (64, 128, 256)
        if head_dim not in supported:
            raise NotImplementedError(f"head dimension {head_dim} has no attention kernel instance")
        self.dims = ModelDims(
            hidden=int(cfg.hidden_size), num_layers=layers, num_heads=heads, num_kv_heads=kv, head_dim=head_dim,
            intermediate=int(getattr(cfg, "intermediate_size", 0) or 0), vocab=int(cfg.vocab_size),
            eps=float(getattr(cfg, "rms_norm_eps", 1e-5)), rope_theta=float(getattr(cfg, "rope_theta", 10000.0) or 10000.0),
            rot_dim=head_dim, max_positions=int(getattr(cfg, "max_position_embeddings", 2048)),
            act=str(getattr(cfg, "hidden_act", "silu")), softmax_scale=head_dim ** -0.5, windows=windows,
            attn_softcap=0.0, logit_softcap=0.0, logit_scale=1.0, embed_scale=1.0, residual_scale=1.0,
            total_heads=total_heads, total_kv_heads=total_kv, attn_head_dim=head_dim)
        self.device, self.dtype = device, dtype
        # Llama-4 style chunked attention (a token sees only the keys of its own chunk) has no counterpart in the
        # paged kernels: contexts that stay inside one chunk are exact, longer ones are refused instead of being
        # silently attended in full
        chunked = layer_types and any(t == "chunked_attention" for t in layer_types)
        self.attention_chunk = int(getattr(cfg, "attention_chunk_size", 0) or 0) if chunked else 0

    @torch.no_grad()
    def forward(self, meta: ForwardMeta, kv_cache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if self.attention_chunk and int(meta.max_kv) > self.attention_chunk:
            raise ValueError(      # fails the batch; the shard keeps serving
                f"a context of {int(meta.max_kv)} tokens crosses the model's attention chunk of {self.attention_chunk} "
                "tokens; chunked attention is not implemented in the paged kernels")
        token = _STEP.set((meta, kv_cache))
        try:
            kw = dict(position_ids=meta.positions.long().unsqueeze(0), use_cache=False, return_dict=True)
            if meta.inputs_embeds is not None:
                kw["inputs_embeds"] = meta.inputs_embeds.unsqueeze(0)
            else:
                kw["input_ids"] = meta.input_ids.long().unsqueeze(0)
            body = getattr(self.hf, self.hf.base_model_prefix, None) or self.hf.model
            hidden = body(**kw).last_hidden_state[0]
        finally:
            _STEP.reset(token)
        if meta.lm_head_indices is not None:
            hidden = hidden[meta.lm_head_indices.long()]
        logits = self.hf.get_output_embeddings()(hidden)
        return logits, None


def supports(cfg_dict: dict) -> bool:
    """True when ``transformers`` has a causal-LM class for this config whose attention goes through the
    attention interface (checked on the class, without instantiating weights)."""
    try:
        from transformers import AutoConfig, AutoModelForCausalLM

        mt = cfg_dict.get("model_type")
        config = AutoConfig.for_model(mt)
        cls = AutoModelForCausalLM._model_mapping.get(type(config), None)
        if cls is None:
            return False
        return bool(getattr(cls, "_supports_attention_backend", False))
    except Exception:
        return False


def load_transformers_flash(path, cfg, process_group, rank, world, dtype, device, tokenizer, speculate,
                            kv_cache_dtype, max_prefill_tokens):
    """Build a ``FlashCausalLM`` around ``AutoModelForCausalLM`` with the paged attention function."""
    from transformers import AutoModelForCausalLM

    from . import resolve_kv_dtype
    from .flash_causal_lm import FlashCausalLM

    register()
    hf = AutoModelForCausalLM.from_pretrained(str(path), torch_dtype=dtype, attn_implementation=ATTN_NAME)
    info = {}
    if world > 1:
        # every rank reads the checkpoint on the host, keeps its slices of the planned layers and moves those to the
        # device; embeddings, norms and the output head stay replicated (every rank computes the same logits)
        info = shard_model(hf, rank, world, process_group)
    hf.to(device)
    model = TransformersDecoder(hf, device, dtype, world, info.get("heads_sharded", False), info.get("kv_sharded", False))
    kv_dtype = resolve_kv_dtype(kv_cache_dtype, dtype)
    if kv_dtype != dtype:
        raise NotImplementedError("the transformers backend keeps the KV cache in the model dtype")
    return FlashCausalLM(model, tokenizer, dtype, device, rank, world, int(speculate or 0), kv_dtype,
                         max_prefill_tokens)
