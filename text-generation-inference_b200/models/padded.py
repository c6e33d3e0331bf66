"""Fallback runners on top of Hugging Face ``transformers`` modules.

Covers what the reference serves through its non-flash paths: ``CausalLM`` (``causal_lm.py:38-891``,
``AutoModelForCausalLM`` with ``past_key_values``; Bloom, MPT, OPT, anything without a native
decoder), ``Seq2SeqLM`` (``seq2seq_lm.py``, T5-style encoder/decoder) and ``Mamba`` (``mamba.py``,
state-space models with a recurrent cache).  It is also the CPU path for architectures the native
decoder does not describe.

The reference pads all requests of a batch to a rectangle and has to slice and re-pad the key/value
tensors whenever requests join or leave.  Here every request owns its cache object and is stepped on
its own, so ``filter`` and ``concatenate`` are list operations and no padding is ever computed; the
logits of all requests are stacked for one vectorised sampling call.  These runners report
``requires_padding=True`` so the router budgets them by padded size, and they do not use the paged
KV cache, chunked prefill or prefix caching.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple, Type

import torch

from ..proto import generate_v3 as pb
from ..utils.tokens import NextTokenChooser, StoppingCriteria, batch_top_tokens
from .model import Model
from .types import Batch, GeneratedText, Generation, Tokens


@dataclass
class PaddedSeq:
    request: object
    ids: List[int]                      # decoder-side tokens: prompt + generated (causal), or decoder ids (seq2seq)
    prompt_len: int
    stopping: StoppingCriteria
    top_n: int
    prefix_offset: int
    read_offset: int
    cache: Any = None                   # past_key_values / cache_params of this request
    encoder_ids: Optional[List[int]] = None
    encoder_out: Any = None
    prefilled: bool = False
    finished: bool = False


class PaddedBatch(Batch):
    def __init__(self, batch_id: int, seqs: List[PaddedSeq], chooser: NextTokenChooser, device):
        self.batch_id, self.seqs, self.next_token_chooser, self.device = batch_id, seqs, chooser, device

    def __len__(self):
        return len(self.seqs)

    @property
    def requests(self):
        return [s.request for s in self.seqs]

    def to_pb(self):
        max_tokens = sum(len(s.ids) + s.stopping.max_new_tokens - s.stopping.current_tokens for s in self.seqs)
        return pb.CachedBatch(id=self.batch_id, request_ids=[s.request.id for s in self.seqs], size=len(self.seqs),
                              max_tokens=max_tokens, current_tokens=sum(len(s.ids) for s in self.seqs))

    seq2seq = False          # encoder/decoder batches start the decoder side from `decoder_start`
    decoder_start = 0

    @classmethod
    def from_pb(cls, batch_pb, tokenizer, dtype, device, speculate: int = 0) -> "PaddedBatch":
        from .flash_causal_lm import FlashCausalLMBatch

        seqs, params = [], []
        tokenized = FlashCausalLMBatch.batch_tokenized_inputs(batch_pb.requests, tokenizer)
        for r, ids in zip(batch_pb.requests, tokenized):
            stopping = StoppingCriteria.from_pb(r.stopping_parameters, tokenizer)
            if cls.seq2seq:
                seqs.append(PaddedSeq(r, [cls.decoder_start], 1, stopping, int(r.top_n_tokens), 0, 1, encoder_ids=ids))
            else:
                seqs.append(PaddedSeq(r, list(ids), len(ids), stopping, int(r.top_n_tokens),
                                      max(0, len(ids) - 5), len(ids)))
            params.append(r.parameters)
        return cls(batch_pb.id, seqs, NextTokenChooser.from_pb(params, device, tokenizer), device)

    def filter(self, request_ids: List[int]) -> Optional["PaddedBatch"]:
        if not request_ids:
            raise ValueError("Batch must have at least one request")
        index = {s.request.id: i for i, s in enumerate(self.seqs)}
        keep = [index[r] for r in request_ids]
        if len(keep) == len(self.seqs):
            return self
        return type(self)(self.batch_id, [self.seqs[i] for i in keep], self.next_token_chooser.select(keep), self.device)

    @classmethod
    def concatenate(cls, batches: List["PaddedBatch"]) -> "PaddedBatch":
        seqs = [s for b in batches for s in b.seqs]
        chooser = NextTokenChooser.concatenate([b.next_token_chooser for b in batches])
        return cls(batches[0].batch_id, seqs, chooser, batches[0].device)


class PaddedSeq2SeqBatch(PaddedBatch):
    seq2seq = True


# Galactica (an OPT checkpoint) tokenises the body of [START_DNA] / [START_SMILES] / [START_I_SMILES] / [START_AMINO]
# spans one character at a time: its tokenizer splits on a marker string that the serving side has to put in front of
# every character of the span and in front of the closing tag (reference: ``models/galactica.py:18-58``).
GALACTICA_SPLIT_MARKER = "SPL" + "1T-TH" + "1S-Pl3A5E"
_GALACTICA_SPAN = None


def galactica_mark_sequences(text: str) -> str:
    global _GALACTICA_SPAN
    if _GALACTICA_SPAN is None:
        import re

        _GALACTICA_SPAN = re.compile(r"\[START_(DNA|SMILES|I_SMILES|AMINO)\](.*?)\[END_\1\]", re.DOTALL)

    def mark(m):
        kind, body = m.group(1), m.group(2)
        spaced = "".join(GALACTICA_SPLIT_MARKER + ch for ch in body)
        return f"[START_{kind}]{spaced}{GALACTICA_SPLIT_MARKER}[END_{kind}]"

    return _GALACTICA_SPAN.sub(mark, text)


class GalacticaBatch(PaddedBatch):
    @classmethod
    def from_pb(cls, batch_pb, tokenizer, dtype, device, speculate: int = 0) -> "GalacticaBatch":
        seqs, params = [], []
        for r in batch_pb.requests:
            text = r.inputs
            if r.HasField("input_chunks") and len(r.input_chunks.chunks) > 0:
                text = "".join(c.text for c in r.input_chunks.chunks if c.WhichOneof("chunk") == "text")
            ids = list(tokenizer(galactica_mark_sequences(text), truncation=False,
                                 add_special_tokens=r.add_special_tokens)["input_ids"])
            if r.truncate and len(ids) > r.truncate:
                ids = ids[-r.truncate:]
            stopping = StoppingCriteria.from_pb(r.stopping_parameters, tokenizer)
            seqs.append(PaddedSeq(r, ids, len(ids), stopping, int(r.top_n_tokens), max(0, len(ids) - 5), len(ids)))
            params.append(r.parameters)
        return cls(batch_pb.id, seqs, NextTokenChooser.from_pb(params, device, tokenizer), device)


class PaddedCausalLM(Model):
    """``AutoModelForCausalLM``-style runner (also state-space models: the cache object is opaque)."""

    seq2seq = False

    def __init__(self, hf_model, tokenizer, dtype, device, rank: int = 0, world_size: int = 1, eos_token_ids=None):
        super().__init__(hf_model, tokenizer, requires_padding=True, dtype=dtype, device=device, rank=rank,
                         world_size=world_size, support_chunking=False, use_prefix_caching=False,
                         attention_impl="transformers")
        self.eos_token_ids = eos_token_ids
        self.hf = hf_model.eval()
        cfg = hf_model.config
        self.decoder_start = int(getattr(cfg, "decoder_start_token_id", None) or getattr(cfg, "pad_token_id", 0) or 0)
        self.kv_cache: list = []
        self.num_blocks = 0

    galactica = False        # set by the loader for facebook/galactica checkpoints

    @property
    def batch_type(self) -> Type[PaddedBatch]:
        if self.seq2seq:
            PaddedSeq2SeqBatch.decoder_start = self.decoder_start
            return PaddedSeq2SeqBatch
        return GalacticaBatch if self.galactica else PaddedBatch

    def init_kv_cache(self, num_blocks: int):      # interface parity with the paged runner
        self.num_blocks = num_blocks

    # ---- one model call for one request ---------------------------------------------------------
    @torch.no_grad()
    def _step(self, s: PaddedSeq) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Returns ``(last-position logits [V], all prompt logits or None)``."""
        dev = self.device
        if not s.prefilled:
            ids = torch.tensor([s.ids], dtype=torch.long, device=dev)
            out = self.hf(input_ids=ids, use_cache=True)
            s.prefilled = True
            prompt_logits = out.logits[0]
        else:
            ids = torch.tensor([[s.ids[-1]]], dtype=torch.long, device=dev)
            kw = {"cache_params": s.cache} if self._uses_cache_params else {"past_key_values": s.cache}
            if self._uses_cache_params:
                kw["cache_position"] = torch.tensor([len(s.ids) - 1], device=dev)
            out = self.hf(input_ids=ids, use_cache=True, **kw)
            prompt_logits = None
        s.cache = getattr(out, "cache_params", None) if self._uses_cache_params else out.past_key_values
        return out.logits[0, -1], prompt_logits

    @property
    def _uses_cache_params(self) -> bool:
        return getattr(self.hf.config, "model_type", "") in ("mamba", "mamba2", "falcon_mamba")

    # ---- engine step ----------------------------------------------------------------------------
    def generate_token(self, batch: PaddedBatch):
        start = time.time_ns()
        seqs = batch.seqs
        rows, prompt_rows = [], []
        for s in seqs:
            was_prefilled = s.prefilled
            last, prompt_logits = self._step(s)
            rows.append(last.float())
            prompt_rows.append(None if was_prefilled else prompt_logits)
        logits = torch.stack(rows)
        forward_ns = time.time_ns() - start
        dstart = time.time_ns()
        L = max(len(s.ids) for s in seqs)
        history = torch.zeros(len(seqs), L, dtype=torch.long, device=logits.device)
        for r, s in enumerate(seqs):
            history[r, :len(s.ids)] = torch.tensor(s.ids, dtype=torch.long)
        next_ids, next_lp, all_logprobs, _acc, _spec = batch.next_token_chooser(history, logits, 0, None, None)
        next_ids_l, next_lp_l = next_ids.tolist(), next_lp.tolist()
        want_top = any(s.top_n > 0 for s in seqs)
        top_ids = top_lps = None
        if want_top:
            top_ids, top_lps = batch_top_tokens([s.top_n for s in seqs], None, all_logprobs,
                                                torch.ones(len(seqs), dtype=torch.long))
        generations: List[Generation] = []
        for r, s in enumerate(seqs):
            tok, lp = next_ids_l[r], next_lp_l[r]
            first = prompt_rows[r] is not None
            s.ids.append(tok)
            text, s.prefix_offset, s.read_offset = self.decode_token(s.ids, s.prefix_offset, s.read_offset)
            batch.next_token_chooser.advance_grammar_single(r, tok)
            stop, reason = s.stopping(tok, text)
            s.finished = stop
            if s.request.id % self.world_size != self.rank:
                continue
            generated_text = None
            if stop:
                output_text, _, _ = self.decode_token(
                    s.ids, prefix_offset=len(s.ids) - s.stopping.current_tokens - 1,
                    read_offset=len(s.ids) - s.stopping.current_tokens, skip_special_tokens=True)
                seed = s.request.parameters.seed if batch.next_token_chooser.do_sample_list[r] else None
                generated_text = GeneratedText(output_text, s.stopping.current_tokens, reason, seed)
            prefill_tokens = None
            if first and s.request.prefill_logprobs and not self.seq2seq:
                lps = torch.log_softmax(prompt_rows[r].float(), -1)
                p_ids = s.ids[:s.prompt_len]
                tgt = torch.tensor(p_ids[1:], dtype=torch.long, device=lps.device)
                vals = [float("nan")] + lps[:-1].gather(1, tgt.view(-1, 1)).view(-1).tolist()
                p_texts = [self.tokenizer.decode([t], skip_special_tokens=False) for t in p_ids]
                prefill_tokens = Tokens(p_ids, vals, p_texts, [t in self.all_special_ids for t in p_ids])
            top_tokens = None
            if top_ids is not None and s.top_n > 0:
                top_tokens = [Tokens(ids_j, lps_j, [self.tokenizer.decode([t], skip_special_tokens=False) for t in ids_j],
                                     [t in self.all_special_ids for t in ids_j])
                              for ids_j, lps_j in zip(top_ids[r][:1], top_lps[r][:1])]
            generations.append(Generation(s.request.id, prefill_tokens,
                                          Tokens([tok], [lp], [text], [tok in self.all_special_ids]),
                                          generated_text, top_tokens))
        decode_ns = time.time_ns() - dstart
        if all(s.finished for s in seqs):
            return generations, None, (forward_ns, decode_ns)
        return generations, batch, (forward_ns, decode_ns)


class PaddedSeq2SeqLM(PaddedCausalLM):
    """Encoder/decoder models: the encoder runs once per request, the decoder steps with its cache."""

    seq2seq = True

    @torch.no_grad()
    def _step(self, s: PaddedSeq):
        dev = self.device
        if not s.prefilled:
            enc_ids = torch.tensor([s.encoder_ids], dtype=torch.long, device=dev)
            s.encoder_out = self.hf.get_encoder()(input_ids=enc_ids)
            s.prefilled = True
            dec = torch.tensor([s.ids], dtype=torch.long, device=dev)
            out = self.hf(encoder_outputs=s.encoder_out, decoder_input_ids=dec, use_cache=True)
        else:
            dec = torch.tensor([[s.ids[-1]]], dtype=torch.long, device=dev)
            out = self.hf(encoder_outputs=s.encoder_out, decoder_input_ids=dec, past_key_values=s.cache, use_cache=True)
        s.cache = out.past_key_values
        return out.logits[0, -1], out.logits[0] if len(s.ids) == 1 else None


# Tensor-parallel plans for model types whose transformers config carries none (module names inside the base model).
# The reference shards these families in its own modelling files (``custom_modeling/opt_modeling.py``,
# ``bloom_modeling.py``): column-parallel q / k / v and first MLP layer, row-parallel output projections.
PADDED_TP = {
    "opt": dict(plan={"decoder.layers.*.self_attn.q_proj": "colwise", "decoder.layers.*.self_attn.k_proj": "colwise",
                      "decoder.layers.*.self_attn.v_proj": "colwise", "decoder.layers.*.self_attn.out_proj": "rowwise",
                      "decoder.layers.*.fc1": "colwise", "decoder.layers.*.fc2": "rowwise"},
                alibi=False),
    # the fused query_key_value is laid out [head, (q, k, v), head_dim]: a contiguous slice of rows is a slice of heads
    "bloom": dict(plan={"h.*.self_attention.query_key_value": "colwise", "h.*.self_attention.dense": "rowwise",
                        "h.*.mlp.dense_h_to_4h": "colwise", "h.*.mlp.dense_4h_to_h": "rowwise"},
                  alibi=True),
}


def _slice_alibi(module, rank: int, world: int):
    """Bloom builds the ALiBi bias for all heads ``[batch * heads, 1, kv]`` outside the attention module; a sharded
    attention module keeps the rows of its own heads."""

    def cut(alibi, batch):
        total = alibi.shape[0] // batch
        per = total // world
        return alibi.view(batch, total, *alibi.shape[1:])[:, rank * per:(rank + 1) * per].reshape(
            batch * per, *alibi.shape[1:])

    def hook(mod, args, kwargs):
        batch = (args[0] if args else kwargs["hidden_states"]).shape[0]
        if "alibi" in kwargs:
            kwargs["alibi"] = cut(kwargs["alibi"], batch)
        elif len(args) > 2:
            args = args[:2] + (cut(args[2], batch),) + args[3:]
        return args, kwargs

    module.register_forward_pre_hook(hook, with_kwargs=True)


def shard_padded(model, model_type: str, rank: int, world: int, group) -> None:
    from .transformers_backend import ShardedLinear, shard_model

    spec = PADDED_TP.get(model_type)
    cfg = model.config
    if spec is None and not getattr(cfg, "base_model_tp_plan", None):
        raise NotImplementedError(f"the fallback runner has no tensor-parallel plan for model type {model_type!r}: "
                                  "run it on one GPU")
    shard_model(model, rank, world, group, plan=spec["plan"] if spec else None, head_attrs=("num_heads",))
    if spec and spec["alibi"]:
        for m in model.modules():
            if isinstance(getattr(m, "query_key_value", None), ShardedLinear):
                _slice_alibi(m, rank, world)


def load_padded(path, cfg, process_group, rank: int, world: int, dtype, device, tokenizer):
    """Instantiate the ``transformers`` implementation of ``path`` and wrap it in a fallback runner."""
    import transformers

    hf_cfg = transformers.AutoConfig.from_pretrained(str(path))
    seq2seq = bool(getattr(hf_cfg, "is_encoder_decoder", False))
    cls = transformers.AutoModelForSeq2SeqLM if seq2seq else transformers.AutoModelForCausalLM
    model = cls.from_pretrained(str(path), torch_dtype=dtype)
    if world > 1:
        if seq2seq:
            raise NotImplementedError("the encoder-decoder fallback runner is not sharded: run it on one GPU")
        shard_padded(model, str(hf_cfg.model_type), rank, world, process_group)
    model = model.to(device)
    if not hasattr(tokenizer, "decode"):
        tokenizer = transformers.AutoTokenizer.from_pretrained(str(path))
    eos = getattr(hf_cfg, "eos_token_id", None)
    eos_ids = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else None)
    runner_cls = PaddedSeq2SeqLM if seq2seq else PaddedCausalLM
    runner = runner_cls(model, tokenizer, dtype, device, rank, world, eos_ids)
    # the reference recognises Galactica by its repository name (``models/__init__.py:742-760``); a local directory
    # is recognised by its name or by the `_name_or_path` the checkpoint's config recorded
    names = (str(path) + " " + str(getattr(hf_cfg, "_name_or_path", ""))).lower()
    if not seq2seq and hf_cfg.model_type == "opt" and "galactica" in names:
        runner.galactica = True
    return runner
