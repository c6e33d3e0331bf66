"""Paged-KV model runner: ragged batch state, chunked prefill, decode, sampling, stop handling.

Reference behaviour covered: ``models/flash_causal_lm.py`` — ``FlashCausalLMBatch`` (``:125-1175``:
``from_pb``/``from_tokenized``, ``filter``, ``concatenate``, ``prepare_for_prefill``) and
``FlashCausalLM`` (``:1193-2478``: ``init_kv_cache``, ``warmup``, ``cuda_graph_warmup``, ``forward``,
``generate_token``).

Design differences:

* One code path for prefill, chunked prefill, decode and speculative verification: every step is a
  ragged batch where sequence ``i`` contributes ``n_i >= 0`` query tokens on top of ``cache_len_i``
  cached tokens.  Prefix-cache hits (``Request.cache_len``) and continuation chunks are the same case.
* Per-sequence state is a small host object (``Seq``); the per-step device metadata (ids, positions,
  slots, block tables, lengths, logit rows) is packed into ONE pinned int32 staging buffer and shipped
  with ONE host-to-device copy.  Decode steps replay a CUDA graph per batch-size bucket that reads
  those static buffers (``models/graphs.py``).
* Results come back with ONE device-to-host copy (ids + logprobs packed in one tensor).
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple, Type

import numpy as np
import torch

from ..proto import generate_v3 as pb
from ..utils.tokens import NextTokenChooser, StoppingCriteria, batch_top_tokens
from .decoder import CausalDecoder, ForwardMeta
from .model import Model
from .types import Batch, GeneratedText, Generation, Tokens

BLOCK_SIZE = int(os.environ.get("TGI_B200_BLOCK_SIZE", "16"))
WIGGLE_ROOM = float(os.environ.get("TGI_WIGGLE_ROOM", "0.90"))
# set by the launcher (reference: models/globals.py:8-20): whether the router may re-use cached prompt prefixes
# and split long prompts into chunks
PREFIX_CACHING = os.environ.get("PREFIX_CACHING", "1").lower() in ("1", "true")
PREFILL_CHUNKING = os.environ.get("PREFILL_CHUNKING", "1").lower() in ("1", "true")


@dataclass
class Seq:
    """Host-side state of one request inside a batch."""

    request: object                      # pb.Request
    ids: List[int]                       # prompt + generated tokens
    prompt_len: int
    cache_len: int                       # tokens whose KV is already in the cache
    blocks: List[int]
    slots: np.ndarray                    # slot of every position this request may ever use
    stopping: StoppingCriteria
    top_n: int
    prefix_offset: int
    read_offset: int
    first_chunk: Optional[int] = None    # router-imposed length of the first prefill chunk
    prefilling: bool = True
    speculative_ids: List[int] = field(default_factory=list)
    prefill_ids: List[int] = field(default_factory=list)
    prefill_logprobs: List[float] = field(default_factory=list)
    adapter_index: int = 0
    finished: bool = False

    @property
    def want_prefill_logprobs(self) -> bool:
        return bool(self.request.prefill_logprobs)


def _adapter_index(request) -> int:
    """Index of the LoRA adapter a request asks for (0: base model or unknown adapter)."""
    if not request.HasField("adapter_id") or not request.adapter_id:
        return 0
    from ..utils.adapter import ADAPTER_TO_INDEX

    return ADAPTER_TO_INDEX.get(request.adapter_id, 0)


class FlashCausalLMBatch(Batch):
    def __init__(self, batch_id: int, seqs: List[Seq], chooser: NextTokenChooser, device, speculate: int = 0):
        self.batch_id = batch_id
        self.seqs = seqs
        self.next_token_chooser = chooser
        self.device = device
        self.speculate = speculate
        self.max_prefill_tokens: Optional[int] = None
        self.history = None          # TokenHistory, created by the first step that needs the ids on the device
        self._reindex()

    def _reindex(self):
        self.requests_idx_mapping = {s.request.id: i for i, s in enumerate(self.seqs)}

    def __len__(self):
        return len(self.seqs)

    @property
    def requests(self):
        return [s.request for s in self.seqs]

    @property
    def num_blocks(self) -> int:
        return sum(len(s.blocks) for s in self.seqs)

    @property
    def prefilling(self) -> bool:
        return any(s.prefilling for s in self.seqs)

    # -- planning --------------------------------------------------------------------------------
    def plan_step(self, max_prefill_tokens: Optional[int] = None) -> List[int]:
        """Number of query tokens each sequence contributes to the next forward pass."""
        budget = max_prefill_tokens if max_prefill_tokens is not None else self.max_prefill_tokens
        counts = []
        # decode rows are always served; what is left of the budget goes to prefill chunks, oldest first
        used = sum(1 + len(s.speculative_ids) for s in self.seqs if not s.prefilling)
        for s in self.seqs:
            if not s.prefilling:
                counts.append(1 + len(s.speculative_ids))
                continue
            remaining = s.prompt_len - s.cache_len
            if s.first_chunk is not None:
                n = min(s.first_chunk, remaining)
            elif budget is None:
                n = remaining
            else:
                n = max(0, min(remaining, budget - used))
            used += n
            counts.append(n)
        return counts

    def to_pb(self):
        return pb.CachedBatch(
            id=self.batch_id,
            request_ids=[s.request.id for s in self.seqs],
            size=len(self.seqs),
            max_tokens=self.num_blocks * BLOCK_SIZE,
            current_tokens=sum(self.plan_step()),
        )

    # -- construction ----------------------------------------------------------------------------
    @classmethod
    def batch_tokenized_inputs(cls, requests, tokenizer) -> List[List[int]]:
        out = []
        for r in requests:
            text = r.inputs
            if r.HasField("input_chunks") and len(r.input_chunks.chunks) > 0:
                parts = []
                for c in r.input_chunks.chunks:
                    if c.WhichOneof("chunk") == "text":
                        parts.append(c.text)
                    else:
                        raise ValueError("image chunks need a vision-language runner")
                text = "".join(parts)
            ids = tokenizer(text, truncation=False, add_special_tokens=r.add_special_tokens)["input_ids"]
            if r.truncate and len(ids) > r.truncate:
                ids = ids[-r.truncate:]
            out.append(list(ids))
        return out

    @classmethod
    def from_pb(cls, batch_pb, tokenizer, dtype, device, speculate: int = 0) -> "FlashCausalLMBatch":
        return cls.from_tokenized(batch_pb, cls.batch_tokenized_inputs(batch_pb.requests, tokenizer),
                                  tokenizer, dtype, device, speculate)

    @classmethod
    def from_tokenized(cls, batch_pb, batch_tokenized_inputs: List[List[int]], tokenizer, dtype, device,
                       speculate: int = 0) -> "FlashCausalLMBatch":
        seqs: List[Seq] = []
        params = []
        block_cursor = 0
        for r, ids in zip(batch_pb.requests, batch_tokenized_inputs):
            prompt_len = len(ids)
            stopping = StoppingCriteria.from_pb(r.stopping_parameters, tokenizer)
            max_new = stopping.max_new_tokens
            needed_tokens = prompt_len + max_new + speculate
            if len(r.blocks) > 0:
                blocks = list(r.blocks)
                slots = np.asarray(r.slots, dtype=np.int32) if len(r.slots) else None
            else:
                # No allocation from the router (warmup, benchmarks): take consecutive blocks.
                nb = math.ceil(needed_tokens / BLOCK_SIZE)
                blocks = list(range(block_cursor, block_cursor + nb))
                block_cursor += nb
                slots = None
            if slots is None or slots.size == 0:
                b = np.asarray(blocks, dtype=np.int32)
                slots = (b[:, None] * BLOCK_SIZE + np.arange(BLOCK_SIZE, dtype=np.int32)[None, :]).reshape(-1)
            cache_len = int(r.cache_len)
            if cache_len >= prompt_len:
                # A fully cached prompt still needs its last token recomputed to produce logits.
                cache_len = prompt_len - 1
            first_chunk = int(r.chunk_len) if r.HasField("chunk_len") else None
            seqs.append(Seq(
                request=r, ids=list(ids), prompt_len=prompt_len, cache_len=cache_len, blocks=blocks, slots=slots,
                stopping=stopping, top_n=int(r.top_n_tokens), prefix_offset=max(0, prompt_len - 5),
                read_offset=prompt_len, first_chunk=first_chunk,
                adapter_index=_adapter_index(r),
            ))
            params.append(r.parameters)
        chooser = NextTokenChooser.from_pb(params, device, tokenizer)
        return cls(batch_pb.id, seqs, chooser, device, speculate)

    # -- batch surgery ---------------------------------------------------------------------------
    def filter(self, request_ids: List[int]) -> "FlashCausalLMBatch":
        if len(request_ids) == 0:
            raise ValueError("Batch must have at least one request")
        if len(request_ids) == len(self.seqs) and all(
            s.request.id == rid for s, rid in zip(self.seqs, request_ids)
        ):
            return self
        indices = [self.requests_idx_mapping[rid] for rid in request_ids]
        self.seqs = [self.seqs[i] for i in indices]
        self.next_token_chooser = self.next_token_chooser.filter(indices)
        self._reindex()
        return self

    @classmethod
    def concatenate(cls, batches: List["FlashCausalLMBatch"]) -> "FlashCausalLMBatch":
        seqs = [s for b in batches for s in b.seqs]
        chooser = NextTokenChooser.concatenate([b.next_token_chooser for b in batches])
        out = cls(batches[0].batch_id, seqs, chooser, batches[0].device, batches[0].speculate)
        budgets = [b.max_prefill_tokens for b in batches if b.max_prefill_tokens is not None]
        out.max_prefill_tokens = min(budgets) if budgets else None
        # rows are keyed by request id: the largest batch's device history stays valid, newcomers are uploaded
        with_hist = [b for b in batches if b.history is not None]
        if with_hist:
            out.history = max(with_hist, key=len).history
        return out

    def device_history(self, active: List[int]) -> torch.Tensor:
        """``[len(active), L]`` matrix of the ids of the rows ``active`` on the device (zero padded)."""
        from ..utils.history import TokenHistory

        if self.history is None:
            self.history = TokenHistory(self.device, rows=max(64, len(self.seqs)))
        self.history.retain(s.request.id for s in self.seqs)
        return self.history.sync([self.seqs[i].request.id for i in active], [self.seqs[i].ids for i in active])


class StepStaging:
    """Pinned host buffer + device mirror for the per-step int32 metadata (one H2D copy per step)."""

    def __init__(self, device: torch.device, capacity: int = 1 << 16):
        self.device = device
        self.capacity = 0
        self.host = None
        self.dev = None
        self._grow(capacity)

    def _grow(self, n: int):
        self.capacity = int(n)
        pin = self.device.type == "cuda"
        self.host = torch.empty(self.capacity, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)

    def upload(self, arrays: List[np.ndarray]) -> List[torch.Tensor]:
        """Copy the arrays back to back (each start aligned to 4 ints = 16 bytes) and return device views."""
        offs, total = [], 0
        for a in arrays:
            offs.append(total)
            total += (a.size + 3) & ~3
        if total > self.capacity:
            self._grow(max(total, self.capacity * 2))
        for a, o in zip(arrays, offs):
            self.host_np[o:o + a.size] = a.reshape(-1)
        if self.device.type == "cuda":
            self.dev[:total].copy_(self.host[:total], non_blocking=True)
        else:
            self.dev[:total] = self.host[:total]
        return [self.dev[o:o + a.size].view(a.shape) for a, o in zip(arrays, offs)]


class FlashCausalLM(Model):
    """Runs a ``CausalDecoder`` over paged KV."""

    def __init__(self, model: CausalDecoder, tokenizer, dtype, device, rank: int = 0, world_size: int = 1,
                 speculate: int = 0, kv_cache_dtype: Optional[torch.dtype] = None,
                 max_prefill_tokens: Optional[int] = None, eos_token_ids=None):
        windows = [w for w in model.dims.windows if w > 0]
        super().__init__(model, tokenizer, requires_padding=False, dtype=dtype, device=device, rank=rank,
                         world_size=world_size, sliding_window=(windows[0] if windows else None),
                         speculate=speculate, support_chunking=PREFILL_CHUNKING, use_prefix_caching=PREFIX_CACHING,
                         block_size=BLOCK_SIZE)
        self.dims = model.dims
        self.kv_cache_dtype = kv_cache_dtype or dtype
        self.kv_cache: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.num_blocks = 0
        self.max_prefill_tokens = max_prefill_tokens
        self.staging = StepStaging(device)
        self.graphs = None
        # (signature, graphs object, (logits, row_owner)) of a decode replay that was put on the stream at the end
        # of the previous step, before its text post-processing (see `_prelaunch_next_decode`)
        self._prelaunched = None
        self.overlap_hits = 0          # steps that found their replay already on the stream
        self.overlap_decode = os.environ.get("TGI_B200_OVERLAP_DECODE", "1") == "1"
        self.eos_token_ids = eos_token_ids
        if eos_token_ids is not None and tokenizer is not None:
            try:
                tokenizer._eos_token_ids = set(eos_token_ids)
            except Exception:
                pass

    @property
    def batch_type(self) -> Type[FlashCausalLMBatch]:
        return FlashCausalLMBatch

    # -- KV cache --------------------------------------------------------------------------------
    def kv_bytes_per_block(self) -> int:
        d = self.dims
        item = torch.empty((), dtype=self.kv_cache_dtype).element_size()
        return 2 * d.num_layers * BLOCK_SIZE * d.num_kv_heads * (d.attn_head_dim or d.head_dim) * item

    def graph_eligible(self, batch) -> bool:
        """Runners whose step cannot be replayed for some batches (per-sequence side inputs) say so here."""
        return True

    def _sample_on_shards(self, chooser, seqs, active, sample_rows, batch):
        """Vocabulary-parallel sampling after a decode graph that left only this rank's logit slice: returns
        ``(ids, logprobs)`` on the device, or ``None`` when a stage needs the whole distribution on one rank
        (top-n tokens, typical-p, watermark, grammar, speculation) and the logits have to be gathered."""
        b, n = self.graphs.last
        comm = getattr(self.model, "comm", None)
        if (comm is None or b.local_logits is None or batch.speculate != 0 or chooser.any_typical or chooser.watermarks
                or chooser.grammar is not None or any(seqs[i].top_n > 0 for i in active)
                or len(active) != n or sample_rows != list(range(n))):
            return None
        from ..ops import cuda as K

        d = self.model.dims
        local = b.local_logits[:n]
        v0 = self.model.head.vocab_start
        scale = float(d.logit_scale)
        if chooser.any_rep or chooser.any_freq:
            local = K.penalties(local, batch.device_history(active), chooser.repetition_penalty if chooser.any_rep else None,
                                chooser.frequency_penalty if chooser.any_freq else None, v0, scale)
            scale = 1.0
        seeds = steps = do_sample = None
        if chooser.any_sample:
            do_sample = chooser.do_sample.to(torch.uint8)
            seeds = torch.tensor([int(s or 0) & 0x7FFFFFFFFFFFFFFF for s in chooser.seeds], dtype=torch.int64)
            steps = torch.tensor(chooser.steps, dtype=torch.int32)
            chooser.steps = [st + (1 if ds else 0) for st, ds in zip(chooser.steps, chooser.do_sample_list)]
        return comm.sample(local, v0, d.vocab, scale,
                           chooser.temperature if chooser.any_temperature else None,
                           chooser.top_k if chooser.any_top_k else None, chooser.top_p if chooser.any_top_p else None,
                           do_sample, seeds, steps)

    def init_kv_cache(self, num_blocks: int):
        d = self.dims
        self.kv_cache = []
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        self.num_blocks = int(num_blocks)
        for _ in range(d.num_layers):
            k = torch.zeros(num_blocks, BLOCK_SIZE, d.num_kv_heads, d.attn_head_dim or d.head_dim,
                            dtype=self.kv_cache_dtype, device=self.device)
            v = torch.zeros_like(k)
            self.kv_cache.append((k, v))

    def warmup(self, batch: FlashCausalLMBatch, max_input_tokens: Optional[int], max_total_tokens: Optional[int]):
        """Size the KV cache from free device memory after a worst-case prefill, then capture decode graphs.

        Returns ``(max_supported_total_tokens, max_input_tokens, max_total_tokens)``.
        """
        batch_blocks = batch.num_blocks
        self.init_kv_cache(max(batch_blocks, 1))
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.generate_token(batch)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            free, total = torch.cuda.mem_get_info(self.device)
            frac = float(os.environ.get("CUDA_MEMORY_FRACTION", "1.0"))
            usable = max(0, free - int((1 - frac) * total))
            num_blocks = int(usable * WIGGLE_ROOM) // self.kv_bytes_per_block() + batch_blocks
        else:
            num_blocks = max(batch_blocks, int(os.environ.get("TGI_B200_CPU_KV_BLOCKS", "4096")))
        if max_total_tokens is not None:
            # no point holding more KV than one maximal batch can use when the operator capped it
            pass
        self.init_kv_cache(num_blocks)
        cap = num_blocks * BLOCK_SIZE
        if max_total_tokens is None:
            mp = self.dims.max_positions
            max_total_tokens = min(cap, mp) if mp else cap
        if max_input_tokens is None:
            max_input_tokens = max_total_tokens - 1
        if self.device.type == "cuda" and os.environ.get("CUDA_GRAPHS", "") != "0":
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self, max_total_tokens)
            self.graphs.capture_all()
        return cap, max_input_tokens, max_total_tokens

    # -- forward ---------------------------------------------------------------------------------
    def build_meta(self, batch: FlashCausalLMBatch, counts: List[int]):
        """Pack the step's metadata; returns ``(ForwardMeta, row bookkeeping)``."""
        seqs = batch.seqs
        B = len(seqs)
        T = sum(counts)
        input_ids = np.empty(T, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        slots = np.empty(T, dtype=np.int32)
        cu = np.zeros(B + 1, dtype=np.int32)
        kv_lens = np.empty(B, dtype=np.int32)
        max_blocks = max(1, max(len(s.blocks) for s in seqs))
        tables = np.zeros((B, max_blocks), dtype=np.int32)
        head_rows: List[int] = []       # rows of the hidden state that need logits
        row_owner: List[Tuple[int, int]] = []  # (seq index, offset inside the chunk) per logits row
        t = 0
        for i, (s, n) in enumerate(zip(seqs, counts)):
            start = s.cache_len
            if s.prefilling:
                toks = s.ids[start:start + n]
            else:
                toks = [s.ids[-1]] + s.speculative_ids
                start = len(s.ids) - 1
            input_ids[t:t + n] = toks
            # `pos_delta`: offset between rotary position and token index after a prompt with images (Qwen2-VL)
            pos0 = start if s.prefilling else start + getattr(s, "pos_delta", 0)
            positions[t:t + n] = np.arange(pos0, pos0 + n, dtype=np.int32)
            slots[t:t + n] = s.slots[start:start + n]
            cu[i + 1] = t + n
            kv_lens[i] = start + n
            tables[i, :len(s.blocks)] = s.blocks
            if n > 0:
                finishing = s.prefilling and (start + n == s.prompt_len)
                if s.prefilling and s.want_prefill_logprobs:
                    head_rows.extend(range(t, t + n))
                    row_owner.extend((i, j) for j in range(n))
                elif finishing:
                    head_rows.append(t + n - 1)
                    row_owner.append((i, n - 1))
                elif not s.prefilling:
                    head_rows.extend(range(t, t + n))
                    row_owner.extend((i, j) for j in range(n))
            t += n
        head = np.asarray(head_rows, dtype=np.int32)
        dev = self.staging.upload([input_ids, positions, slots, cu, kv_lens, tables, head])
        meta = ForwardMeta(
            input_ids=dev[0], positions=dev[1], slots=dev[2], cu_seqlens_q=dev[3], kv_lens=dev[4],
            block_tables=dev[5], max_q=max(counts) if counts else 0, max_kv=int(kv_lens.max()) if B else 0,
            lm_head_indices=dev[6] if len(head_rows) != T else None,
        )
        lora = getattr(self, "lora", None)
        if lora is not None and any(s.adapter_index > 0 for s in seqs):
            token_adapter = np.repeat(np.asarray([s.adapter_index for s in seqs], dtype=np.int64),
                                      np.asarray(counts, dtype=np.int64))
            meta.adapter_data = lora.batch_data(token_adapter, self.device)
        return meta, row_owner

    @staticmethod
    def _decode_signature(seqs) -> tuple:
        """Identity of a decode step: which sequences (the objects themselves: holding them keeps their identity
        from being recycled by a later batch), and how long each is."""
        return tuple(seqs), tuple(len(s.ids) for s in seqs)

    @staticmethod
    def _same_step(sig: tuple, seqs) -> bool:
        held, lens = sig
        return (len(held) == len(seqs) and all(a is b for a, b in zip(held, seqs))
                and all(n == len(s.ids) for n, s in zip(lens, seqs)))

    @staticmethod
    def _nobody_finishes(seqs, next_ids) -> bool:
        """True when no sequence can stop on the token it just received: decided without detokenising
        (length and EOS checks); a sequence with stop strings always counts as "might stop"."""
        for s, tok in zip(seqs, next_ids):
            st = s.stopping
            if st.stop_sequence_criterias or st.current_tokens + 1 >= st.max_new_tokens:
                return False
            if not st.ignore_eos_token and tok in st.eos_token_ids:
                return False
            if len(s.ids) + 1 >= len(s.slots):      # the next step would need a slot past the allocation
                return False
        return True

    def forward(self, meta: ForwardMeta) -> torch.Tensor:
        logits, spec = self.model.forward(meta, self.kv_cache)
        self.last_speculative_logits = spec     # [rows, n_heads, V] when a speculator head is attached
        return logits

    # -- one engine step -------------------------------------------------------------------------
    def generate_token(self, batch: FlashCausalLMBatch):
        start_ns = time.time_ns()
        if not self.kv_cache:
            self.init_kv_cache(max(batch.num_blocks, max((max(s.blocks) for s in batch.seqs), default=0) + 1))
        if batch.max_prefill_tokens is None:
            batch.max_prefill_tokens = self.max_prefill_tokens
        seqs = batch.seqs
        counts = batch.plan_step()
        B = len(seqs)

        use_graph = (self.graphs is not None and not batch.prefilling and batch.speculate == 0
                     and self.graphs.supports(batch) and self.graph_eligible(batch)
                     # adapters ride the graphs through the LoRA kernels on one GPU; with tensor parallelism
                     # the row-parallel targets need a collective between the two kernels and stay eager
                     and not (getattr(self, "lora", None) is not None and self.world_size > 1
                              and any(s.adapter_index > 0 for s in seqs)))
        pre, self._prelaunched = self._prelaunched, None
        if use_graph:
            if (pre is not None and pre[1] is self.graphs and self._same_step(pre[0], seqs)
                    and all(c == 1 for c in counts)):
                logits, row_owner = pre[2]          # this step's replay is already on the stream
                self.overlap_hits += 1
            else:
                logits, row_owner = self.graphs.run(batch, counts)
        else:
            meta, row_owner = self.build_meta(batch, counts)
            logits = self.forward(meta) if row_owner or any(counts) else None
        forward_ns = time.time_ns() - start_ns
        decode_start = time.time_ns()

        # rows by owner
        rows_of: Dict[int, List[int]] = {}
        for r, (i, j) in enumerate(row_owner):
            rows_of.setdefault(i, []).append(r)

        # --- prefill logprobs -------------------------------------------------------------------
        all_lp_cache = None
        for i, s in enumerate(seqs):
            if s.prefilling and s.want_prefill_logprobs and counts[i] > 0:
                if all_lp_cache is None:
                    all_lp_cache = torch.log_softmax(logits.float(), dim=-1)
                rows = rows_of[i]
                start = s.cache_len
                n = counts[i]
                # row j predicts the prompt token at position start+j+1 (the last row of the last
                # chunk predicts the first generated token and is handled by the sampler)
                targets = s.ids[start + 1:start + n + 1][: n if start + n < s.prompt_len else n - 1]
                if targets:
                    tgt = torch.tensor(targets, dtype=torch.long, device=logits.device)
                    lp = all_lp_cache[rows[:len(targets)]].gather(1, tgt.view(-1, 1)).view(-1).tolist()
                    s.prefill_logprobs.extend(lp)
                    s.prefill_ids.extend(targets)

        # --- which sequences emit a token this step ---------------------------------------------
        active: List[int] = []
        sample_rows: List[int] = []
        S = 1 + batch.speculate if (batch.speculate and not batch.prefilling) else 1
        for i, s in enumerate(seqs):
            n = counts[i]
            if n == 0:
                continue
            if s.prefilling:
                if s.cache_len + n == s.prompt_len:
                    active.append(i)
                    sample_rows.append(rows_of[i][-1])
            else:
                active.append(i)
                sample_rows.extend(rows_of[i])

        generations: List[Generation] = []
        next_ids_l: List[int] = []
        if active:
            chooser = batch.next_token_chooser if len(active) == B else batch.next_token_chooser.select(active)
            greedy_dev = None
            if logits is None:
                # the decode graph ended in the vocabulary-parallel argmax: full logits exist only if gathered
                plain = (chooser.is_greedy_plain and batch.speculate == 0
                         and not any(seqs[i].top_n > 0 for i in active))
                if plain:
                    greedy_dev = self.graphs.greedy()
                if greedy_dev is None:
                    # samplers made of temperature / top-k / top-p / penalties run on the vocabulary shards
                    greedy_dev = self._sample_on_shards(chooser, seqs, active, sample_rows, batch)
                if greedy_dev is None:
                    logits = self.graphs.gather_last_logits()
            # sequences in the same step may carry different numbers of speculative tokens only when
            # some have none yet (first decode after prefill): pad those with a token that cannot match
            spec_lens = [0 if seqs[i].prefilling else len(seqs[i].speculative_ids) for i in active]
            Smax = 1 + max(spec_lens)
            if greedy_dev is not None:
                sel_rows, sel, speculated = sample_rows, None, None
            elif all(l == spec_lens[0] for l in spec_lens):
                sel_rows = sample_rows
                sel = logits if len(sample_rows) == logits.shape[0] else logits[
                    torch.tensor(sample_rows, dtype=torch.long, device=logits.device)]
                speculated = None
                if Smax > 1:
                    speculated = torch.tensor([seqs[i].speculative_ids for i in active], dtype=torch.long,
                                              device=logits.device)
            else:
                # ragged: expand every sequence to Smax rows by repeating its last row
                idx, spec = [], []
                for i, l in zip(active, spec_lens):
                    rows = rows_of[i][-(l + 1):] if not seqs[i].prefilling else [rows_of[i][-1]]
                    idx.extend(rows + [rows[-1]] * (Smax - len(rows)))
                    spec.append((seqs[i].speculative_ids if not seqs[i].prefilling else []) + [-1] * (Smax - 1 - l))
                sel_rows = idx
                sel = logits[torch.tensor(idx, dtype=torch.long, device=logits.device)]
                speculated = torch.tensor(spec, dtype=torch.long, device=logits.device)
            need_history = (chooser.any_rep or chooser.any_freq or bool(chooser.watermarks) or batch.speculate > 0)
            if greedy_dev is not None:
                history = None
            elif need_history:
                history = batch.device_history(active)
            else:
                history = torch.zeros(len(active), 1, dtype=torch.long, device=logits.device)
            want_top = any(seqs[i].top_n > 0 for i in active)
            if greedy_dev is not None or (chooser.is_greedy_plain and batch.speculate == 0 and not want_top
                                          and speculated is None):
                from .. import ops

                ids_t, lp_t = greedy_dev if greedy_dev is not None else ops.argmax_logprob(sel)
                packed = torch.stack([ids_t.float(), lp_t.float()]).cpu()
                next_ids_l = [int(x) for x in packed[0].tolist()]
                next_lp_l = packed[1].tolist()
                accepted_l = [1] * len(active)
                spec_next = None
                all_logprobs = None
            else:
                spec_scores = getattr(self, "last_speculative_logits", None)
                if spec_scores is not None and not use_graph:
                    spec_scores = spec_scores[torch.tensor(sel_rows, dtype=torch.long, device=logits.device)]
                    spec_scores = spec_scores[:, : batch.speculate]
                else:
                    spec_scores = None
                next_ids, next_lp, all_logprobs, accepted, spec_next = chooser(
                    history, sel, batch.speculate, speculated, spec_scores, need_logprobs=want_top)
                next_ids_l = next_ids.tolist()
                next_lp_l = next_lp.tolist()
                accepted_l = accepted.tolist()
                if spec_next is not None:
                    spec_next = spec_next.tolist()
            top_ids = top_lps = None
            if want_top and all_logprobs is not None:
                # all_logprobs has one row per candidate position; keep the accepted ones
                keep = []
                Srow = all_logprobs.shape[0] // len(active)
                for r, a in enumerate(accepted_l):
                    keep.extend(range(r * Srow, r * Srow + a))
                lp_rows = all_logprobs[torch.tensor(keep, dtype=torch.long, device=all_logprobs.device)]
                top_ids, top_lps = batch_top_tokens(
                    [seqs[i].top_n for i in active], None, lp_rows,
                    torch.tensor(accepted_l, dtype=torch.long))

            # Overlap: when this was a plain graph decode step and no sequence can finish on it (checked on
            # token ids alone), the next step's replay goes on the stream now, and the detokenisation /
            # stop-sequence / response building below runs while the GPU computes it.
            appended = False
            if (use_graph and self.overlap_decode and batch.speculate == 0 and len(active) == B
                    and all(a == 1 for a in accepted_l) and self._nobody_finishes(seqs, next_ids_l)):
                for s, tok in zip(seqs, next_ids_l):
                    s.ids.append(tok)
                appended = True
                if self.graphs.supports(batch):
                    out = self.graphs.advance(seqs, next_ids_l)     # same bucket as the step that just ran
                    self._prelaunched = (self._decode_signature(seqs), self.graphs, out)
            cursor = 0
            for r, i in enumerate(active):
                s = seqs[i]
                a = accepted_l[r]
                new_ids = next_ids_l[cursor:cursor + a]
                new_lps = next_lp_l[cursor:cursor + a]
                cursor += a
                was_prefilling = s.prefilling
                if was_prefilling:
                    s.cache_len += counts[i]
                    s.prefilling = False
                    s.first_chunk = None
                texts, specials, kept_ids, kept_lps = [], [], [], []
                stop, reason = False, None
                for tok, lp in zip(new_ids, new_lps):
                    if not appended:
                        s.ids.append(tok)
                    text, s.prefix_offset, s.read_offset = self.decode_token(s.ids, s.prefix_offset, s.read_offset)
                    kept_ids.append(tok)
                    kept_lps.append(lp)
                    texts.append(text)
                    specials.append(tok in self.all_special_ids)
                    batch.next_token_chooser.advance_grammar_single(i, tok)
                    stop, reason = s.stopping(tok, text)
                    if stop:
                        break
                if not was_prefilling:
                    # KV of the accepted tokens' predecessors is now valid
                    s.cache_len = len(s.ids) - 1
                else:
                    s.cache_len = len(s.ids) - 1
                s.speculative_ids = [] if spec_next is None or stop else list(spec_next[r])
                s.finished = stop
                if s.request.id % self.world_size != self.rank:
                    continue
                generated_text = None
                if stop:
                    out_ids = s.ids[s.prompt_len:]
                    output_text, _, _ = self.decode_token(
                        s.ids, prefix_offset=len(s.ids) - s.stopping.current_tokens - 1,
                        read_offset=len(s.ids) - s.stopping.current_tokens, skip_special_tokens=True)
                    seed = s.request.parameters.seed if batch.next_token_chooser.do_sample_list[i] else None
                    generated_text = GeneratedText(output_text, s.stopping.current_tokens, reason, seed)
                prefill_tokens = None
                if was_prefilling and s.want_prefill_logprobs:
                    p_ids = [s.ids[0]] + s.prefill_ids if s.request.cache_len == 0 else s.prefill_ids
                    p_lps = [float("nan")] + s.prefill_logprobs if s.request.cache_len == 0 else s.prefill_logprobs
                    p_texts = [self.tokenizer.decode([t], skip_special_tokens=False) for t in p_ids]
                    prefill_tokens = Tokens(p_ids, p_lps, p_texts, [t in self.all_special_ids for t in p_ids])
                top_tokens = None
                if top_ids is not None and s.top_n > 0:
                    top_tokens = []
                    for ids_j, lps_j in zip(top_ids[r][:len(kept_ids)], top_lps[r][:len(kept_ids)]):
                        toptexts = [self.tokenizer.decode([t], skip_special_tokens=False) for t in ids_j]
                        top_tokens.append(Tokens(ids_j, lps_j, toptexts, [t in self.all_special_ids for t in ids_j]))
                generations.append(Generation(
                    s.request.id, prefill_tokens, Tokens(kept_ids, kept_lps, texts, specials), generated_text,
                    top_tokens))
        # sequences that processed a chunk but did not finish their prompt
        for i, s in enumerate(seqs):
            if s.prefilling and counts[i] > 0 and i not in active:
                s.cache_len += counts[i]
                s.first_chunk = None
        decode_ns = time.time_ns() - decode_start
        if all(s.finished for s in seqs):
            return generations, None, (forward_ns, decode_ns)
        return generations, batch, (forward_ns, decode_ns)
