"""CUDA-graph decode: one captured forward per batch-size bucket.

The reference captures the decode forward for batch sizes ``CUDA_GRAPHS`` (default 1,2,4,8,16,32)
into ``torch.cuda.CUDAGraph`` objects with static input tensors and pads a batch to the next size
(``models/flash_causal_lm.py:1438-1505`` capture, ``:1792-1888`` replay).  Same idea here with two
changes: buckets go up to the maximum batch size (256 by default) because a launch-bound decode step
is where B200 loses most, and all static inputs of a bucket live in ONE int32 buffer that is filled
by a single host-to-device copy per step.

Padding rows use slot ``-1`` (the RoPE+KV-store kernel skips the write) and a KV length of 0 (the
attention kernel produces zeros), so they never touch real cache pages.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .decoder import ForwardMeta

DEFAULT_BUCKETS = [1, 2, 4, 8, 16, 32, 64, 96, 128, 192, 256]


def configured_buckets() -> List[int]:
    env = os.environ.get("CUDA_GRAPHS")
    if env:
        vals = sorted({int(x) for x in env.split(",") if x.strip() and int(x) > 0})
        return vals
    return list(DEFAULT_BUCKETS)


class _Bucket:
    def __init__(self, runner, bs: int, max_blocks: int, pool):
        dev = runner.device
        self.bs, self.max_blocks = bs, max_blocks
        # layout of the static int32 buffer (every segment starts on a 16-byte boundary)
        seg = lambda n: (n + 3) & ~3
        self.off_ids = 0
        self.off_pos = self.off_ids + seg(bs)
        self.off_slots = self.off_pos + seg(bs)
        self.off_cu = self.off_slots + seg(bs)
        self.off_kv = self.off_cu + seg(bs + 1)
        self.off_bt = self.off_kv + seg(bs)
        self.off_ad = self.off_bt + seg(bs * max_blocks)     # LoRA adapter index per row (0 = none)
        self.total = self.off_ad + seg(bs)
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=dev)
        self.host_np[self.off_cu:self.off_cu + bs + 1] = np.arange(bs + 1, dtype=np.int32)
        self.host_np[self.off_slots:self.off_slots + bs] = -1
        self.dev.copy_(self.host)
        d = self.dev
        self.meta = ForwardMeta(
            input_ids=d[self.off_ids:self.off_ids + bs],
            positions=d[self.off_pos:self.off_pos + bs],
            slots=d[self.off_slots:self.off_slots + bs],
            cu_seqlens_q=d[self.off_cu:self.off_cu + bs + 1],
            kv_lens=d[self.off_kv:self.off_kv + bs],
            block_tables=d[self.off_bt:self.off_bt + bs * max_blocks].view(bs, max_blocks),
            max_q=1,
            max_kv=runner_max_kv(runner),
            lm_head_indices=None,
        )
        self.token_adapter = d[self.off_ad:self.off_ad + bs]
        self.row_owner: List[Optional[tuple]] = [None] * bs   # (block list, its length) whose table sits in row i
        self.staged = torch.cuda.Event()        # recorded after every host-to-device copy of the static buffer
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None          # full logits [bs, V] (gathered-head graphs)
        self.local_logits: Optional[torch.Tensor] = None    # vocabulary shard [bs, V / tp] (local-head graphs)
        self.greedy_ids: Optional[torch.Tensor] = None      # filled inside the graph by the peer argmax
        self.greedy_logprobs: Optional[torch.Tensor] = None


def runner_max_kv(runner) -> int:
    return int(getattr(runner, "_graph_max_total_tokens", 4096))


class DecodeGraphs:
    def __init__(self, runner, max_total_tokens: int, buckets: Optional[List[int]] = None):
        self.runner = runner
        self.max_total_tokens = int(max_total_tokens)
        runner._graph_max_total_tokens = self.max_total_tokens
        self.max_blocks = math.ceil(self.max_total_tokens / runner.block_size)
        self.sizes = buckets or configured_buckets()
        self.buckets: Dict[int, _Bucket] = {}
        # graphs whose forward includes the multi-adapter LoRA kernels; captured on first use of a size, so
        # batches without adapters never pay for the extra launches
        self.lora_buckets: Dict[int, _Bucket] = {}
        self.pool = None

    def capture_all(self):
        for bs in sorted(self.sizes, reverse=True):
            self.capture(bs)

    def capture(self, bs: int, lora: bool = False):
        r = self.runner
        b = _Bucket(r, bs, self.max_blocks, self.pool)
        if lora:
            from ..utils.adapter import LoraBatchData

            b.meta.adapter_data = LoraBatchData.static(r.lora, b.token_adapter)
        # warm-up run outside capture: lazy kernel attributes and persistent scratch get set up here
        torch.cuda.synchronize(r.device)
        r.model.forward(b.meta, r.kv_cache)
        torch.cuda.synchronize(r.device)
        g = torch.cuda.CUDAGraph()
        local_head = bool(getattr(r.model, "supports_local_head", False))
        if local_head:
            # Sharded lm_head: the graph ends with the vocabulary-parallel argmax, so a greedy step never
            # gathers logits; samplers that need the distribution gather the shard after the replay.
            d = r.model.dims
            b.greedy_ids = torch.zeros(bs, dtype=torch.int64, device=r.device)
            b.greedy_logprobs = torch.zeros(bs, dtype=torch.float32, device=r.device)
            local, v0 = r.model.forward_local(b.meta, r.kv_cache)
            r.model.comm.argmax(local, v0, d.logit_scale, b.greedy_ids, b.greedy_logprobs)
            torch.cuda.synchronize(r.device)
            with torch.cuda.graph(g, pool=self.pool):
                local, v0 = r.model.forward_local(b.meta, r.kv_cache)
                r.model.comm.argmax(local, v0, d.logit_scale, b.greedy_ids, b.greedy_logprobs)
            b.local_logits = local
        else:
            with torch.cuda.graph(g, pool=self.pool):
                logits, _ = r.model.forward(b.meta, r.kv_cache)
            b.logits = logits
        if self.pool is None:
            self.pool = g.pool()
        torch.cuda.synchronize(r.device)
        b.graph = g
        (self.lora_buckets if lora else self.buckets)[bs] = b

    def supports(self, batch) -> bool:
        n = len(batch)
        if not self.buckets or n > max(self.buckets):
            return False
        for s in batch.seqs:
            if len(s.blocks) > self.max_blocks or len(s.ids) > self.max_total_tokens:
                return False
        return True

    def run(self, batch, counts: List[int]):
        seqs = batch.seqs
        n = len(seqs)
        bs = min(k for k in self.buckets if k >= n)
        lora = getattr(self.runner, "lora", None) is not None and any(s.adapter_index > 0 for s in seqs)
        if lora and bs not in self.lora_buckets:
            self.capture(bs, lora=True)
        b = self.lora_buckets[bs] if lora else self.buckets[bs]
        b.staged.synchronize()      # the pinned buffer is rewritten below: its previous copy must have left the host
        h = b.host_np
        ids = h[b.off_ids:b.off_ids + bs]
        pos = h[b.off_pos:b.off_pos + bs]
        slots = h[b.off_slots:b.off_slots + bs]
        kv = h[b.off_kv:b.off_kv + bs]
        bt = h[b.off_bt:b.off_bt + bs * b.max_blocks].reshape(bs, b.max_blocks)
        for i, s in enumerate(seqs):
            p = len(s.ids) - 1
            ids[i] = s.ids[-1]
            pos[i] = p + getattr(s, "pos_delta", 0)
            slots[i] = s.slots[p]
            kv[i] = p + 1
            nb = len(s.blocks)
            held = b.row_owner[i]
            if held is None or held[0] is not s.blocks or held[1] != nb:
                # the block table row of a sequence is written once per placement; the bucket keeps a reference to
                # the list, so "same list object" cannot be a recycled identity
                bt[i, :nb] = s.blocks
                b.row_owner[i] = (s.blocks, nb)
        if lora:
            ad = h[b.off_ad:b.off_ad + bs]
            ad[:n] = [s.adapter_index for s in seqs]
            ad[n:] = 0
        if n < bs:
            ids[n:] = 0
            pos[n:] = 0
            slots[n:] = -1
            kv[n:] = 0
        b.dev.copy_(b.host, non_blocking=True)
        b.staged.record()
        b.graph.replay()
        row_owner = [(i, 0) for i in range(n)]
        self.last = (b, n)
        return (b.logits[:n] if b.logits is not None else None), row_owner

    def advance(self, seqs, next_ids: List[int]):
        """Replay the bucket of the last step once more for the same sequences, one token further: ids, positions
        and KV lengths are updated in place (block tables and adapter indices stay), so the host work between
        two decode steps is a handful of vector operations.  The caller has appended ``next_ids`` to the sequences."""
        b, n = self.last
        b.staged.synchronize()
        h = b.host_np
        h[b.off_ids:b.off_ids + n] = next_ids
        h[b.off_pos:b.off_pos + n] += 1
        h[b.off_kv:b.off_kv + n] += 1
        slots = h[b.off_slots:b.off_slots + n]
        for i, s in enumerate(seqs):
            slots[i] = s.slots[len(s.ids) - 1]
        b.dev.copy_(b.host, non_blocking=True)
        b.staged.record()
        b.graph.replay()
        return (b.logits[:n] if b.logits is not None else None), [(i, 0) for i in range(n)]

    def greedy(self):
        """``(ids, logprobs)`` of the last replay when its graph sampled greedily in-kernel, else ``None``."""
        b, n = self.last
        if b.greedy_ids is None:
            return None
        return b.greedy_ids[:n], b.greedy_logprobs[:n]

    def gather_last_logits(self) -> torch.Tensor:
        b, n = self.last
        return self.runner.model.gather_logits(b.local_logits)[:n]
