"""Token history of a running batch, kept on the device.

Repetition / frequency penalties, watermarks and n-gram speculation read every sequence's ids each step.  The
reference keeps an ``all_input_ids_tensor`` per batch on the device and writes the new ids into it after
sampling (``models/flash_causal_lm.py:1971-1975``, ``2284-2296``); rebuilding that matrix from the host lists
every step costs a list-to-array conversion per sequence and megabytes of host-to-device traffic at 256
sequences.  ``TokenHistory`` owns a ``[rows, capacity]`` int64 buffer with one row per request id.  ``sync``
uploads a request's ids once, when it first shows up, and afterwards only the ids appended since the previous
step (one small copy and one scatter for the whole batch), then returns the ``[len(seqs), L]`` zero-padded matrix
for the rows asked for.  Rows of requests that left the batch are recycled.  The id lists are append-only (the
engine only ever appends accepted tokens), which is what lets a length stand for a list's contents.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import numpy as np
import torch


class TokenHistory:
    def __init__(self, device, rows: int = 64, capacity: int = 2048):
        self.device = torch.device(device)
        self.buf = torch.zeros(rows, capacity, dtype=torch.int64, device=self.device)
        self.row_of: Dict[int, int] = {}        # request id -> row
        self.len_of: Dict[int, int] = {}        # request id -> ids already on the device
        self.free: List[int] = list(range(rows - 1, -1, -1))

    # -- storage -----------------------------------------------------------------------------------
    def _grow(self, rows: int, capacity: int):
        r0, c0 = self.buf.shape
        r1 = max(r0, rows)
        c1 = c0
        while c1 < capacity:
            c1 *= 2
        if (r1, c1) == (r0, c0):
            return
        if r1 > r0:
            r1 = max(r1, 2 * r0)
            self.free = list(range(r1 - 1, r0 - 1, -1)) + self.free
        buf = torch.zeros(r1, c1, dtype=torch.int64, device=self.device)
        buf[:r0, :c0] = self.buf
        self.buf = buf

    def retain(self, request_ids: Iterable[int]):
        """Forget every request that is not in ``request_ids`` (its row is cleared and reused)."""
        keep = set(request_ids)
        gone = [rid for rid in self.row_of if rid not in keep]
        if not gone:
            return
        rows = [self.row_of.pop(rid) for rid in gone]
        for rid in gone:
            self.len_of.pop(rid, None)
        self.buf[torch.tensor(rows, dtype=torch.long, device=self.device)] = 0
        self.free.extend(rows)

    # -- per step ----------------------------------------------------------------------------------
    def sync(self, request_ids: Sequence[int], ids: Sequence[Sequence[int]]) -> torch.Tensor:
        """Bring the rows of ``request_ids`` up to date with ``ids`` (the full id list of each request) and return
        them as one ``[n, L]`` matrix, ``L`` the longest list, shorter rows zero padded."""
        n = len(request_ids)
        longest = max((len(x) for x in ids), default=1)
        new = [rid for rid in request_ids if rid not in self.row_of]
        self._grow(len(self.row_of) + len(new), longest)
        for rid in new:
            self.row_of[rid] = self.free.pop()
            self.len_of[rid] = 0
        rows_l, pos_l, tok_l = [], [], []
        for rid, seq in zip(request_ids, ids):
            have, row = self.len_of[rid], self.row_of[rid]
            if have > len(seq):                 # a request id reused for a shorter list: start the row over
                self.buf[row, :have] = 0
                have = 0
            if have < len(seq):
                k = len(seq) - have
                rows_l.append(np.full(k, row, dtype=np.int64))
                pos_l.append(np.arange(have, len(seq), dtype=np.int64))
                tok_l.append(np.asarray(seq[have:], dtype=np.int64))
                self.len_of[rid] = len(seq)
        if rows_l:
            packed = np.stack([np.concatenate(rows_l), np.concatenate(pos_l), np.concatenate(tok_l)])
            t = torch.from_numpy(packed).to(self.device)       # a few hundred bytes per step
            self.buf.index_put_((t[0], t[1]), t[2])
        order = [self.row_of[rid] for rid in request_ids]
        if n and order == list(range(order[0], order[0] + n)):     # neighbouring rows: a view, no gather
            return self.buf[order[0]:order[0] + n, :longest]
        return self.buf.index_select(0, torch.tensor(order, dtype=torch.long, device=self.device))[:, :longest]
