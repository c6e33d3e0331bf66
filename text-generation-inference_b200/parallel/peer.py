"""Tensor-parallel communication over NVLink peer memory.

The reference reduces the output of every row-parallel linear with an NCCL all-reduce and then runs
residual-add + RMSNorm as separate kernels (``layers/tensor_parallel.py:202-209``,
``layers/layernorm.py:161-187``).  Here each rank owns a *heap* (one ``cudaMalloc`` block) that is
mapped into every other rank with CUDA IPC, and one kernel (``csrc/peer_comm.cu``) does
reduce-scatter by peer loads, the residual/norm/quantisation math on the rows a rank owns, and the
all-gather by peer stores.  ``torch.distributed`` is only used to exchange the IPC handles.

Buffers at fixed offsets of every heap:

    flags    uint32 [2][256][8]          block-to-block signals of the kernel
    partial  bf16   [max_tokens, width]  written by the local producer (GEMM output, embedding rows)
    gather   bf16   [max_tokens, width]  result rows pushed by their owners (reused for e4m3 bytes)
    gscale   fp32   [width/128, pitch]   1x128 activation scales of the e4m3 result, K-block major

The un-normalised residual stream of the rows a rank owns stays in ``self.residual`` on that rank and
never crosses NVLink.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch

from ..ops import cuda as K
from . import dist as pdist

FP8 = torch.float8_e4m3fn
_ALIGN = 1024


class _Span:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_Span(ptr, nbytes), device=device)


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def exchange_handles(group, rank: int, world: int, handle: bytes) -> List[bytes]:
    """All-gather of the 64-byte IPC handles (works on NCCL and gloo groups)."""
    import torch.distributed as dist

    out: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(out, handle, group=group)
    return [bytes(h) for h in out]


class PeerComm:
    """Peer-memory collectives of one tensor-parallel group (world <= 8, one node)."""

    def __init__(self, group, rank: int, world: int, device: torch.device, max_tokens: int, width: int):
        assert 1 <= world <= 8
        self.group, self.rank, self.world, self.device = group, rank, world, device
        self.max_tokens, self.width = int(max_tokens), int(width)
        lib = self.lib = K.load()
        for name in ("tgi_peer_alloc", "tgi_peer_free", "tgi_peer_export", "tgi_peer_import", "tgi_peer_unmap",
                     "tgi_peer_max_blocks", "tgi_peer_reduce", "tgi_peer_argmax", "tgi_peer_sample"):
            getattr(lib, name).restype = ctypes.c_int
        lib.tgi_peer_sample_xchg_bytes.restype = ctypes.c_longlong
        self.max_blocks = int(lib.tgi_peer_max_blocks())
        self.pitch = _round_up(self.max_tokens, 4)
        nflag = 2 * self.max_blocks * 8 * 4
        nrows = self.max_tokens * self.width * 2
        self.off_flags = 0
        self.off_push_flags = nflag           # uint32 [8]: call counter of every source's last finished push
        self.off_partial = _round_up(nflag + 64, _ALIGN)
        # as push slots [world][ceil(T / world)][width] the region can need up to world - 1 rows more than T
        self.off_gather = self.off_partial + _round_up(nrows + 8 * self.width * 2, _ALIGN)
        self.off_gscale = self.off_gather + _round_up(nrows, _ALIGN)
        self.off_cand = self.off_gscale + _round_up(max(self.width // 128, 1) * self.pitch * 4, _ALIGN)
        self.max_argmax_rows = 1024          # greedy candidates: 16 bytes per row and rank
        self.off_xchg = self.off_cand + _round_up(self.max_argmax_rows * 8 * 16, _ALIGN)   # sampler exchange words
        self.heap_bytes = self.off_xchg + _round_up(int(lib.tgi_peer_sample_xchg_bytes()), _ALIGN)

        torch.cuda.set_device(device)
        base = ctypes.c_void_p()
        rc = lib.tgi_peer_alloc(ctypes.c_longlong(self.heap_bytes), ctypes.byref(base))
        if rc != 0:
            raise K.KernelError(f"peer heap allocation of {self.heap_bytes} bytes failed ({rc})")
        self.base = int(base.value)
        self._mapped: List[int] = []
        self.heaps = [0] * world
        self.heaps[rank] = self.base
        if world > 1:
            handle = (ctypes.c_ubyte * 64)()
            if lib.tgi_peer_export(ctypes.c_void_p(self.base), handle) != 0:
                raise K.KernelError("cudaIpcGetMemHandle failed for the peer heap")
            handles = exchange_handles(group, rank, world, bytes(handle))
            for r, h in enumerate(handles):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                rc = lib.tgi_peer_import(buf, ctypes.byref(p))
                if rc != 0:
                    raise K.KernelError(f"cudaIpcOpenMemHandle failed for the heap of rank {r} (cuda error {-rc})")
                self.heaps[r] = int(p.value)
                self._mapped.append(int(p.value))
        self._heap_arr = (ctypes.c_void_p * 8)(*(self.heaps + [0] * (8 - world)))
        self._heap_t = tensor_from_ptr(self.base, self.heap_bytes, device)
        self._partial = self._heap_t[self.off_partial:self.off_partial + nrows].view(torch.bfloat16)
        self._gather = self._heap_t[self.off_gather:self.off_gather + nrows]
        self._gscale = self._heap_t[self.off_gscale:self.off_cand].view(torch.float32)
        self.epoch = torch.zeros(self.max_blocks, dtype=torch.int32, device=device)
        self.push_state = torch.zeros(2, dtype=torch.int32, device=device)   # [finished CTAs, call counter]
        self.xseq = torch.zeros(self.max_blocks, dtype=torch.int32, device=device)   # sampler exchange rounds per block
        # row-parallel GEMMs push their rows to the owners from this many tokens on; smaller steps pull
        self.push_min_tokens = int(os.environ.get("TGI_B200_PUSH_MIN_TOKENS", "512"))
        rows_per = (self.max_tokens + world - 1) // world
        self.residual = torch.zeros(rows_per, self.width, dtype=torch.bfloat16, device=device)
        self.status = K.state(device).status
        # every rank must have mapped every heap before anyone's kernel writes into a peer
        pdist.barrier(group)

    # ---- buffers -------------------------------------------------------------------------------
    def partial(self, T: int, H: Optional[int] = None) -> torch.Tensor:
        """``[T, H]`` bf16 view of the partial-sum buffer: the producer of a reduction writes here."""
        H = H or self.width
        assert T * H <= self.max_tokens * self.width, "reduction larger than the peer buffers"
        return self._partial[: T * H].view(T, H)

    def _gather_bf16(self, T: int, H: int) -> torch.Tensor:
        return self._gather[: T * H * 2].view(torch.bfloat16).view(T, H)

    def _gather_fp8(self, T: int, H: int) -> Tuple[torch.Tensor, torch.Tensor]:
        q = self._gather[: T * H].view(FP8).view(T, H)
        s = self._gscale[: (H // 128) * self.pitch].view(H // 128, self.pitch)[:, :T].t()
        return q, s

    def _blocks(self, T: int) -> int:
        return max(1, min(128, self.max_blocks, (T + self.world - 1) // self.world))

    def _launch(self, T: int, H: int, mode: int, residual_in, residual_out, weight, eps: float, w_offset: float,
                pushed: bool = False):
        rc = self.lib.tgi_peer_reduce(
            self._heap_arr, ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_int(T), ctypes.c_int(H),
            ctypes.c_longlong(self.off_partial), ctypes.c_longlong(self.off_gather), ctypes.c_longlong(self.off_gscale),
            ctypes.c_int(self.pitch), ctypes.c_longlong(self.off_flags), K._ptr(self.epoch),
            K._ptr(residual_in), K._ptr(residual_out), K._ptr(weight), ctypes.c_float(eps), ctypes.c_float(w_offset),
            ctypes.c_int(mode), ctypes.c_int(self._blocks(T)), K._ptr(self.status),
            ctypes.c_int(1 if pushed else 0), ctypes.c_longlong(self.off_push_flags),
            ctypes.c_void_p(self.push_state.data_ptr() + 4), K._stream())
        K._check(rc, "peer_reduce")

    def push_target(self, T: int, N: Optional[int] = None) -> "PeerPush":
        """Destination object for a row-parallel GEMM (pass it as ``out=``): the GEMM's epilogue stores
        every output row into the peer-memory slot of the rank that owns the row.  If the linear
        cannot push (no native kernel for its weight format) it writes ``fallback`` instead and the
        reduction pulls as usual; ``used`` tells which happened."""
        return PeerPush(self, T, N or self.width)

    # ---- collectives ---------------------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over ranks of a bf16 ``[..., H]`` tensor (other dtypes go through the group)."""
        if self.world == 1:
            return t
        H = t.shape[-1] if t.dim() > 0 else 1
        if t.dtype != torch.bfloat16 or H % 8 != 0 or not t.is_contiguous():
            return pdist.all_reduce(t, self.group)
        flat = t.view(-1, H)
        cap = max(1, (self.max_tokens * self.width) // H)
        for r0 in range(0, flat.shape[0], cap):
            rows = flat[r0:r0 + cap]
            T = rows.shape[0]
            if rows.data_ptr() != self._partial.data_ptr():
                self.partial(T, H).copy_(rows)
            self._launch(T, H, 0, None, None, None, 0.0, 0.0)
            rows.copy_(self._gather_bf16(T, H))
        return t

    def reduce_norm(self, T: int, weight: torch.Tensor, eps: float, w_offset: float = 0.0, quant: bool = False,
                    first: bool = False, source: Optional["PeerPush"] = None):
        """Sum the ranks' ``partial(T)`` rows, add the residual stream, RMSNorm (and quantise).

        Returns the normalised activations of all ``T`` rows: a bf16 ``[T, H]`` tensor, or
        ``(xq, xs)`` with 1x128 scales when ``quant``.  The tensors are views of the gather buffer and
        are overwritten by the next collective.  ``first`` starts a new residual stream (the summed
        rows themselves become the residual), as at the embedding.
        """
        H = self.width
        assert T <= self.max_tokens and weight.shape[0] == H
        pushed = source is not None and source.used
        self._launch(T, H, 2 if quant else 1, None if first else self.residual, self.residual, weight, eps, w_offset,
                     pushed=pushed)
        if quant:
            return self._gather_fp8(T, H)
        return self._gather_bf16(T, H)

    def argmax(self, local_logits: torch.Tensor, vocab_start: int, logit_scale: float = 1.0,
               out_ids: Optional[torch.Tensor] = None, out_logprobs: Optional[torch.Tensor] = None):
        """Greedy token ids (int64) and their log-probabilities from vocabulary-sharded bf16 logits
        ``[B, V / world]``: only a 16-byte candidate per row and rank crosses NVLink."""
        B, Vl = local_logits.shape
        assert local_logits.dtype == torch.bfloat16 and local_logits.stride(1) == 1 and B <= self.max_argmax_rows
        ids = out_ids if out_ids is not None else torch.empty(B, dtype=torch.int64, device=self.device)
        lps = out_logprobs if out_logprobs is not None else torch.empty(B, dtype=torch.float32, device=self.device)
        rc = self.lib.tgi_peer_argmax(
            self._heap_arr, ctypes.c_int(self.rank), ctypes.c_int(self.world), K._ptr(local_logits), ctypes.c_int(B),
            ctypes.c_int(Vl), ctypes.c_longlong(local_logits.stride(0)), ctypes.c_int(vocab_start),
            ctypes.c_float(logit_scale), ctypes.c_longlong(self.off_cand), ctypes.c_longlong(self.off_flags),
            K._ptr(self.epoch), K._ptr(ids), K._ptr(lps), ctypes.c_int(max(1, min(B, self.max_blocks))),
            K._ptr(self.status), K._stream())
        K._check(rc, "peer_argmax")
        return ids, lps

    def sample(self, local_scores: torch.Tensor, vocab_start: int, vocab_total: int, logit_scale: float = 1.0,
               temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
               top_p: Optional[torch.Tensor] = None, do_sample: Optional[torch.Tensor] = None,
               seeds: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None):
        """Temperature / top-k / top-p / seeded sampling on vocabulary-sharded scores ``[B, V / world]`` (bf16
        logits, or fp32 scores that already carry the penalties): the ranks exchange a few scalars per row instead
        of gathering ``[B, V]`` logits, and all of them return the same ``(ids int64, logprobs fp32)``.  The draw
        for a seed equals the single-GPU fused sampler's (``ops.fused_sample``)."""
        B, Vl = local_scores.shape
        assert local_scores.stride(1) == 1 and local_scores.dtype in (torch.bfloat16, torch.float32)
        dev = self.device

        def as_(t, dtype):
            return None if t is None else t.to(device=dev, dtype=dtype).contiguous()

        temperature, top_p = as_(temperature, torch.float32), as_(top_p, torch.float32)
        top_k, steps = as_(top_k, torch.int32), as_(steps, torch.int32)
        do_sample, seeds = as_(do_sample, torch.uint8), as_(seeds, torch.int64)
        ids = torch.empty(B, dtype=torch.int64, device=dev)
        lps = torch.empty(B, dtype=torch.float32, device=dev)
        rc = self.lib.tgi_peer_sample(
            self._heap_arr, ctypes.c_int(self.rank), ctypes.c_int(self.world), K._ptr(local_scores),
            ctypes.c_int(1 if local_scores.dtype == torch.float32 else 0), ctypes.c_int(B), ctypes.c_int(Vl),
            ctypes.c_longlong(local_scores.stride(0)), ctypes.c_int(vocab_start), ctypes.c_int(vocab_total),
            ctypes.c_float(logit_scale), K._ptr(temperature), K._ptr(top_k), K._ptr(top_p), K._ptr(do_sample),
            K._ptr(seeds), K._ptr(steps), ctypes.c_longlong(self.off_xchg), K._ptr(self.xseq), K._ptr(ids), K._ptr(lps),
            ctypes.c_int(max(1, min(B, self.max_blocks))), K._ptr(self.status), K._stream())
        K._check(rc, "peer_sample")
        return ids, lps

    def check(self) -> int:
        return K.check_status(self.device)

    def close(self):
        torch.cuda.synchronize(self.device)
        pdist.barrier(self.group)
        for p in self._mapped:
            self.lib.tgi_peer_unmap(ctypes.c_void_p(p))
        self._mapped = []
        if self.base:
            self.lib.tgi_peer_free(ctypes.c_void_p(self.base))
            self.base = 0


class PeerPush:
    """``out=`` target that makes a GEMM store its rows into the owners' peer-memory slots.

    ``ops.cuda.gemm_bf16`` / ``gemm_fp8_block`` recognise it by ``is_peer_push`` and call
    ``launch(...)``; any other producer may write the plain tensor ``fallback`` (the pull buffer)."""

    is_peer_push = True

    def __init__(self, comm: PeerComm, T: int, N: int):
        self.comm, self.T, self.N = comm, T, N
        self.rows_per = (T + comm.world - 1) // comm.world
        self.used = False
        assert comm.world * self.rows_per * N <= (comm.max_tokens + 8) * comm.width

    @property
    def fallback(self) -> torch.Tensor:
        return self.comm.partial(self.T, self.N)

    def gemm_args(self):
        """Trailing arguments of ``tgi_gemm_push`` that describe the destination."""
        c = self.comm
        self.used = True
        return (c._heap_arr, ctypes.c_int(c.rank), ctypes.c_int(c.world), ctypes.c_int(self.rows_per),
                ctypes.c_longlong(c.off_partial), ctypes.c_longlong(c.off_push_flags),
                ctypes.c_void_p(c.push_state.data_ptr()), ctypes.c_void_p(c.push_state.data_ptr() + 4))


def make_comm(group, rank: int, world: int, device: torch.device, hidden: int, max_tokens: int):
    """Peer-memory communicator of a tensor-parallel group, or ``None`` when it does not apply
    (one rank, CPU run, ``TGI_B200_COMM=nccl`` for the library baseline, or a ``FakeGroup``)."""
    import os

    if world == 1 or device.type != "cuda" or isinstance(group, pdist.FakeGroup):
        return None
    if os.environ.get("TGI_B200_COMM", "peer") == "nccl":
        return None
    return PeerComm(group, rank, world, device, max_tokens, hidden)
