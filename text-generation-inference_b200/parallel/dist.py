"""Process-group bootstrap: one process per GPU, ``torch.distributed`` for the plumbing.

Same role as ``server/text_generation_server/utils/dist.py:16-112`` of the
reference (NCCL group with a timeout, a ``FakeGroup`` when the world has one
rank or ``DEBUG=1``).  Differences: the rendezvous defaults to ``127.0.0.1``,
CPU runs use ``gloo`` so multi-process host logic can be tested without GPUs,
and the hot collectives of the forward pass do not go through this group at all
(see ``parallel/peer.py``): NCCL is used for bootstrap (exchange of peer-memory
handles, barriers) and as the baseline path.
"""
from __future__ import annotations

import os
from datetime import timedelta
from typing import List, Optional, Tuple

import torch


class FakeGroup:
    """Stand-in for a process group of a given shape that never communicates."""

    def __init__(self, rank: int = 0, size: int = 1):
        self._rank, self._size = rank, size

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._size

    # collectives used by the layers; identity on one rank
    def allreduce(self, *a, **k):
        return _Done()

    def allgather(self, inputs, local_tensor, **k):
        for t in inputs:
            for x in (t if isinstance(t, (list, tuple)) else [t]):
                x[:] = local_tensor
        return _Done()

    def barrier(self, *a, **k):
        return _Done()


class _Done:
    def wait(self):
        return None


def initialize_torch_distributed(timeout_s: Optional[float] = None) -> Tuple[object, int, int]:
    """Join the job described by ``RANK``/``WORLD_SIZE``/``MASTER_ADDR``/``MASTER_PORT``.

    Returns ``(process_group, rank, world_size)``.  ``DEBUG=1`` with ``WORLD_SIZE>1`` returns a
    ``FakeGroup`` of that shape so a single shard of a sharded model can be loaded alone.
    """
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if timeout_s is None:
        timeout_s = float(os.environ.get("TGI_B200_DIST_TIMEOUT", "120"))
    if world == 1:
        return FakeGroup(0, 1), 0, 1
    if os.environ.get("DEBUG") == "1":
        return FakeGroup(rank, world), rank, world
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
            torch.cuda.set_device(local)
            backend = "nccl"
            kwargs["device_id"] = torch.device("cuda", local)
        else:
            backend = "gloo"
        dist.init_process_group(backend=backend, world_size=world, rank=rank,
                                timeout=timedelta(seconds=timeout_s), **kwargs)
    return dist.group.WORLD, rank, world


def pin_cpu_threads(local_rank: int, local_world: int, cpus: Optional[List[int]] = None) -> List[int]:
    """Give every shard process its own slice of the host cores (reference: ``init_cpu_threads_env``,
    ``models/flash_causal_lm.py:91-122``): the tokenizer threads, the Python step loop and the torch
    intra-op pool of one shard then do not migrate onto the cores of another.  The cores the process may
    use are split into ``local_world`` contiguous slices (contiguous ids share a socket on the usual
    enumerations); returns the slice taken.  Opt-in through ``TGI_B200_PIN_CPU=1`` in the shard CLI."""
    cpus = sorted(cpus if cpus is not None else os.sched_getaffinity(0))
    per = len(cpus) // max(local_world, 1)
    if per < 1:
        return cpus                      # fewer cores than shards: leave the scheduler alone
    mine = cpus[local_rank * per:(local_rank + 1) * per]
    try:
        os.sched_setaffinity(0, mine)
    except (AttributeError, OSError):
        return cpus
    torch.set_num_threads(max(1, min(len(mine), int(os.environ.get("OMP_NUM_THREADS", len(mine))))))
    return mine


def all_reduce(t: torch.Tensor, group) -> torch.Tensor:
    if group is None or group.size() == 1 or isinstance(group, FakeGroup):
        return t
    import torch.distributed as dist

    dist.all_reduce(t, group=group)
    return t


def all_gather_into(out: torch.Tensor, t: torch.Tensor, group) -> torch.Tensor:
    if group is None or group.size() == 1 or isinstance(group, FakeGroup):
        out.copy_(t.view_as(out))
        return out
    import torch.distributed as dist

    dist.all_gather_into_tensor(out, t, group=group)
    return out


def barrier(group) -> None:
    if group is None or group.size() == 1 or isinstance(group, FakeGroup):
        return
    import torch.distributed as dist

    dist.barrier(group=group)
