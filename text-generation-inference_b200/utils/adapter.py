"""Multi-LoRA serving: adapter discovery, sharded loading and per-batch application.

Reference: ``utils/adapter.py:50-329`` (``LORA_ADAPTERS`` parsing, loading), ``adapters/lora.py``
(``LoraWeights`` / ``BatchLoraWeights``), ``layers/lora.py:35-356`` (SGMV/BGMV application and the
tensor-parallel collectives), ``utils/merges`` (combining several adapters into one).

An adapter adds ``scale * (x A^T) B^T`` to the output of a target projection.  A request selects
its adapter with ``adapter_id``; one forward pass can mix requests of different adapters and of the
base model.  Tokens are grouped by adapter and each group runs two skinny GEMMs.

Tensor parallelism: for column-parallel targets (q/k/v/gate/up) ``B`` is sharded like the base
weight's output rows and ``A`` is replicated, so no communication is needed.  For row-parallel
targets (o/down) ``A`` is sharded along the input and the ``[T, r]`` intermediate is all-reduced
before ``B`` is applied (the reference does the same, ``layers/lora.py:347-356``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..parallel import dist as pdist
from .weights import SafetensorsFile, shard_bounds

COLUMN_TARGETS = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
ROW_TARGETS = ("o_proj", "down_proj")
BASE_MODEL_ADAPTER_ID = "__base_model__"

# adapter_id -> index (0 is the base model); filled by ``load_and_attach_adapters``
ADAPTER_TO_INDEX: Dict[str, int] = {}


@dataclass
class AdapterParameters:
    adapter_id: str
    path: Optional[str] = None
    revision: Optional[str] = None


def parse_lora_adapters(spec: Optional[str]) -> List[AdapterParameters]:
    """``"id1,id2=/path/to/dir,id3@rev"`` -> adapter descriptions (the ``LORA_ADAPTERS`` format)."""
    out: List[AdapterParameters] = []
    if not spec:
        return out
    for item in spec.split(","):
        item = item.strip()
        if not item:
            continue
        path = None
        if "=" in item:
            item, path = item.split("=", 1)
        revision = None
        if "@" in item:
            item, revision = item.split("@", 1)
        if not item:
            raise ValueError(f"invalid LoRA adapter specification {spec!r}")
        out.append(AdapterParameters(item, path, revision))
    ids = [a.adapter_id for a in out]
    if len(set(ids)) != len(ids):
        raise ValueError("duplicate adapter ids in LORA_ADAPTERS")
    return out


@dataclass
class LoraConfig:
    r: int
    lora_alpha: float
    target_modules: List[str]
    use_rslora: bool = False

    @property
    def scale(self) -> float:
        return self.lora_alpha / (self.r ** 0.5 if self.use_rslora else self.r)

    @classmethod
    def load(cls, path: Path) -> "LoraConfig":
        cfg = json.loads((Path(path) / "adapter_config.json").read_text())
        return cls(int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"])), list(cfg.get("target_modules") or []),
                   bool(cfg.get("use_rslora", False)))


@dataclass
class LoraLayer:
    """One target projection of one adapter on this rank: ``A[r, in]``, ``B[out, r]``."""

    a: torch.Tensor
    b: torch.Tensor
    scale: float


@dataclass
class LoraAdapter:
    adapter_id: str
    config: LoraConfig
    layers: Dict[Tuple[int, str], LoraLayer] = field(default_factory=dict)


def _find_adapter_file(path: Path) -> Path:
    for name in ("adapter_model.safetensors", "adapter.safetensors"):
        if (path / name).exists():
            return path / name
    raise FileNotFoundError(f"no adapter_model.safetensors in {path}")


def _kv_bounds(total_kv: int, head_dim: int, rank: int, world: int) -> Tuple[int, int]:
    if total_kv >= world:
        per = total_kv // world
        return rank * per * head_dim, (rank + 1) * per * head_dim
    h = rank * total_kv // world          # fewer KV heads than ranks: the owning head is replicated
    return h * head_dim, (h + 1) * head_dim


def load_adapter(adapter_id: str, path: Path, dims, rank: int, world: int, device, dtype) -> LoraAdapter:
    """Read a PEFT LoRA checkpoint and keep this rank's shard of every target projection."""
    path = Path(path)
    cfg = LoraConfig.load(path)
    adapter = LoraAdapter(adapter_id, cfg)
    f = SafetensorsFile(_find_adapter_file(path))
    names = list(f.keys())
    D = dims.head_dim
    for name in names:
        if ".lora_A" not in name:
            continue
        parts = name.split(".")
        try:
            li = int(parts[parts.index("layers") + 1])
        except (ValueError, IndexError):
            continue
        proj = next((p for p in COLUMN_TARGETS + ROW_TARGETS if p in parts), None)
        if proj is None:
            continue
        a = f.get_tensor(name).to(torch.float32)
        b = f.get_tensor(name.replace("lora_A", "lora_B")).to(torch.float32)
        if world > 1:
            if proj in ROW_TARGETS:
                lo, hi = shard_bounds(a.shape[1], rank, world)
                a = a[:, lo:hi]
            elif proj == "q_proj":
                lo, hi = shard_bounds(b.shape[0], rank, world)
                b = b[lo:hi]
            elif proj in ("k_proj", "v_proj"):
                lo, hi = _kv_bounds(dims.total_kv_heads, D, rank, world)
                b = b[lo:hi]
            else:
                lo, hi = shard_bounds(b.shape[0], rank, world)
                b = b[lo:hi]
        # clone: on CPU the tensors may still alias the file mapping that is closed below
        adapter.layers[(li, proj)] = LoraLayer(a.to(device=device, dtype=dtype).clone().contiguous(),
                                               b.to(device=device, dtype=dtype).clone().contiguous(), cfg.scale)
    f.close()
    return adapter


def merge_adapters(adapters: List[LoraAdapter], weights: List[float], merged_id: str, strategy: str = "linear",
                   density: float = 1.0, seed: int = 0) -> LoraAdapter:
    """Combine adapters of equal rank into one (``utils/merges`` of the reference).

    ``linear``: weighted sum of the factors.  ``dare``: random drop of ``1 - density`` of every factor's
    entries with rescaling, then the weighted sum.  ``ties``: keep the top ``density`` fraction of
    entries by magnitude, elect a sign per entry from the weighted sum, and average the entries that
    agree with it.
    """
    assert adapters and len(adapters) == len(weights)
    base = adapters[0]
    out = LoraAdapter(merged_id, base.config)
    gen = torch.Generator().manual_seed(seed)

    def prune(t: torch.Tensor) -> torch.Tensor:
        if strategy == "dare" and density < 1.0:
            mask = (torch.rand(t.shape, generator=gen) < density).to(t.device)
            return t * mask / density
        if strategy == "ties" and density < 1.0:
            k = max(1, int(density * t.numel()))
            thresh = t.abs().flatten().float().kthvalue(t.numel() - k + 1).values
            return t * (t.abs() >= thresh)
        return t

    def combine(ts: List[torch.Tensor]) -> torch.Tensor:
        ts = [prune(t.float()) * w for t, w in zip(ts, weights)]
        stack = torch.stack(ts)
        if strategy == "ties":
            sign = torch.sign(stack.sum(0))
            agree = (torch.sign(stack) == sign) & (stack != 0)
            return (stack * agree).sum(0) / agree.sum(0).clamp(min=1)
        return stack.sum(0)

    for key, layer in base.layers.items():
        if not all(key in ad.layers for ad in adapters):
            continue
        a = combine([ad.layers[key].a for ad in adapters]).to(layer.a.dtype)
        b = combine([ad.layers[key].b for ad in adapters]).to(layer.b.dtype)
        out.layers[key] = LoraLayer(a, b, layer.scale)
    return out


class LoraBatchData:
    """Adapter routing of one forward pass: which rows of the ragged batch use which adapter.

    On CUDA (bf16) every target projection is two kernel launches for the whole batch
    (``ops/csrc/lora_sm100.cu``: shrink to ``[T, r]``, expand into the output in place) driven by a
    per-row adapter index; elsewhere the rows are grouped by adapter and go through plain matmuls."""

    def __init__(self, manager: "LoraManager", token_adapter: np.ndarray, device):
        self.manager = manager
        self.groups: List[Tuple[int, torch.Tensor]] = []
        self.token_adapter = None
        if torch.device(device).type == "cuda":
            self.token_adapter = torch.from_numpy(np.ascontiguousarray(token_adapter, dtype=np.int32)).to(device)
        for idx in np.unique(token_adapter):
            if idx <= 0:
                continue
            rows = np.nonzero(token_adapter == idx)[0]
            self.groups.append((int(idx), torch.from_numpy(rows).to(device=device, dtype=torch.long)))

    @classmethod
    def static(cls, manager: "LoraManager", token_adapter: torch.Tensor) -> "LoraBatchData":
        """Routing that reads the adapter index of every row from a fixed device tensor (CUDA-graph decode:
        the tensor is rewritten before each replay)."""
        self = cls.__new__(cls)
        self.manager, self.groups, self.token_adapter = manager, [], token_adapter
        return self

    def _apply(self, layer: int, proj: str, x: torch.Tensor, out: torch.Tensor, col0: int, reduce_group=None):
        if self.token_adapter is not None and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
            tab = self.manager.table(layer, proj, x.device)
            if tab is None:
                return
            from ..ops import cuda as K

            v = K.lora_shrink(x, tab.a_ptrs, tab.ranks, self.token_adapter, tab.rmax)
            if reduce_group is not None:
                pdist.all_reduce(v, reduce_group)
            K.lora_expand(v, tab.b_ptrs, tab.ranks, tab.scales, self.token_adapter, out, col0, tab.ncols)
            return
        for idx, rows in self.groups:
            lora = self.manager.adapters[idx - 1].layers.get((layer, proj))
            if lora is None:
                continue
            z = x.index_select(0, rows) @ lora.a.t()
            if reduce_group is not None:
                pdist.all_reduce(z, reduce_group)
            delta = (z @ lora.b.t()) * lora.scale
            out[:, col0:col0 + delta.shape[1]].index_add_(0, rows, delta.to(out.dtype))

    def apply_qkv(self, layer: int, x: torch.Tensor, qkv: torch.Tensor) -> torch.Tensor:
        d = self.manager.dims
        nq, nk = d.num_heads * d.head_dim, d.num_kv_heads * d.head_dim
        self._apply(layer, "q_proj", x, qkv, 0)
        self._apply(layer, "k_proj", x, qkv, nq)
        self._apply(layer, "v_proj", x, qkv, nq + nk)
        return qkv

    def apply_gate_up(self, layer: int, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        half = h.shape[1] // 2
        self._apply(layer, "gate_proj", x, h, 0)
        self._apply(layer, "up_proj", x, h, half)
        return h

    def apply_row(self, layer: int, proj: str, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        pg = self.manager.process_group
        group = pg if pg is not None and pg.size() > 1 else None
        self._apply(layer, proj, x, out, 0, reduce_group=group)
        return out


@dataclass
class LoraTable:
    """Device-side pointer table of one (layer, projection): entry ``i`` describes adapter index ``i``
    (entry 0 and adapters without this target are null / rank 0)."""

    a_ptrs: torch.Tensor     # int64 [n + 1]
    b_ptrs: torch.Tensor     # int64 [n + 1]
    ranks: torch.Tensor      # int32 [n + 1]
    scales: torch.Tensor     # fp32 [n + 1]
    rmax: int
    ncols: int
    keep: list               # the contiguous A / B tensors the pointers refer to


class LoraManager:
    def __init__(self, dims, process_group):
        self.dims, self.process_group = dims, process_group
        self.adapters: List[LoraAdapter] = []
        self._tables: Dict[Tuple[int, str], Optional[LoraTable]] = {}

    def table(self, layer: int, proj: str, device) -> Optional[LoraTable]:
        key = (layer, proj)
        if key not in self._tables:
            n = len(self.adapters)
            a_ptrs, b_ptrs, ranks, scales, keep = [0] * (n + 1), [0] * (n + 1), [0] * (n + 1), [0.0] * (n + 1), []
            ncols = 0
            for i, ad in enumerate(self.adapters, start=1):
                lora = ad.layers.get(key)
                if lora is None:
                    continue
                a, b = lora.a.contiguous(), lora.b.contiguous()
                keep += [a, b]
                a_ptrs[i], b_ptrs[i], ranks[i], scales[i] = a.data_ptr(), b.data_ptr(), a.shape[0], float(lora.scale)
                ncols = max(ncols, b.shape[0])
            if not keep or max(ranks) > 128:
                self._tables[key] = None       # no adapter targets this projection (or rank beyond the kernels)
            else:
                self._tables[key] = LoraTable(
                    torch.tensor(a_ptrs, dtype=torch.int64, device=device),
                    torch.tensor(b_ptrs, dtype=torch.int64, device=device),
                    torch.tensor(ranks, dtype=torch.int32, device=device),
                    torch.tensor(scales, dtype=torch.float32, device=device), max(ranks), ncols, keep)
        return self._tables[key]

    def add(self, adapter: LoraAdapter) -> int:
        self._tables.clear()
        self.adapters.append(adapter)
        ADAPTER_TO_INDEX[adapter.adapter_id] = len(self.adapters)
        return len(self.adapters)

    def index_of(self, adapter_id: Optional[str]) -> int:
        if not adapter_id or adapter_id == BASE_MODEL_ADAPTER_ID:
            return 0
        return ADAPTER_TO_INDEX.get(adapter_id, 0)

    def batch_data(self, token_adapter: np.ndarray, device) -> Optional[LoraBatchData]:
        if not self.adapters or not (token_adapter > 0).any():
            return None
        return LoraBatchData(self, token_adapter, device)


def resolve_adapter_path(params: AdapterParameters) -> Path:
    if params.path:
        return Path(params.path)
    p = Path(params.adapter_id)
    if p.is_dir():
        return p
    from .hub import resolve_model_path

    return resolve_model_path(params.adapter_id, params.revision)


def load_and_attach_adapters(runner, model_id: str, adapters: List[AdapterParameters]) -> "LoraManager":
    """Load every adapter's shard and hang a ``LoraManager`` on the runner (``runner.lora``)."""
    model = runner.model
    pg = model.pg
    manager = LoraManager(model.dims, pg)
    for params in adapters:
        path = resolve_adapter_path(params)
        adapter = load_adapter(params.adapter_id, path, model.dims, pg.rank(), pg.size(), model.device, model.dtype)
        if not adapter.layers:
            raise ValueError(f"adapter {params.adapter_id} has no LoRA weights for this model's layers")
        manager.add(adapter)
    runner.lora = manager
    return manager
