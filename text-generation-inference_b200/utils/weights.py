"""Checkpoint access and tensor-parallel sharding of HF safetensors weights.

Covers what the reference's ``server/text_generation_server/utils/weights.py``
does (``Weights`` at ``:139-442``, ``WeightsLoader`` strategy at ``:13-96``,
``DefaultWeightsLoader`` at ``:99-136``) with a different construction:

* ``SafetensorsFile`` is a small zero-copy reader: the file is ``mmap``-ed once,
  the JSON header is parsed, and every tensor (or a *slice* of it along one
  dimension) is a ``torch.frombuffer`` view into the mapping.  A shard of a
  row-major matrix along dim 0 is one contiguous byte range; along dim 1 it is
  a strided view that is made contiguous only while being copied to the GPU.
  The same class reads an in-memory ``bytes`` object, which is what the unit
  tests use instead of a mocked filesystem.
* ``Weights`` owns the routing table *tensor name -> file*, the process group
  (``rank``/``size``), the target device/dtype and the name aliases, and offers
  the sharding primitives: ``get_partial_sharded`` (ceil-div blocks, the last
  rank may get less), ``get_sharded`` (must divide), ``get_packed_sharded``
  (fused QKV / gate_up stored as one matrix whose parts have different widths)
  and the column/row conveniences used by the layers.
* Quantised formats are handled by *loader* objects (``utils/quantization.py``)
  that are handed the ``Weights`` instance; ``use_loader`` swaps the loader in a
  scope (the reference uses that to keep some layers un-quantised).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from contextlib import contextmanager
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

_ST_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn,
    "F8_E5M2": torch.float8_e5m2,
}
_ST_NAMES = {v: k for k, v in _ST_DTYPES.items()}


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class TensorSlice:
    """Lazy view of one tensor inside a safetensors blob.

    ``slice_dim(dim, start, stop)`` returns a torch view of the rows/columns
    ``[start, stop)`` without touching the rest of the tensor.
    """

    def __init__(self, buf, dtype: torch.dtype, shape: Sequence[int], begin: int, end: int):
        self._buf = buf
        self.dtype = dtype
        self.shape = tuple(int(s) for s in shape)
        self._begin = begin
        self._end = end

    def get_shape(self) -> Tuple[int, ...]:
        return self.shape

    def _full(self) -> torch.Tensor:
        n = 1
        for s in self.shape:
            n *= s
        if n == 0:
            return torch.empty(self.shape, dtype=self.dtype)
        # uint8 view first: torch.frombuffer has no fp8 support on every build.
        raw = torch.frombuffer(self._buf, dtype=torch.uint8, count=self._end - self._begin, offset=self._begin)
        return raw.view(self.dtype).view(self.shape)

    def tensor(self) -> torch.Tensor:
        return self._full()

    def slice_dim(self, dim: int, start: int, stop: int) -> torch.Tensor:
        full = self._full()
        if full.dim() == 0:
            return full
        return full.narrow(dim, start, max(0, stop - start))

    def __getitem__(self, idx):
        return self._full()[idx]


class SafetensorsFile:
    """Zero-copy safetensors reader over a file path or an in-memory blob."""

    def __init__(self, source: Union[str, os.PathLike, bytes, bytearray, memoryview]):
        self._file = None
        if isinstance(source, (bytes, bytearray, memoryview)):
            self._buf = bytearray(source) if not isinstance(source, bytearray) else source
            self.name = "<memory>"
        else:
            self.name = str(source)
            self._file = open(source, "rb")
            size = os.fstat(self._file.fileno()).st_size
            if size < 8:
                raise ValueError(f"{self.name}: not a safetensors file")
            # ACCESS_COPY gives a writable private mapping, which torch.frombuffer
            # accepts without a warning; pages stay shared until written (never).
            self._buf = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)
        (hlen,) = struct.unpack("<Q", bytes(self._buf[:8]))
        header = json.loads(bytes(self._buf[8 : 8 + hlen]).decode("utf-8"))
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: Dict[str, dict] = header

    def keys(self) -> List[str]:
        return list(self._entries.keys())

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def get_slice(self, name: str) -> TensorSlice:
        e = self._entries[name]
        b, en = e["data_offsets"]
        return TensorSlice(self._buf, _ST_DTYPES[e["dtype"]], e["shape"], self._base + b, self._base + en)

    def get_tensor(self, name: str) -> torch.Tensor:
        return self.get_slice(name).tensor()

    def close(self):
        if self._file is not None:
            try:
                self._buf.close()
            except (BufferError, ValueError):
                pass  # live tensor views keep the mapping open
            self._file.close()
            self._file = None


def serialize_safetensors(tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> bytes:
    """Serialise ``tensors`` in the safetensors layout (header JSON + raw little-endian data)."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = metadata
    chunks: List[bytes] = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    return struct.pack("<Q", len(hjson)) + hjson + b"".join(chunks)


def save_safetensors(tensors: Dict[str, torch.Tensor], path: Union[str, os.PathLike], metadata=None) -> None:
    with open(path, "wb") as f:
        f.write(serialize_safetensors(tensors, metadata))


class ProcessGroupView:
    """The two facts sharding needs from a process group."""

    def __init__(self, rank: int = 0, size: int = 1):
        self._rank, self._size = rank, size

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._size


def shard_bounds(total: int, rank: int, world: int, exact: bool = False) -> Tuple[int, int]:
    """``[start, stop)`` of ``rank``'s block when ``total`` rows are split in ``world`` ceil-div blocks."""
    if exact and total % world != 0:
        raise ValueError(f"size {total} is not divisible by the {world} shards")
    block = (total + world - 1) // world
    start = min(rank * block, total)
    return start, min(start + block, total)


class Weights:
    """Routing table over safetensors files plus tensor-parallel slicing."""

    def __init__(
        self,
        filenames: Iterable[Union[str, os.PathLike, bytes, SafetensorsFile]],
        device: Union[str, torch.device] = "cpu",
        dtype: torch.dtype = torch.float32,
        process_group=None,
        aliases: Optional[Dict[str, List[str]]] = None,
        prefix: Optional[str] = None,
        loader=None,
        renames: Optional[List[Tuple[str, str]]] = None,
    ):
        self._handles: List[SafetensorsFile] = []
        self.routing: Dict[str, int] = {}
        for src in filenames:
            h = src if isinstance(src, SafetensorsFile) else SafetensorsFile(src)
            idx = len(self._handles)
            self._handles.append(h)
            for k in h.keys():
                if k in self.routing:
                    raise RuntimeError(
                        f"tensor {k} is present in {self._handles[self.routing[k]].name} and {h.name}; "
                        "a checkpoint must hold each tensor once"
                    )
                self.routing[k] = idx
        self.aliases = aliases or {}
        # (old prefix, new prefix) pairs: a name that starts with the old prefix is also looked up under the
        # new one (checkpoints of one architecture published under different module layouts)
        self.renames = list(renames or [])
        self.device = torch.device(device)
        self.dtype = dtype
        self.process_group = process_group or ProcessGroupView()
        self.prefix = prefix
        if loader is None:
            from .quantization import DefaultWeightsLoader

            loader = DefaultWeightsLoader()
        self.weights_loader = loader
        # optional hook ``derive(weights, name) -> tensor or None`` for tensors a checkpoint stores in another form
        # (consulted by has_tensor / get_tensor when the name itself is absent)
        self.derive = None

    # -- lookup ---------------------------------------------------------------------
    def _candidates(self, name: str) -> List[str]:
        names = [name]
        if self.prefix:
            names.append(f"{self.prefix}.{name}")
        for old, new in self.renames:
            if name.startswith(old):
                names.append(new + name[len(old):])
        return names

    def resolve(self, name: str) -> Tuple[SafetensorsFile, str]:
        for cand in self._candidates(name):
            if cand in self.routing:
                return self._handles[self.routing[cand]], cand
        for cand in self._candidates(name):
            for alias in self.aliases.get(cand, []):
                if alias in self.routing:
                    return self._handles[self.routing[alias]], alias
        raise KeyError(f"weight {name} does not exist")

    def has_tensor(self, name: str) -> bool:
        try:
            self.resolve(name)
            return True
        except KeyError:
            return self.derive is not None and self.derive(self, name, probe=True) is not None

    def _slice(self, name: str) -> TensorSlice:
        h, real = self.resolve(name)
        return h.get_slice(real)

    def get_shape(self, name: str) -> Tuple[int, ...]:
        return self._slice(name).get_shape()

    # -- dtype/device policy --------------------------------------------------------
    def _finish(self, t: torch.Tensor, to_device: bool, to_dtype: bool) -> torch.Tensor:
        # Packed integer and fp8 payloads keep their storage type; everything
        # floating is brought to the serving dtype.
        src_ptr = t.data_ptr()
        if to_dtype and t.dtype in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            t = t.to(self.dtype)
        if to_device:
            t = t.to(self.device, non_blocking=False)
        if t.device.type == "cpu" and t.data_ptr() == src_ptr:
            # Still a view into the file mapping: detach it so the mapping can be closed.
            t = t.clone(memory_format=torch.contiguous_format)
        return t.contiguous()

    def get_tensor(self, name: str, to_device: bool = True, to_dtype: bool = True) -> torch.Tensor:
        if self.derive is not None:
            try:
                self.resolve(name)
            except KeyError:
                t = self.derive(self, name, probe=False)
                if t is not None:
                    return self._finish(t, to_device, to_dtype)
        return self._finish(self._slice(name).tensor(), to_device, to_dtype)

    # -- sharding -------------------------------------------------------------------
    def get_partial_sharded(self, name: str, dim: int, to_device=True, to_dtype=True) -> torch.Tensor:
        sl = self._slice(name)
        start, stop = shard_bounds(sl.get_shape()[dim], self.process_group.rank(), self.process_group.size())
        return self._finish(sl.slice_dim(dim, start, stop), to_device, to_dtype)

    def get_sharded(self, name: str, dim: int, to_device=True, to_dtype=True) -> torch.Tensor:
        size = self._slice(name).get_shape()[dim]
        world = self.process_group.size()
        if size % world != 0:
            raise ValueError(f"The choosen size {size} is not compatible with sharding on {world} shards")
        return self.get_partial_sharded(name, dim, to_device, to_dtype)

    def get_packed_sharded(
        self,
        name: str,
        dim: int,
        block_sizes: Union[int, Sequence[int]],
        to_device=True,
        to_dtype=True,
    ) -> torch.Tensor:
        """Shard a matrix that stores several logical matrices packed along ``dim``.

        ``block_sizes`` is either the number of equally sized parts or the list
        of part widths (only their proportions matter).  Every part is sharded
        on its own and the rank's pieces are concatenated, so that e.g. a packed
        ``[q|k|v]`` matrix gives each rank ``[q_r|k_r|v_r]``.
        """
        sl = self._slice(name)
        total = sl.get_shape()[dim]
        parts = _block_sizes(total, block_sizes)
        rank, world = self.process_group.rank(), self.process_group.size()
        pieces = []
        off = 0
        for width in parts:
            if width % world != 0:
                raise ValueError(f"packed block of {width} rows cannot be split across {world} shards")
            per = width // world
            pieces.append(sl.slice_dim(dim, off + rank * per, off + (rank + 1) * per))
            off += width
        return self._finish(torch.cat(pieces, dim=dim), to_device, to_dtype)

    # -- loader front ends ----------------------------------------------------------
    def get_weights(self, prefix: str):
        return self.weights_loader.get_weights(self, prefix)

    def get_weights_col_packed_qkv(self, prefix: str, num_heads: int, num_key_value_heads: int):
        return self.get_weights_col_packed(prefix, [num_heads, num_key_value_heads, num_key_value_heads])

    def get_weights_col_packed_gate_up(self, prefix: str):
        return self.get_weights_col_packed(prefix, 2)

    def get_weights_col_packed(self, prefix: str, block_sizes: Union[int, Sequence[int]]):
        return self.weights_loader.get_weights_col_packed(self, prefix, block_sizes)

    def get_weights_col(self, prefix: str):
        return self.weights_loader.get_weights_col(self, prefix)

    def get_multi_weights_col(self, prefixes: List[str], dim: int = 0):
        return self.weights_loader.get_multi_weights_col(self, prefixes, dim)

    def get_weights_row(self, prefix: str):
        return self.weights_loader.get_weights_row(self, prefix)

    @contextmanager
    def use_loader(self, loader):
        old = self.weights_loader
        self.weights_loader = loader
        try:
            yield
        finally:
            self.weights_loader = old

    def loader_config(self):
        return self.weights_loader

    def close(self):
        for h in self._handles:
            h.close()


def _block_sizes(total: int, block_sizes: Union[int, Sequence[int]]) -> List[int]:
    if isinstance(block_sizes, int):
        if total % block_sizes != 0:
            raise ValueError(f"cannot split {total} rows in {block_sizes} equal blocks")
        return [total // block_sizes] * block_sizes
    denom = sum(block_sizes)
    if total % denom != 0:
        raise ValueError(f"cannot split {total} rows in the proportions {list(block_sizes)}")
    unit = total // denom
    return [b * unit for b in block_sizes]


def weight_files(model_path: Union[str, os.PathLike], extension: str = ".safetensors") -> List[Path]:
    """Checkpoint shards of a local model directory, following ``*.index.json`` when present."""
    p = Path(model_path)
    if p.is_file():
        return [p]
    index = p / f"model{extension}.index.json"
    if index.exists():
        with open(index) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [p / n for n in names]
    files = sorted(f for f in p.glob(f"*{extension}") if not f.name.startswith("."))
    if not files:
        raise FileNotFoundError(f"no {extension} weights found in {p}")
    return files
