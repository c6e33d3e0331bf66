"""Locating, downloading and converting model weights.

Role of the reference's ``utils/hub.py`` + ``utils/convert.py`` + the ``download-weights`` command
(``cli.py:134-335``): resolve a model id to local files (a directory, or the Hugging Face cache in
offline mode), prefer safetensors, convert ``*.bin`` / ``*.pt`` checkpoints once (de-duplicating
tensors that share storage), optionally merge a PEFT adapter into its base model first.
Serving never touches the network: anything not found locally is an error that says what to fetch.
"""
from __future__ import annotations

import json
import logging
import os
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional

import torch

from .weights import save_safetensors

log = logging.getLogger("tgi_b200.hub")
WEIGHTS_CACHE_OVERRIDE = os.environ.get("WEIGHTS_CACHE_OVERRIDE")
HF_HUB_OFFLINE = os.environ.get("HF_HUB_OFFLINE", "1") in ("1", "ON", "true")


class LocalEntryNotFoundError(FileNotFoundError):
    pass


def resolve_model_path(model_id: str, revision: Optional[str] = None) -> Path:
    """Directory holding ``config.json`` for ``model_id``: a local path, ``WEIGHTS_CACHE_OVERRIDE``,
    or the snapshot directory of the Hugging Face cache."""
    p = Path(model_id)
    if p.is_dir():
        return p
    if WEIGHTS_CACHE_OVERRIDE and Path(WEIGHTS_CACHE_OVERRIDE).is_dir():
        return Path(WEIGHTS_CACHE_OVERRIDE)
    cache = Path(os.environ.get("HUGGINGFACE_HUB_CACHE", os.environ.get("HF_HOME", Path.home() / ".cache/huggingface") ) )
    cache = cache / "hub" if (cache / "hub").is_dir() else cache
    repo = cache / ("models--" + model_id.replace("/", "--"))
    if repo.is_dir():
        rev = revision
        ref = repo / "refs" / (revision or "main")
        if ref.exists():
            rev = ref.read_text().strip()
        snaps = repo / "snapshots"
        if rev and (snaps / rev).is_dir():
            return snaps / rev
        if snaps.is_dir():
            cands = sorted(snaps.iterdir())
            if cands:
                return cands[-1]
    raise LocalEntryNotFoundError(
        f"Model {model_id} is not available locally. Download it first (e.g. `huggingface-cli download {model_id}`) "
        "or pass a directory.")


def weight_files_local(model_id: str, revision: Optional[str] = None, extension: str = ".safetensors") -> List[Path]:
    root = resolve_model_path(model_id, revision)
    files = sorted(f for f in root.glob(f"*{extension}")
                   if not any(x in f.name for x in ("arguments", "args", "training", "optimizer", "scheduler")))
    if not files:
        raise LocalEntryNotFoundError(f"No local weights found in {root} with extension {extension}")
    return files


def _remove_shared_pointers(tensors: Dict[str, torch.Tensor]) -> List[str]:
    """Names that alias the storage of another tensor (tied weights); the first name is kept."""
    by_ptr = defaultdict(list)
    for k, v in tensors.items():
        by_ptr[(v.untyped_storage().data_ptr(), v.storage_offset(), tuple(v.shape))].append(k)
    dropped = []
    for names in by_ptr.values():
        for n in sorted(names)[1:]:
            dropped.append(n)
    return dropped


def convert_file(pt_file: Path, sf_file: Path, discard_names: Optional[List[str]] = None) -> None:
    """Convert one pickle checkpoint to safetensors and verify the round trip."""
    loaded = torch.load(pt_file, map_location="cpu", weights_only=True)
    if "state_dict" in loaded:
        loaded = loaded["state_dict"]
    drop = set(_remove_shared_pointers(loaded)) | set(discard_names or [])
    out = {k: v.contiguous() for k, v in loaded.items() if k not in drop}
    sf_file.parent.mkdir(parents=True, exist_ok=True)
    save_safetensors(out, sf_file, {"format": "pt"})
    from .weights import SafetensorsFile

    back = SafetensorsFile(sf_file)
    for k, v in out.items():
        if not torch.equal(v, back.get_tensor(k)):
            raise RuntimeError(f"The output tensors do not match for key {k}")
    back.close()


def convert_files(pt_files: List[Path], sf_files: List[Path], discard_names: Optional[List[str]] = None) -> None:
    assert len(pt_files) == len(sf_files)
    for i, (pt, sf) in enumerate(zip(pt_files, sf_files)):
        if any(x in pt.name for x in ("arguments", "args", "training")):
            continue
        log.info("Convert: [%d/%d] %s", i + 1, len(pt_files), pt.name)
        convert_file(pt, sf, discard_names)


def download_weights(model_id: str, revision: Optional[str] = None, extension: str = ".safetensors",
                     auto_convert: bool = True, merge_lora: bool = False) -> List[Path]:
    """Make sure safetensors weights of ``model_id`` exist locally; convert ``.bin`` files if needed."""
    root = resolve_model_path(model_id, revision)
    if merge_lora and (root / "adapter_config.json").exists():
        from .peft import merge_and_unload

        merge_and_unload(root)
    try:
        files = weight_files_local(str(root), revision, extension)
        log.info("Files are already present on the host. Skipping download.")
        return files
    except LocalEntryNotFoundError:
        pass
    if extension != ".safetensors" or not auto_convert:
        raise LocalEntryNotFoundError(f"No {extension} weights in {root}; network downloads are disabled in this build")
    pt_files = sorted(list(root.glob("*.bin")) + list(root.glob("*.pt")))
    pt_files = [f for f in pt_files if "training" not in f.name and "optimizer" not in f.name]
    if not pt_files:
        raise LocalEntryNotFoundError(f"No weights found in {root}")
    discard = []
    cfg = root / "config.json"
    if cfg.exists():
        c = json.loads(cfg.read_text())
        if c.get("tie_word_embeddings"):
            discard = ["lm_head.weight"]
    sf_files = [f.with_suffix(".safetensors") for f in pt_files]
    convert_files(pt_files, sf_files, discard)
    return sf_files
