"""Merging a LoRA (PEFT) adapter checkpoint into its base model on disk (``download-weights --merge-lora``).

The reference uses the ``peft`` package for this (``utils/peft.py``); the merge itself is the
identity ``W <- W + (alpha / r) * B @ A`` per adapted linear, done here directly on safetensors.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .weights import SafetensorsFile, save_safetensors, weight_files


def merge_and_unload(adapter_dir: Path, base_dir: Path = None, out_dir: Path = None) -> Path:
    adapter_dir = Path(adapter_dir)
    cfg = json.loads((adapter_dir / "adapter_config.json").read_text())
    base_dir = Path(base_dir or cfg["base_model_name_or_path"])
    out_dir = Path(out_dir or adapter_dir)
    scale = cfg.get("lora_alpha", cfg["r"]) / cfg["r"]
    ad_file = adapter_dir / "adapter_model.safetensors"
    ad = SafetensorsFile(ad_file)
    lora = {}
    for k in ad.keys():
        name = k.replace("base_model.model.", "")
        if ".lora_A" in name:
            lora.setdefault(name.split(".lora_A")[0], {})["A"] = ad.get_tensor(k).float()
        elif ".lora_B" in name:
            lora.setdefault(name.split(".lora_B")[0], {})["B"] = ad.get_tensor(k).float()
    merged = {}
    for f in weight_files(base_dir):
        h = SafetensorsFile(f)
        for k in h.keys():
            t = h.get_tensor(k).clone()
            mod = k[: -len(".weight")] if k.endswith(".weight") else None
            if mod in lora and "A" in lora[mod] and "B" in lora[mod]:
                delta = (lora[mod]["B"] @ lora[mod]["A"]) * scale
                if cfg.get("fan_in_fan_out"):
                    delta = delta.t()
                t = (t.float() + delta).to(t.dtype)
            merged[k] = t
        h.close()
    out_dir.mkdir(parents=True, exist_ok=True)
    save_safetensors(merged, out_dir / "model.safetensors", {"format": "pt"})
    for extra in ("config.json", "tokenizer.json", "tokenizer_config.json", "generation_config.json"):
        src = base_dir / extra
        if src.exists() and not (out_dir / extra).exists():
            (out_dir / extra).write_bytes(src.read_bytes())
    return out_dir
