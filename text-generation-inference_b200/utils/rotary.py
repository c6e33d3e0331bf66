"""Rotary position embedding tables and their scaling variants.

The reference builds a ``PositionRotaryEmbedding`` object per model and selects
cos/sin rows per step (``server/text_generation_server/layers/rotary.py:34-80``
for the base class, ``:82-203`` for the ``rope_scaling`` dispatch, ``:289-602``
for linear / dynamic-NTK / YaRN / llama3 / su-longrope / mrope variants).

Here a variant is a pure function ``config -> inv_freq (and an amplitude
factor)``; the result is one fp32 table ``cos_sin[max_positions, rot_dim]``
(``cos`` in the first half of each row, ``sin`` in the second) that stays on the
device and is indexed by position *inside* the fused RoPE+KV-store kernel, so no
per-step gather is launched.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch


def _base_inv_freq(base: float, dim: int) -> torch.Tensor:
    return 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))


def _yarn_find_correction_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_linear_ramp(lo: float, hi: float, n: int) -> torch.Tensor:
    if lo == hi:
        hi += 0.001
    return ((torch.arange(n, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)


def _yarn_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def llama3_inv_freq(inv_freq: torch.Tensor, factor: float, low: float, high: float, original_max: int) -> torch.Tensor:
    """Llama-3.1 frequency-dependent scaling: long wavelengths are divided by ``factor``, short ones kept."""
    low_wavelen = original_max / low
    high_wavelen = original_max / high
    out = []
    for f in inv_freq.tolist():
        wavelen = 2 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / factor)
        else:
            smooth = (original_max / wavelen - low) / (high - low)
            out.append((1 - smooth) * f / factor + smooth * f)
    return torch.tensor(out, dtype=torch.float32)


class RotaryTable:
    """cos/sin table for one model.

    Attributes
    ----------
    rot_dim: number of rotated features per head (0 = no rotary embedding).
    neox: ``True`` pairs feature ``i`` with ``i + rot_dim/2`` (Llama/NeoX), ``False`` pairs ``2i, 2i+1`` (GPT-J).
    cos_sin: ``[max_positions, rot_dim]`` fp32.
    mrope_section: optional list for multimodal 3-axis RoPE (Qwen2-VL).
    """

    def __init__(self, cos_sin: torch.Tensor, rot_dim: int, neox: bool = True, mrope_section=None):
        self.cos_sin = cos_sin
        self.rot_dim = rot_dim
        self.neox = neox
        self.mrope_section = mrope_section

    def to(self, device) -> "RotaryTable":
        self.cos_sin = self.cos_sin.to(device)
        return self

    @staticmethod
    def _table(inv_freq: torch.Tensor, max_positions: int, position_scale: float = 1.0, mscale: float = 1.0):
        t = torch.arange(max_positions, dtype=torch.float32) / position_scale
        freqs = torch.outer(t, inv_freq)
        return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).contiguous()

    @classmethod
    def from_config(cls, config, dim: int, base: float, max_positions: int, neox: bool = True) -> "RotaryTable":
        """Build the table from an HF config (``rope_scaling`` / ``rope_parameters`` dict; env override
        ``ROPE_SCALING`` + ``ROPE_FACTOR`` as in ``layers/rotary.py:24-31``)."""
        if dim <= 0:
            return cls(torch.zeros(max_positions, 0), 0, neox)
        inv_freq = _base_inv_freq(base, dim)
        rs = getattr(config, "rope_scaling", None) or getattr(config, "rope_parameters", None)
        if isinstance(rs, dict) and isinstance(rs.get("full_attention"), dict):
            rs = rs["full_attention"]      # per-layer-type parameters (Gemma-3): the global layers' entry
        if (isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in (None, "default") and "factor" not in rs
                and "mrope_section" not in rs):
            rs = None
        env_type = os.environ.get("ROPE_SCALING")
        if env_type:
            rs = {"type": env_type, "factor": float(os.environ.get("ROPE_FACTOR", 1.0))}
        mrope_section = None
        position_scale, mscale = 1.0, 1.0
        if rs:
            kind = rs.get("rope_type", rs.get("type", "default"))
            factor = float(rs.get("factor", 1.0))
            orig_max = int(
                rs.get("original_max_position_embeddings")
                or getattr(config, "original_max_position_embeddings", None)
                or getattr(config, "max_position_embeddings", max_positions)
            )
            if kind in ("default", "mrope"):
                mrope_section = rs.get("mrope_section")
            elif kind == "linear":
                position_scale = factor
            elif kind == "dynamic":
                # NTK-aware: rescale the base once for the longest sequence the engine will serve.
                if max_positions > orig_max:
                    nb = base * ((factor * max_positions / orig_max) - (factor - 1)) ** (dim / (dim - 2))
                    inv_freq = _base_inv_freq(nb, dim)
            elif kind == "llama3":
                inv_freq = llama3_inv_freq(
                    inv_freq, factor, float(rs["low_freq_factor"]), float(rs["high_freq_factor"]), orig_max
                )
            elif kind == "yarn":
                beta_fast, beta_slow = float(rs.get("beta_fast", 32)), float(rs.get("beta_slow", 1))
                lo = max(math.floor(_yarn_find_correction_dim(beta_fast, dim, base, orig_max)), 0)
                hi = min(math.ceil(_yarn_find_correction_dim(beta_slow, dim, base, orig_max)), dim - 1)
                extrap = inv_freq
                interp = inv_freq / factor
                mask = 1 - _yarn_linear_ramp(lo, hi, dim // 2)
                inv_freq = interp * (1 - mask) + extrap * mask
                m_all = float(rs.get("mscale_all_dim", 0) or 0)
                m = float(rs.get("mscale", 1) or 1)
                if m_all:
                    mscale = _yarn_mscale(factor, m) / _yarn_mscale(factor, m_all)
                else:
                    mscale = float(rs.get("attention_factor") or _yarn_mscale(factor))
            elif kind in ("su", "longrope"):
                short = torch.tensor(rs["short_factor"], dtype=torch.float32)
                long = torch.tensor(rs["long_factor"], dtype=torch.float32)
                scale = getattr(config, "max_position_embeddings", max_positions) / orig_max
                mscale = 1.0 if scale <= 1.0 else math.sqrt(1 + math.log(scale) / math.log(orig_max))
                # Positions below the original window use the short factors, the rest the long ones.
                short_tab = cls._table(inv_freq / short, min(orig_max, max_positions), 1.0, mscale)
                if max_positions > orig_max:
                    long_tab = cls._table(inv_freq / long, max_positions, 1.0, mscale)
                    cos_sin = torch.cat([short_tab, long_tab[orig_max:]], dim=0)
                else:
                    cos_sin = short_tab
                return cls(cos_sin, dim, neox)
            else:
                raise NotImplementedError(f"rope scaling type {kind} is not implemented")
        return cls(cls._table(inv_freq, max_positions, position_scale, mscale), dim, neox, mrope_section)

    def mrope_rows(self, pos3: torch.Tensor) -> torch.Tensor:
        """Rows ``[T, rot_dim]`` for three position streams ``[3, T]`` (time, height, width): frequency ``d``
        follows the stream its ``mrope_section`` assigns it to (``layers/rotary.py:563-602`` in the reference)."""
        h = self.rot_dim // 2
        owner = torch.repeat_interleave(torch.arange(len(self.mrope_section)), torch.tensor(self.mrope_section))[:h]
        owner = torch.cat([owner, owner]).to(self.cos_sin.device)                    # cos half, sin half
        rows = self.cos_sin[pos3.long()]                                              # [3, T, rot_dim]
        return torch.gather(rows, 0, owner.view(1, 1, -1).expand(1, rows.shape[1], -1))[0].contiguous()

    def lookup(self, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        cs = self.cos_sin[positions.long()]
        h = self.rot_dim // 2
        return cs[..., :h], cs[..., h:]
