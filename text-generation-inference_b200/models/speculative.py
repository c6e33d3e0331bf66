"""Speculative heads: Medusa (v1 and v2 layouts) and the MLP speculator.

Reference: ``layers/medusa.py`` (``ResBlock``/``MedusaHead``/``MedusaModel`` ``:14-80``, the fused
``MedusaHeadV2`` ``:100-191``), ``layers/mlp.py`` (``MLPSpeculatorModel`` ``:63-170``,
``MLPSpeculatorHead`` ``:173-282``) and ``layers/speculative.py`` (dispatch on the speculator's
``config.json``).  A head maps the final hidden states ``[T, H]`` to speculative logits
``[T, n_heads, V]``; the sampler takes their argmax at the last accepted position as the next
step's draft tokens, and the next forward verifies them.

All heads are small dense layers evaluated on the rows that are sampled, so they run as plain
``ops.linear`` calls (the bf16 tcgen05 GEMM on CUDA tensors).
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import List, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..utils.weights import Weights, weight_files


class _ResBlock:
    """``x + silu(W x + b)``"""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor]):
        self.weight, self.bias = weight, bias

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return x + F.silu(ops.linear(x, self.weight, self.bias))


class MedusaV1:
    """Independent heads: ``n_layers`` residual blocks, then the head's own vocabulary projection."""

    def __init__(self, blocks: List[List[_ResBlock]], outs: List[torch.Tensor]):
        self.blocks, self.outs = blocks, outs
        self.n_heads = len(outs)

    @classmethod
    def load(cls, cfg: dict, weights: Weights, prefix: str = ""):
        blocks, outs = [], []
        n_layers = int(cfg.get("medusa_num_layers", 1))
        for h in range(int(cfg["medusa_num_heads"])):
            px = f"{prefix}{h}"
            blocks.append([_ResBlock(weights.get_tensor(f"{px}.{l}.linear.weight"),
                                     weights.get_tensor(f"{px}.{l}.linear.bias")) for l in range(n_layers)])
            outs.append(weights.get_tensor(f"{px}.{n_layers}.weight"))
        return cls(blocks, outs)

    def __call__(self, hidden: torch.Tensor, base_logits: torch.Tensor) -> torch.Tensor:
        res = []
        for blocks, out in zip(self.blocks, self.outs):
            x = hidden
            for b in blocks:
                x = b(x)
            res.append(ops.linear(x, out))
        return torch.stack(res, dim=1)


class MedusaV2:
    """Fused layout: one ``[n_heads * H, H]`` residual projection, then the *base* lm_head per head."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], n_heads: int, lm_head):
        self.weight, self.bias, self.n_heads, self.lm_head = weight, bias, n_heads, lm_head

    @classmethod
    def load(cls, cfg: dict, weights: Weights, lm_head, prefix: str = ""):
        n = int(cfg["medusa_num_heads"])
        ws = [weights.get_tensor(f"{prefix}{h}.0.linear.weight") for h in range(n)]
        bs = [weights.get_tensor(f"{prefix}{h}.0.linear.bias") for h in range(n)]
        return cls(torch.cat(ws, 0).contiguous(), torch.cat(bs, 0).contiguous(), n, lm_head)

    def __call__(self, hidden: torch.Tensor, base_logits: torch.Tensor) -> torch.Tensor:
        T, H = hidden.shape
        y = ops.linear(hidden, self.weight, self.bias).view(T, self.n_heads, H)
        y = hidden.unsqueeze(1) + F.silu(y)
        return self.lm_head(y.reshape(T * self.n_heads, H)).view(T, self.n_heads, -1)


class MLPSpeculator:
    """Recurrent MLP speculator: head ``i`` mixes the running state with the embedding of the token
    predicted by head ``i-1`` (head 0: the base model's greedy token)."""

    def __init__(self, emb, proj, ln_w, ln_b, heads, n_predict, emb_dim, inner_dim, scale_input, eps=1e-6):
        self.emb, self.proj, self.ln_w, self.ln_b, self.heads = emb, proj, ln_w, ln_b, heads
        self.n_heads = self.n_predict = n_predict
        self.scale_input = scale_input
        self.state_weight = 0.5 ** (0.5 / n_predict)
        self.emb_weight = math.sqrt((1 - self.state_weight ** 2) * (inner_dim / 2))
        self.eps = eps
        self.emb_dim, self.inner_dim = emb_dim, inner_dim

    @classmethod
    def load(cls, cfg: dict, weights: Weights, prefix: str = "speculator"):
        n = int(cfg["n_predict"])
        tie = bool(cfg.get("tie_weights", False))

        def pick(name, i):
            return weights.get_tensor(f"{prefix}.{name}.{0 if tie and name != 'proj' else i}.weight")

        emb = [pick("emb", i) for i in range(n)]
        proj = [weights.get_tensor(f"{prefix}.proj.{i if not tie else min(i, 1)}.weight") for i in range(n)]
        heads = [pick("head", i) for i in range(n)]
        ln_w = [weights.get_tensor(f"{prefix}.ln.{0 if tie else i}.weight") for i in range(n)]
        ln_b = [weights.get_tensor(f"{prefix}.ln.{0 if tie else i}.bias") for i in range(n)]
        inner = int(cfg.get("inner_dim") or cfg.get("speculator_width") or emb[0].shape[1])
        return cls(emb, proj, ln_w, ln_b, heads, n, int(cfg.get("emb_dim", proj[0].shape[1])), inner,
                   bool(cfg.get("scale_input", False)))

    def _ln(self, x, w, b):
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * w.float() + b.float()).to(x.dtype)

    def __call__(self, hidden: torch.Tensor, base_logits: torch.Tensor) -> torch.Tensor:
        state = hidden
        if self.scale_input:
            xf = state.float()
            state = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) / math.sqrt(2)).to(hidden.dtype)
        ids = base_logits.argmax(-1)
        out = []
        for i in range(self.n_predict):
            z = F.embedding(ids, self.emb[i])
            state = ops.linear(state, self.proj[i])
            state = torch.add(state.float() * self.state_weight, z.float(), alpha=self.emb_weight).to(hidden.dtype)
            state = F.gelu(self._ln(state, self.ln_w[i], self.ln_b[i]))
            logits = ops.linear(state, self.heads[i])
            out.append(logits)
            ids = logits.argmax(-1)
        return torch.stack(out, dim=1)


def find_speculator(model_path: Path) -> Optional[Path]:
    """Directory holding a speculator for ``model_path``: the model directory itself when it ships
    Medusa heads, or the ``speculator`` sub-directory / ``speculator.path`` named by its config."""
    model_path = Path(model_path)
    if (model_path / "medusa_lm_head.safetensors").exists():
        return model_path
    cfg_file = model_path / "config.json"
    if cfg_file.exists():
        cfg = json.loads(cfg_file.read_text())
        if cfg.get("model_type") == "mlp_speculator" or "medusa_num_heads" in cfg:
            return model_path
        spec = cfg.get("speculator")
        if isinstance(spec, dict) and spec.get("path"):
            p = Path(spec["path"])
            return p if p.is_absolute() else model_path / p
    sub = model_path / "speculator"
    return sub if sub.is_dir() else None


def load_speculator(spec_path: Path, device, dtype, process_group, lm_head):
    """Build the head described by ``spec_path/config.json``; returns ``(head, n_speculative_tokens)``."""
    spec_path = Path(spec_path)
    cfg = json.loads((spec_path / "config.json").read_text())
    if cfg.get("model_type") == "mlp_speculator":
        files = weight_files(spec_path)
        w = Weights(files, device, dtype, process_group=process_group)
        head = MLPSpeculator.load(cfg, w)
        w.close()
        return head, head.n_predict
    medusa_file = spec_path / "medusa_lm_head.safetensors"
    if not medusa_file.exists():
        raise FileNotFoundError(f"{medusa_file} not found: no speculator weights in {spec_path}")
    w = Weights([medusa_file], device, dtype, process_group=process_group)
    n_layers = int(cfg.get("medusa_num_layers", 1))
    has_own_out = w.has_tensor(f"0.{n_layers}.weight")
    head = MedusaV1.load(cfg, w) if has_own_out else MedusaV2.load(cfg, w, lm_head)
    w.close()
    return head, head.n_heads
