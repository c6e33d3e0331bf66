"""Offline GPTQ calibration: ``text-generation-server quantize MODEL_DIR OUT_DIR``.

Role of ``layers/gptq/quantize.py`` in the reference (1 026 lines around the original GPTQ code): run
calibration sequences through the model one decoder layer at a time, accumulate for every linear
layer the Hessian ``H = 2/n * sum x x^T`` of its inputs, quantise the weight columns left to right with
the optimal-brain-surgeon update (the error of each column is propagated to the columns not yet
quantised through the Cholesky factor of ``H^-1``), then write ``qweight / qzeros / scales / g_idx``
in the AutoGPTQ layout together with ``quantize_config.json``.

The model is instantiated through ``transformers`` (any decoder-only architecture whose blocks are
``nn.Linear`` based).  Calibration data: a text file given with ``dataset=...`` (one sample per
line), otherwise seeded random token sequences, because no dataset can be downloaded in an offline
deployment; random tokens still exercise every input channel, real text gives better Hessians.
"""
from __future__ import annotations

import json
import logging
import math
import shutil
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .weights import save_safetensors

log = logging.getLogger("tgi_b200.gptq")


class _Quantizer:
    """Asymmetric (or symmetric) min/max grid per output row (optionally per group of input columns)."""

    def __init__(self, bits: int, sym: bool):
        self.maxq = 2 ** bits - 1
        self.sym = sym
        self.scale = self.zero = None

    def find_params(self, w: torch.Tensor):           # w [rows, cols of the group]
        xmin = w.min(dim=1).values.clamp(max=0)
        xmax = w.max(dim=1).values.clamp(min=0)
        if self.sym:
            xmax = torch.maximum(xmin.abs(), xmax)
            xmin = -xmax
        dead = (xmin == 0) & (xmax == 0)
        xmin[dead], xmax[dead] = -1, 1
        self.scale = ((xmax - xmin) / self.maxq).unsqueeze(1)
        if self.sym:
            self.zero = torch.full_like(self.scale, (self.maxq + 1) / 2)
        else:
            self.zero = torch.round(-xmin.unsqueeze(1) / self.scale)

    def quantize(self, col: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        q = torch.clamp(torch.round(col / self.scale) + self.zero, 0, self.maxq)
        return self.scale * (q - self.zero), q


class GPTQ:
    """Hessian accumulator and solver of one linear layer (weight ``[out, in]``)."""

    def __init__(self, layer: nn.Linear):
        self.layer = layer
        self.rows, self.columns = layer.weight.shape
        self.H = torch.zeros(self.columns, self.columns, dtype=torch.float32, device=layer.weight.device)
        self.nsamples = 0

    def add_batch(self, inp: torch.Tensor):
        x = inp.reshape(-1, inp.shape[-1]).float().t()          # [in, tokens]
        n = x.shape[1]
        self.H *= self.nsamples / (self.nsamples + n)
        self.nsamples += n
        x = math.sqrt(2 / self.nsamples) * x
        self.H += x @ x.t()

    def fasterquant(self, bits: int, groupsize: int, act_order: bool, percdamp: float, sym: bool, blocksize: int = 128):
        """Returns ``(q_int [out, in], scales [groups, out], zeros [groups, out], g_idx [in])``; the
        layer's weight is replaced by its de-quantised value so later layers calibrate on it."""
        W = self.layer.weight.data.clone().float()
        H = self.H
        dead = torch.diag(H) == 0
        H[dead, dead] = 1
        W[:, dead] = 0
        perm = None
        if act_order:
            perm = torch.argsort(torch.diag(H), descending=True)
            W = W[:, perm]
            H = H[perm][:, perm]
        damp = percdamp * torch.mean(torch.diag(H))
        H = H + damp * torch.eye(self.columns, device=H.device)
        L = torch.linalg.cholesky(H)
        Hinv = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)
        quant = _Quantizer(bits, sym)
        gs = groupsize if groupsize > 0 else self.columns
        n_groups = (self.columns + gs - 1) // gs
        Q = torch.zeros_like(W)
        Qint = torch.zeros_like(W)
        scales = torch.zeros(n_groups, self.rows, device=W.device)
        zeros = torch.zeros(n_groups, self.rows, device=W.device)
        if groupsize <= 0:
            quant.find_params(W)
            scales[0], zeros[0] = quant.scale.squeeze(1), quant.zero.squeeze(1)
        for i1 in range(0, self.columns, blocksize):
            i2 = min(i1 + blocksize, self.columns)
            W1 = W[:, i1:i2].clone()
            Err1 = torch.zeros_like(W1)
            Hinv1 = Hinv[i1:i2, i1:i2]
            for i in range(i2 - i1):
                col = i1 + i
                if groupsize > 0 and col % gs == 0:
                    quant.find_params(W[:, col:col + gs])
                    scales[col // gs], zeros[col // gs] = quant.scale.squeeze(1), quant.zero.squeeze(1)
                w = W1[:, i]
                d = Hinv1[i, i]
                dq, qi = quant.quantize(w.unsqueeze(1))
                dq, qi = dq.squeeze(1), qi.squeeze(1)
                Q[:, col], Qint[:, col] = dq, qi
                err = (w - dq) / d
                W1[:, i:] -= err.unsqueeze(1) * Hinv1[i, i:].unsqueeze(0)
                Err1[:, i] = err
            W[:, i2:] -= Err1 @ Hinv[i1:i2, i2:]
        g_idx = torch.arange(self.columns, device=W.device) // gs
        if perm is not None:
            inv = torch.argsort(perm)
            Q, Qint = Q[:, inv], Qint[:, inv]
            g_idx = g_idx[inv]
        self.layer.weight.data = Q.to(self.layer.weight.dtype)
        return Qint.to(torch.int32), scales, zeros.to(torch.int32), g_idx.to(torch.int32)


def pack(qint: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, g_idx: torch.Tensor, bits: int) -> Dict[str, torch.Tensor]:
    """AutoGPTQ tensors of one layer: ``qweight [in*bits/32, out]`` packed along the input dimension,
    ``qzeros [groups, out*bits/32]`` holding ``zero - 1``, ``scales [groups, out]`` fp16, ``g_idx [in]``."""
    per = 32 // bits
    out_f, in_f = qint.shape
    assert in_f % per == 0 and out_f % per == 0, "feature sizes must be multiples of 32 / bits"
    w = qint.t().contiguous().to(torch.int64)                    # [in, out]
    shifts = (torch.arange(per, device=w.device, dtype=torch.int64) * bits).view(1, per, 1)
    qweight = (w.view(in_f // per, per, out_f) << shifts).sum(dim=1)
    z = (zeros.to(torch.int64) - 1) & (2 ** bits - 1)            # [groups, out]
    zshifts = (torch.arange(per, device=w.device, dtype=torch.int64) * bits).view(1, 1, per)
    qzeros = (z.view(z.shape[0], out_f // per, per) << zshifts).sum(dim=2)

    def to_i32(t):
        return torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)

    return {"qweight": to_i32(qweight).cpu().contiguous(), "qzeros": to_i32(qzeros).cpu().contiguous(),
            "scales": scales.to(torch.float16).cpu().contiguous(), "g_idx": g_idx.cpu().contiguous()}


def calibration_batches(tokenizer, vocab: int, nsamples: int, seqlen: int, seed: int, dataset: Optional[str]) -> List[torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    if dataset and Path(dataset).exists() and tokenizer is not None:
        lines = [l for l in Path(dataset).read_text().splitlines() if l.strip()]
        out = []
        for i in torch.randperm(len(lines), generator=g).tolist()[:nsamples]:
            ids = tokenizer(lines[i])["input_ids"][:seqlen]
            if len(ids) >= 2:
                out.append(torch.tensor([ids], dtype=torch.long))
        if out:
            return out
    return [torch.randint(3, vocab, (1, seqlen), generator=g) for _ in range(nsamples)]


def _decoder_layers(model: nn.Module) -> nn.ModuleList:
    best = None
    for _, m in model.named_modules():
        if isinstance(m, nn.ModuleList) and len(m) > 0 and (best is None or len(m) > len(best)):
            best = m
    if best is None:
        raise ValueError("could not find the list of decoder layers in this model")
    return best


def _name_of(model: nn.Module, target: nn.Module) -> str:
    for n, m in model.named_modules():
        if m is target:
            return n
    raise KeyError("module not found")


class _Stop(Exception):
    pass


@torch.no_grad()
def quantize(model_id: str, output_dir: str, bits: int = 4, groupsize: int = 128, act_order: bool = False,
             percdamp: float = 0.01, nsamples: int = 128, seed: int = 0, seqlen: int = 512, sym: bool = False,
             dataset: Optional[str] = None, device: Optional[str] = None, trust_remote_code: bool = False) -> Path:
    import transformers

    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    src = Path(model_id)
    model = transformers.AutoModelForCausalLM.from_pretrained(str(src), torch_dtype=torch.float32,
                                                              trust_remote_code=trust_remote_code).eval()
    try:
        tokenizer = transformers.AutoTokenizer.from_pretrained(str(src))
    except Exception:  # noqa: BLE001 - checkpoints without tokenizer files calibrate on random tokens
        tokenizer = None
    vocab = int(model.config.vocab_size)
    seqlen = min(seqlen, int(getattr(model.config, "max_position_embeddings", seqlen)))
    batches = calibration_batches(tokenizer, vocab, nsamples, seqlen, seed, dataset)
    layers = _decoder_layers(model)
    layer_prefix = _name_of(model, layers)

    # ---- capture the inputs of the first decoder layer -------------------------------------------
    captured: List[Tuple[tuple, dict]] = []

    class Catcher(nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, *args, **kwargs):
            captured.append((args, kwargs))
            raise _Stop()

    model.to(dev)
    layers[0] = Catcher(layers[0])
    for b in batches:
        try:
            model(b.to(dev), use_cache=False)
        except _Stop:
            pass
    layers[0] = layers[0].inner
    hidden = [a[0] for a, _ in captured]
    kwargs_list = [{k: v for k, v in kw.items() if k not in ("past_key_values", "past_key_value", "use_cache")}
                   for _, kw in captured]

    tensors: Dict[str, torch.Tensor] = {}
    for li, layer in enumerate(layers):
        linears = {n: m for n, m in layer.named_modules() if isinstance(m, nn.Linear)}
        solvers = {n: GPTQ(m) for n, m in linears.items()}
        hooks = [m.register_forward_hook(lambda mod, inp, out, n=n: solvers[n].add_batch(inp[0].detach()))
                 for n, m in linears.items()]
        for h, kw in zip(hidden, kwargs_list):
            layer(h, **kw)
        for hk in hooks:
            hk.remove()
        for n, solver in solvers.items():
            qint, scales, zeros, g_idx = solver.fasterquant(bits, groupsize, act_order, percdamp, sym)
            full = f"{layer_prefix}.{li}.{n}"
            for k, v in pack(qint, scales, zeros, g_idx, bits).items():
                tensors[f"{full}.{k}"] = v
            if linears[n].bias is not None:
                tensors[f"{full}.bias"] = linears[n].bias.detach().cpu().to(torch.float16)
            log.info("layer %d %s quantised (%d calibration tokens)", li, n, solver.nsamples)
        # outputs of the quantised layer are the next layer's calibration inputs
        new_hidden = []
        for h, kw in zip(hidden, kwargs_list):
            out = layer(h, **kw)
            new_hidden.append(out[0] if isinstance(out, (tuple, list)) else out)
        hidden = new_hidden

    # ---- everything that is not a quantised linear stays in half precision ---------------------------
    quantised = {k.rsplit(".", 1)[0] for k in tensors if k.endswith(".qweight")}
    for name, p in model.state_dict().items():
        base = name.rsplit(".", 1)[0]
        if base in quantised:
            continue
        tensors[name] = p.detach().cpu().to(torch.float16).contiguous()
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    save_safetensors(tensors, out / "model.safetensors", {"format": "pt"})
    cfg = json.loads((src / "config.json").read_text())
    qcfg = {"bits": bits, "group_size": groupsize, "desc_act": act_order, "sym": sym, "damp_percent": percdamp,
            "quant_method": "gptq", "checkpoint_format": "gptq", "true_sequential": True}
    cfg["quantization_config"] = qcfg
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    (out / "quantize_config.json").write_text(json.dumps(qcfg, indent=1))
    for extra in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json",
                  "generation_config.json", "vocab.json", "merges.txt"):
        if (src / extra).exists():
            shutil.copy(src / extra, out / extra)
    return out
