"""Next-token selection, stopping criteria, top-n tokens and n-gram speculation.

What the reference spreads over ``utils/tokens.py`` (``HeterogeneousNextTokenChooser``
``:233-503``, ``StoppingCriteria`` ``:131-206``, ``batch_top_tokens`` ``:567-645``,
``create_n_gram_speculation`` ``:209-230``) and the per-warper classes of
``utils/logits_process.py`` is one batch object here, ``NextTokenChooser``:

* the sampling parameters of all requests of the batch are a struct of arrays
  on the device; a parameter's neutral value (temperature 1, top_k 0, top_p 1,
  typical_p 1, penalties 1 / 0) disables that stage for the row, so filtering or
  concatenating a batch is an ``index_select``/``cat`` over a few tensors;
* the order of stages is the reference's: watermark, repetition penalty,
  frequency penalty, grammar mask, temperature, top-k, top-p, typical-p, choice,
  then ``log_softmax`` of the warped scores for the reported log-probabilities;
* sampling draws ``argmax(p / E)`` with ``E ~ Exp(1)`` from a per-request seeded
  generator, so a request's tokens depend only on its own seed, whatever batch it
  shares a step with;
* on CUDA the stages run as the fused sampling kernels of ``ops`` when every
  row's configuration is supported by them.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch

from ..proto import generate_v3 as pb
from .grammar import GrammarBatch
from .watermark import WatermarkProcessor


class Sampling:
    """Seeded multinomial choice for one request (used by the per-request CPU path and by tests)."""

    def __init__(self, seed: int, device="cpu"):
        self.generator = torch.Generator(device)
        self.generator.manual_seed(seed)
        self.seed = seed

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        probs = torch.softmax(logits.float(), -1)
        q = torch.empty_like(probs).exponential_(1, generator=self.generator)
        return probs.div_(q).argmax(-1)


class Greedy:
    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        return logits.argmax(-1)


def apply_repetition_penalty(scores: torch.Tensor, input_ids: torch.Tensor, penalty: torch.Tensor) -> torch.Tensor:
    """``score <- score*p`` if negative else ``score/p`` for every token present in ``input_ids[B,S]``."""
    ids = input_ids.long()
    s = scores.gather(1, ids)
    p = penalty.view(-1, 1).to(scores.dtype)
    s = torch.where(s < 0, s * p, s / p)
    return scores.scatter(1, ids, s)


def apply_frequency_penalty(scores: torch.Tensor, input_ids: torch.Tensor, penalty: torch.Tensor) -> torch.Tensor:
    """Subtract ``penalty * count(token)`` (count over ``input_ids``) divided by the vocabulary-independent 1."""
    ids = input_ids.long()
    B, S = ids.shape
    counts = torch.zeros_like(scores)
    counts.scatter_add_(1, ids, torch.ones(B, S, dtype=scores.dtype, device=scores.device))
    return scores - counts * penalty.view(-1, 1).to(scores.dtype)


def top_k_filter(scores: torch.Tensor, top_k: torch.Tensor) -> torch.Tensor:
    """Keep each row's ``top_k[b]`` largest scores (0 disables the row)."""
    V = scores.shape[-1]
    kmax = int(min(max(int(top_k.max().item()), 1), V))
    kth_idx = (top_k.clamp(min=1, max=kmax) - 1).long().view(-1, 1)
    kth = torch.topk(scores, kmax, dim=-1)[0].gather(1, kth_idx)
    kth = kth.masked_fill((top_k == 0).view(-1, 1), -math.inf)
    return scores.masked_fill(scores < kth, -math.inf)


def top_p_filter(scores: torch.Tensor, top_p: torch.Tensor) -> torch.Tensor:
    """Nucleus filtering: drop the low-probability tail whose cumulative mass is ``<= 1 - top_p``."""
    sorted_logits, sorted_idx = torch.sort(scores, descending=False, dim=-1)
    cum = sorted_logits.softmax(-1).cumsum(-1)
    remove = cum <= (1 - top_p).view(-1, 1).to(cum.dtype)
    remove[..., -1:] = False
    remove = remove.scatter(1, sorted_idx, remove)
    return scores.masked_fill(remove, -math.inf)


def typical_p_filter(scores: torch.Tensor, mass: torch.Tensor) -> torch.Tensor:
    """Typical decoding (arXiv:2202.00666): keep tokens whose surprise is closest to the entropy."""
    normalized = torch.log_softmax(scores, dim=-1)
    p = normalized.exp()
    ent = -(normalized * p).nansum(-1, keepdim=True)
    shifted = ((-normalized) - ent).abs()
    sorted_scores, sorted_idx = torch.sort(shifted, descending=False, dim=-1)
    sorted_logits = scores.gather(-1, sorted_idx)
    cum = sorted_logits.softmax(-1).cumsum(-1)
    last = (cum < mass.view(-1, 1).to(cum.dtype)).sum(dim=1).clamp(min=0, max=scores.shape[-1] - 1)
    last = torch.where(mass >= 1.0, torch.full_like(last, scores.shape[-1] - 1), last)
    remove = sorted_scores > sorted_scores.gather(1, last.view(-1, 1))
    remove = remove.scatter(1, sorted_idx, remove)
    return scores.masked_fill(remove, -math.inf)


class NextTokenChooser:
    """Sampling state of a whole batch."""

    def __init__(
        self,
        device,
        watermark: List[bool],
        temperature: List[float],
        repetition_penalty: List[float],
        frequency_penalty: List[float],
        top_k: List[int],
        top_p: List[float],
        typical_p: List[float],
        do_sample: List[bool],
        seeds: List[int],
        tokenizer=None,
        grammars: Optional[List[str]] = None,
        grammar_types: Optional[List[int]] = None,
        fsm_grammar_states: Optional[List[int]] = None,
        steps: Optional[List[int]] = None,
    ):
        n = len(temperature)
        self.device = torch.device(device)
        self.n = n
        # A stage that is configured away from neutral turns sampling on for that row.
        self.do_sample_list = [
            bool(s) or t != 1.0 or k != 0 or p < 1.0 or ty < 1.0
            for s, t, k, p, ty in zip(do_sample, temperature, top_k, top_p, typical_p)
        ]
        self.lists = dict(
            watermark=list(watermark), temperature=list(temperature), repetition_penalty=list(repetition_penalty),
            frequency_penalty=list(frequency_penalty), top_k=list(top_k), top_p=list(top_p),
            typical_p=list(typical_p), seeds=list(seeds),
        )
        self.seeds = list(seeds)
        self.tokenizer = tokenizer
        self.grammars = list(grammars) if grammars is not None else [""] * n
        self.grammar_types = list(grammar_types) if grammar_types is not None else [0] * n
        self.fsm_grammar_states = list(fsm_grammar_states) if fsm_grammar_states is not None else [0] * n
        self.generators: List[Optional[torch.Generator]] = []
        for s, flag in zip(seeds, self.do_sample_list):
            if flag:
                g = torch.Generator("cpu")
                g.manual_seed(int(s) & 0x7FFFFFFFFFFFFFFF)
                self.generators.append(g)
            else:
                self.generators.append(None)
        self.steps = list(steps) if steps is not None else [0] * n
        self._build_tensors()
        self.watermarks: Dict[int, WatermarkProcessor] = {
            i: WatermarkProcessor(device=self.device) for i, w in enumerate(watermark) if w
        }
        self.grammar = (
            GrammarBatch(tokenizer, self.device, self.grammars, self.grammar_types)
            if any(g != "" for g in self.grammars) else None
        )

    def _build_tensors(self):
        L, dev = self.lists, self.device
        f = lambda name: torch.tensor(L[name], dtype=torch.float32, device=dev)
        self.temperature = f("temperature")
        self.repetition_penalty = f("repetition_penalty")
        self.frequency_penalty = f("frequency_penalty")
        self.top_p = f("top_p")
        self.typical_p = f("typical_p")
        self.top_k = torch.tensor(L["top_k"], dtype=torch.int32, device=dev)
        self.do_sample = torch.tensor(self.do_sample_list, dtype=torch.bool, device=dev)
        self.any_temperature = any(x != 1.0 for x in L["temperature"])
        self.any_rep = any(x != 1.0 for x in L["repetition_penalty"])
        self.any_freq = any(x != 0.0 for x in L["frequency_penalty"])
        self.any_top_k = any(x != 0 for x in L["top_k"])
        self.any_top_p = any(x < 1.0 for x in L["top_p"])
        self.any_typical = any(x < 1.0 for x in L["typical_p"])
        self.any_sample = any(self.do_sample_list)

    # ------------------------------------------------------------------------------------------
    @property
    def is_greedy_plain(self) -> bool:
        """No stage changes the scores and every row takes the argmax (fast path: fused argmax+logprob)."""
        return not (self.any_sample or self.any_rep or self.any_freq or self.watermarks or self.grammar)

    def warp(self, input_ids: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
        """All score-modifying stages for one position; ``scores[B,V]`` float32."""
        for i, wm in self.watermarks.items():
            scores[i : i + 1] = wm(input_ids[i : i + 1], scores[i : i + 1])
        if self.any_rep:
            scores = apply_repetition_penalty(scores, input_ids, self.repetition_penalty)
        if self.any_freq:
            scores = apply_frequency_penalty(scores, input_ids, self.frequency_penalty)
        if self.grammar is not None:
            scores = self.grammar.mask(scores, self.fsm_grammar_states)
        if self.any_temperature:
            scores = scores / self.temperature.view(-1, 1)
        if self.any_top_k:
            scores = top_k_filter(scores, self.top_k)
        if self.any_top_p:
            scores = top_p_filter(scores, self.top_p)
        if self.any_typical:
            scores = typical_p_filter(scores, self.typical_p)
        return scores

    def choose(self, scores: torch.Tensor) -> torch.Tensor:
        out = scores.argmax(-1)
        if self.any_sample:
            probs = torch.softmax(scores, -1)
            for i, g in enumerate(self.generators):
                if g is None:
                    continue
                row = probs[i].cpu() if probs.is_cuda else probs[i]
                q = torch.empty_like(row).exponential_(1, generator=g)
                out[i] = row.div(q).argmax(-1)
        return out

    def __call__(
        self,
        input_ids: torch.Tensor,
        scores: torch.Tensor,
        speculate: int = 0,
        speculated_ids: Optional[torch.Tensor] = None,
        speculative_scores: Optional[torch.Tensor] = None,
        need_logprobs: bool = True,
    ):
        """Returns ``(next_ids, next_logprobs, all_logprobs, accepted_ids, speculative_ids)``.

        ``need_logprobs=False`` tells the chooser that the caller will not read ``all_logprobs`` (no
        top-n tokens requested); on CUDA tensors the warpers and the sampling then run as one kernel
        and ``all_logprobs`` is ``None``.

        ``scores`` has ``B*(S)`` rows, ``S = 1 + speculated_ids.shape[1]``; ``input_ids[B, L]`` is the
        token history used by the penalties (padding rows with id 0 as the reference does).
        """
        S = 1 if speculated_ids is None else speculated_ids.shape[1] + 1
        B = scores.shape[0] // S
        if S == 1 and not need_logprobs and speculate == 0 and speculative_scores is None and scores.is_cuda:
            from .. import ops

            if ops.has_fused_sample(scores):
                return self._fused(input_ids, scores)
        scores = scores.float().view(B, S, -1)
        next_ids = torch.zeros(B, S, dtype=torch.long, device=scores.device)
        for j in range(S):
            sj = self.warp(input_ids, scores[:, j].clone())
            scores[:, j] = sj
            next_ids[:, j] = self.choose(sj)
        next_ids = next_ids.view(B * S)
        all_logprobs = torch.log_softmax(scores.view(B * S, -1), -1)
        if speculated_ids is not None:
            nl = next_ids.view(B, S).tolist()
            sl = speculated_ids.tolist()
            indices, accepted = [], []
            for i in range(B):
                acc = 1
                indices.append(i * S)
                for j in range(S - 1):
                    if nl[i][j] == sl[i][j]:
                        acc += 1
                        indices.append(i * S + j + 1)
                    else:
                        break
                accepted.append(acc)
            accepted_ids = torch.tensor(accepted, dtype=torch.long, device=scores.device)
            idx = torch.tensor(indices, dtype=torch.long, device=scores.device)
            next_ids = next_ids[idx]
            logprobs = all_logprobs[idx]
            if speculative_scores is not None:
                base = torch.arange(B, device=scores.device) * S
                speculative_scores = speculative_scores[base + accepted_ids - 1]
        else:
            accepted_ids = torch.ones_like(next_ids)
            logprobs = all_logprobs
        next_logprobs = logprobs.gather(1, next_ids.view(-1, 1)).view(-1)
        speculative_ids = None
        if speculate > 0:
            if speculative_scores is not None:
                speculative_ids = speculative_scores.argmax(-1)
            else:
                speculative_ids = create_n_gram_speculation(input_ids, next_ids, accepted_ids, speculate)
        return next_ids, next_logprobs, all_logprobs, accepted_ids, speculative_ids

    def _fused(self, input_ids: torch.Tensor, scores: torch.Tensor):
        """CUDA fast path: stages that need the token history or an automaton run in torch on a float
        copy (only when active), then temperature / top-k / top-p / typical-p / sampling / log-probability are
        one kernel launch for the whole batch (``ops.fused_sample``)."""
        from .. import ops

        if (self.any_rep or self.any_freq) and not self.watermarks and self.grammar is None and hasattr(ops, "penalties"):
            # penalties from the token history in one kernel (fp32 copy of the scores)
            scores = ops.penalties(scores, input_ids, self.repetition_penalty if self.any_rep else None,
                                   self.frequency_penalty if self.any_freq else None)
        elif self.watermarks or self.any_rep or self.any_freq or self.grammar is not None:
            scores = scores.float().clone()
            for i, wm in self.watermarks.items():
                scores[i : i + 1] = wm(input_ids[i : i + 1], scores[i : i + 1])
            if self.any_rep:
                scores = apply_repetition_penalty(scores, input_ids, self.repetition_penalty)
            if self.any_freq:
                scores = apply_frequency_penalty(scores, input_ids, self.frequency_penalty)
            if self.grammar is not None:
                scores = self.grammar.mask(scores, self.fsm_grammar_states)
        elif scores.dtype not in (torch.float32, torch.bfloat16):
            scores = scores.float()
        dev = scores.device
        seeds = steps = do_sample = None
        if self.any_sample:
            do_sample = self.do_sample.to(torch.uint8)
            seeds = torch.tensor([int(s or 0) & 0x7FFFFFFFFFFFFFFF for s in self.seeds], dtype=torch.int64, device=dev)
            steps = torch.tensor(self.steps, dtype=torch.int32, device=dev)
            self.steps = [st + (1 if d else 0) for st, d in zip(self.steps, self.do_sample_list)]
        next_ids, next_logprobs = ops.fused_sample(
            scores, self.temperature if self.any_temperature else None, self.top_k if self.any_top_k else None,
            self.top_p if self.any_top_p else None, do_sample, seeds, steps,
            typical_p=self.typical_p if self.any_typical else None)
        return next_ids, next_logprobs, None, torch.ones_like(next_ids), None

    def advance_grammar(self, next_ids: List[int]):
        if self.grammar is not None:
            self.fsm_grammar_states = self.grammar.advance_batch(next_ids, self.fsm_grammar_states)
        return self

    def advance_grammar_single(self, idx: int, next_id: int):
        if self.grammar is not None:
            self.fsm_grammar_states[idx] = self.grammar.advance_at_index(next_id, self.fsm_grammar_states[idx], idx)
        return self

    # ------------------------------------------------------------------------------------------
    def select(self, indices: List[int]) -> "NextTokenChooser":
        """A chooser over a subset of rows that shares generators and grammar automata with ``self``."""
        out = self.__class__.__new__(self.__class__)
        out.device, out.tokenizer = self.device, self.tokenizer
        out.lists = {k: [v[i] for i in indices] for k, v in self.lists.items()}
        out.seeds = [self.seeds[i] for i in indices]
        out.do_sample_list = [self.do_sample_list[i] for i in indices]
        out.generators = [self.generators[i] for i in indices]
        out.steps = [self.steps[i] for i in indices]
        out.grammars = [self.grammars[i] for i in indices]
        out.grammar_types = [self.grammar_types[i] for i in indices]
        out.fsm_grammar_states = [self.fsm_grammar_states[i] for i in indices]
        out.watermarks = {new: self.watermarks[old] for new, old in enumerate(indices) if old in self.watermarks}
        out.n = len(indices)
        out._build_tensors()
        out.grammar = None
        if self.grammar is not None:
            import copy

            g = copy.copy(self.grammar)
            g.fsms = [self.grammar.fsms[i] for i in indices]
            out.grammar = g if any(f is not None for f in g.fsms) else None
        return out

    def filter(self, indices: List[int]) -> "NextTokenChooser":
        for k, v in self.lists.items():
            self.lists[k] = [v[i] for i in indices]
        self.seeds = [self.seeds[i] for i in indices]
        self.do_sample_list = [self.do_sample_list[i] for i in indices]
        self.generators = [self.generators[i] for i in indices]
        self.steps = [self.steps[i] for i in indices]
        self.grammars = [self.grammars[i] for i in indices]
        self.grammar_types = [self.grammar_types[i] for i in indices]
        self.fsm_grammar_states = [self.fsm_grammar_states[i] for i in indices]
        self.watermarks = {new: self.watermarks[old] for new, old in enumerate(indices) if old in self.watermarks}
        self.n = len(indices)
        self._build_tensors()
        if self.grammar is not None:
            self.grammar = self.grammar.filter(indices)
        return self

    @classmethod
    def concatenate(cls, choosers: Sequence["NextTokenChooser"]) -> "NextTokenChooser":
        first = choosers[0]
        out = cls.__new__(cls)
        out.device, out.tokenizer = first.device, first.tokenizer
        out.lists = {k: sum((c.lists[k] for c in choosers), []) for k in first.lists}
        out.seeds = sum((c.seeds for c in choosers), [])
        out.do_sample_list = sum((c.do_sample_list for c in choosers), [])
        out.generators = sum((c.generators for c in choosers), [])
        out.steps = sum((c.steps for c in choosers), [])
        out.grammars = sum((c.grammars for c in choosers), [])
        out.grammar_types = sum((c.grammar_types for c in choosers), [])
        out.fsm_grammar_states = sum((c.fsm_grammar_states for c in choosers), [])
        out.watermarks = {}
        off = 0
        for c in choosers:
            for i, w in c.watermarks.items():
                out.watermarks[off + i] = w
            off += c.n
        out.n = off
        out._build_tensors()
        out.grammar = (
            GrammarBatch(out.tokenizer, out.device, out.grammars, out.grammar_types)
            if any(g != "" for g in out.grammars) else None
        )
        return out

    @classmethod
    def from_pb(cls, params: Sequence, device, tokenizer=None, fsm_grammar_states: Optional[List[int]] = None):
        return cls(
            device=device,
            watermark=[p.watermark for p in params],
            temperature=[p.temperature if p.temperature > 0 else 1.0 for p in params],
            repetition_penalty=[p.repetition_penalty if p.repetition_penalty > 0 else 1.0 for p in params],
            frequency_penalty=[p.frequency_penalty for p in params],
            top_k=[p.top_k for p in params],
            top_p=[p.top_p if p.top_p > 0 else 1.0 for p in params],
            typical_p=[p.typical_p if p.typical_p > 0 else 1.0 for p in params],
            do_sample=[p.do_sample for p in params],
            seeds=[p.seed for p in params],
            tokenizer=tokenizer,
            grammars=[p.grammar for p in params],
            grammar_types=[p.grammar_type for p in params],
            fsm_grammar_states=fsm_grammar_states if fsm_grammar_states else [0] * len(params),
        )


def create_n_gram_speculation(input_ids: torch.Tensor, next_ids: torch.Tensor, accepted_ids: torch.Tensor,
                              speculate: int) -> torch.Tensor:
    """Propose ``speculate`` tokens per row: find the last accepted token earlier in the row's history
    and copy what followed it there (prompt-lookup decoding)."""
    B = accepted_ids.shape[0]
    cum = accepted_ids.cumsum(0) - 1  # index in next_ids of every row's last accepted token
    seeds = next_ids[cum]
    hit = input_ids == seeds.view(-1, 1)
    first = hit.float().argmax(dim=1)  # first occurrence (0 when there is none, like the reference)
    idx = (first.view(-1, 1) + torch.arange(1, speculate + 1, device=input_ids.device)).clamp(max=input_ids.shape[1] - 1)
    return input_ids.gather(1, idx)


# ---------------------------------------------------------------------------------------------
class StopSequenceCriteria:
    def __init__(self, stop_sequence: str):
        self.regex = re.compile(re.escape(stop_sequence) + "$")

    def __call__(self, output: str) -> bool:
        return self.regex.search(output) is not None


class StoppingCriteria:
    def __init__(self, eos_token_ids: Optional[Set[int]], stop_sequence_criterias: List[StopSequenceCriteria],
                 max_new_tokens: int = 20, ignore_eos_token: bool = False):
        if eos_token_ids is None:
            eos_token_ids = set()
        elif isinstance(eos_token_ids, int):
            eos_token_ids = {eos_token_ids}
        self.eos_token_ids = set(eos_token_ids)
        self.stop_sequence_criterias = stop_sequence_criterias
        self.max_new_tokens = max_new_tokens
        self.current_tokens = 0
        self.current_output = ""
        self.ignore_eos_token = ignore_eos_token

    def __call__(self, last_token: int, last_output: str) -> Tuple[bool, Optional[int]]:
        self.current_tokens += 1
        if self.current_tokens >= self.max_new_tokens:
            return True, pb.FINISH_REASON_LENGTH
        if not self.ignore_eos_token and last_token in self.eos_token_ids:
            return True, pb.FINISH_REASON_EOS_TOKEN
        if self.stop_sequence_criterias:
            self.current_output += last_output
            # keep the rolling text bounded: only the tail can complete a stop sequence
            for c in self.stop_sequence_criterias:
                if c(self.current_output):
                    return True, pb.FINISH_REASON_STOP_SEQUENCE
        return False, None

    @classmethod
    def from_pb(cls, p, tokenizer, eos_token_ids: Optional[Set[int]] = None) -> "StoppingCriteria":
        eos = eos_token_ids
        if eos is None:
            eos = getattr(tokenizer, "_eos_token_ids", None)
            if eos is None:
                e = getattr(tokenizer, "eos_token_id", None)
                eos = set() if e is None else {e}
        return cls(eos, [StopSequenceCriteria(s) for s in p.stop_sequences], p.max_new_tokens, p.ignore_eos_token)


def batch_top_tokens(top_n_tokens: List[int], top_n_tokens_tensor: torch.Tensor, logprobs: torch.Tensor,
                     accepted_ids: torch.Tensor) -> Tuple[List[List[List[int]]], List[List[List[float]]]]:
    """Top-n tokens (ties included) for every accepted position of every request.

    Returns nested lists ``[request][accepted position][token]`` of ids and log-probabilities.
    """
    max_top_n = max(top_n_tokens) if top_n_tokens else 0
    if max_top_n == 0:
        return [[[]]] * len(top_n_tokens), [[[]]] * len(top_n_tokens)
    acc = accepted_ids.tolist()
    rep_n, rep_t = [], []
    for n, a in zip(top_n_tokens, acc):
        rep_n += [n] * a
    top_n_rows = torch.tensor([max(n, 1) for n in rep_n], device=logprobs.device)
    sorted_lp, sorted_idx = torch.sort(logprobs, dim=1, descending=True, stable=True)
    nth = sorted_lp.gather(1, (top_n_rows - 1).clamp(min=0).view(-1, 1))
    nth[nth == -math.inf] = torch.finfo(logprobs.dtype).min
    counts = (logprobs >= nth).sum(1).tolist()
    k = max(max(counts), max_top_n)
    top_vals, top_idx = sorted_lp[:, :k].tolist(), sorted_idx[:, :k].tolist()
    out_ids, out_lp = [], []
    row = 0
    for n, a in zip(top_n_tokens, acc):
        ids_r, lp_r = [], []
        for _ in range(a):
            if n == 0:
                ids_r.append([])
                lp_r.append([])
            else:
                c = counts[row]
                ids_r.append(top_idx[row][:c])
                lp_r.append(top_vals[row][:c])
            row += 1
        out_ids.append(ids_r)
        out_lp.append(lp_r)
    return out_ids, out_lp
