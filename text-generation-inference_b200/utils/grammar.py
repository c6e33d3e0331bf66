"""Grammar-constrained decoding (JSON schema or regex) with a token-level finite-state index.

Role of ``GrammarLogitProcessor`` / ``HeterogeneousGrammarLogitProcessor`` in the reference
(``utils/logits_process.py:482-625``): a regex (or a JSON schema compiled to a regex) becomes an
index ``state -> allowed token ids`` over the tokenizer's vocabulary; before choosing a token the
disallowed logits are set to ``-inf``; after choosing, the request's state advances.  State ``-1``
means the grammar is complete and nothing is masked any more.

The index is ``outlines_core.Index`` (automaton construction in native code); compiled indices
are kept in an LRU cache keyed by ``(grammar, type, tokenizer)`` because requests re-use schemas.
"""
from __future__ import annotations

import json
import math
from functools import lru_cache
from typing import Dict, List, Optional

import torch

GRAMMAR_NONE, GRAMMAR_JSON, GRAMMAR_REGEX = 0, 1, 2

_VOCAB_CACHE: Dict[int, object] = {}


def _token_strings(tokenizer) -> Dict[str, List[int]]:
    """Map decoded token text -> token ids (several ids can decode to the same text)."""
    vocab = tokenizer.get_vocab()
    special = set(getattr(tokenizer, "all_special_ids", []) or [])
    out: Dict[str, List[int]] = {}
    for tok, tid in vocab.items():
        if tid in special:
            continue
        try:
            s = tokenizer.convert_tokens_to_string([tok])
        except Exception:
            s = tok
        # sentencepiece drops the leading space of a word-initial piece when decoded alone
        if tok.startswith("▁") or tok.startswith("Ġ") or tok == "<0x20>":
            if not s.startswith(" "):
                s = " " + s
        if s == "":
            continue
        out.setdefault(s, []).append(tid)
    return out


def _vocabulary(tokenizer):
    from outlines_core import Vocabulary

    key = id(tokenizer)
    if key not in _VOCAB_CACHE:
        eos = tokenizer.eos_token_id if tokenizer.eos_token_id is not None else 0
        _VOCAB_CACHE[key] = Vocabulary(eos, _token_strings(tokenizer))
    return _VOCAB_CACHE[key]


def schema_to_regex(schema: str) -> str:
    from outlines_core.json_schema import build_regex_from_schema

    if not isinstance(schema, str):
        schema = json.dumps(schema)
    return build_regex_from_schema(schema)


class CompiledGrammar:
    def __init__(self, index, eos_token_id: int):
        self.index = index
        self.eos_token_id = eos_token_id
        self.initial = index.get_initial_state()
        self._allowed: Dict[int, List[int]] = {}

    def allowed(self, state: int) -> List[int]:
        a = self._allowed.get(state)
        if a is None:
            a = self.index.get_allowed_tokens(state) or []
            self._allowed[state] = a
        return a

    def next_state(self, state: int, token: int) -> int:
        if state == -1:
            return -1
        if token == self.eos_token_id and self.index.is_final_state(state):
            return -1
        nxt = self.index.get_next_state(state, token)
        return -1 if nxt is None else nxt


_COMPILED: Dict[tuple, CompiledGrammar] = {}


def compile_grammar(grammar: str, grammar_type: int, tokenizer) -> CompiledGrammar:
    from outlines_core import Index

    key = (grammar, grammar_type, id(tokenizer))
    hit = _COMPILED.get(key)
    if hit is not None:
        return hit
    regex = schema_to_regex(grammar) if grammar_type == GRAMMAR_JSON else grammar
    eos = tokenizer.eos_token_id if tokenizer.eos_token_id is not None else 0
    compiled = CompiledGrammar(Index(regex, _vocabulary(tokenizer)), eos)
    if len(_COMPILED) >= 32:
        _COMPILED.pop(next(iter(_COMPILED)))
    _COMPILED[key] = compiled
    return compiled


class GrammarBatch:
    """Grammars of every request of a batch (``None`` where a request has none).

    FSM states held by the caller are encoded: ``0`` is the grammar's start, ``-1`` is done, and
    ``s + 1`` stands for automaton state ``s`` (so an automaton state numbered 0 stays distinct
    from "start").
    """

    def __init__(self, tokenizer, device, grammars: List[str], grammar_types: List[int]):
        self.device = device
        self.tokenizer = tokenizer
        self.fsms: List[Optional[CompiledGrammar]] = []
        for g, t in zip(grammars, grammar_types):
            self.fsms.append(None if (g == "" or t == GRAMMAR_NONE) else compile_grammar(g, t, tokenizer))

    def _state(self, fsm: CompiledGrammar, s: int) -> int:
        return fsm.initial if s == 0 else s - 1

    def mask(self, scores: torch.Tensor, states: List[int]) -> torch.Tensor:
        for i, fsm in enumerate(self.fsms):
            if fsm is None or states[i] == -1:
                continue
            allowed = fsm.allowed(self._state(fsm, states[i]))
            m = torch.full_like(scores[i], -math.inf)
            if allowed:
                idx = torch.tensor(allowed, dtype=torch.long, device=scores.device)
                idx = idx[idx < scores.shape[-1]]
                m[idx] = 0
            scores[i] = scores[i] + m
        return scores

    def advance_at_index(self, next_id: int, state: int, i: int) -> int:
        fsm = self.fsms[i]
        if fsm is None or state == -1:
            return state
        nxt = fsm.next_state(self._state(fsm, state), int(next_id))
        return -1 if nxt == -1 else nxt + 1

    def advance_batch(self, next_ids: List[int], states: List[int]) -> List[int]:
        return [self.advance_at_index(t, s, i) for i, (t, s) in enumerate(zip(next_ids, states))]

    def filter(self, indices: List[int]) -> Optional["GrammarBatch"]:
        self.fsms = [self.fsms[i] for i in indices]
        return self if any(f is not None for f in self.fsms) else None
