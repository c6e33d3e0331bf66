"""Tokenizer loading plus a dependency-free byte tokenizer for synthetic models.

The engine needs from a tokenizer: ``__call__``/``encode`` with truncation from the left,
``decode``, ``eos_token_id``, ``all_special_ids``, ``get_vocab`` and ``convert_tokens_to_string``
(for grammar indices).  A Hugging Face fast tokenizer provides all of that; ``ByteTokenizer`` is a
256-byte vocabulary with ``<pad>/<s>/</s>`` used when a model directory has no tokenizer (random-
weight benchmark models) and in unit tests.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional


class ByteTokenizer:
    """UTF-8 bytes as tokens: id ``b + 3`` for byte ``b``; 0 pad, 1 bos, 2 eos; ids above 258 decode to ''."""

    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2
    truncation_side = "left"
    padding_side = "left"

    def __init__(self, vocab_size: int = 259, add_bos: bool = False):
        self.vocab_size = max(vocab_size, 259)
        self.add_bos = add_bos
        self.all_special_ids = [0, 1, 2]
        self.chat_template = None

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids = [b + 3 for b in text.encode("utf-8")]
        if self.add_bos and add_special_tokens:
            ids = [1] + ids
        return ids

    def __call__(self, text, add_special_tokens=True, truncation=False, max_length=None, **kw):
        single = isinstance(text, str)
        out = []
        for t in ([text] if single else text):
            ids = self.encode(t, add_special_tokens)
            if truncation and max_length is not None and len(ids) > max_length:
                ids = ids[-max_length:]
            out.append(ids)
        return {"input_ids": out[0] if single else out}

    def decode(self, ids, skip_special_tokens: bool = False, **kw) -> str:
        bs = bytearray()
        parts: List[str] = []
        names = {0: "<pad>", 1: "<s>", 2: "</s>"}
        for i in ids:
            i = int(i)
            if 3 <= i < 259:
                bs.append(i - 3)
            elif i in names and not skip_special_tokens:
                parts.append(bs.decode("utf-8", errors="replace"))
                bs = bytearray()
                parts.append(names[i])
        parts.append(bs.decode("utf-8", errors="replace"))
        return "".join(parts)

    def get_vocab(self) -> Dict[str, int]:
        v = {"<pad>": 0, "<s>": 1, "</s>": 2}
        for b in range(256):
            v[f"<0x{b:02X}>"] = b + 3
        return v

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        v = self.get_vocab()
        return self.decode([v[t] for t in tokens])

    def convert_ids_to_tokens(self, ids):
        inv = {i: t for t, i in self.get_vocab().items()}
        return [inv.get(int(i), "") for i in ids]

    def __len__(self):
        return self.vocab_size


def load_tokenizer(model_path: Optional[str], revision: Optional[str] = None, trust_remote_code: bool = False,
                   vocab_size: int = 259):
    """Hugging Face tokenizer of a model directory (left truncation/padding), else a ``ByteTokenizer``."""
    if model_path and os.path.isdir(model_path) and any(
        os.path.exists(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json")
    ):
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(model_path, revision=revision, padding_side="left",
                                            truncation_side="left", trust_remote_code=trust_remote_code)
        return tok
    return ByteTokenizer(vocab_size)
