"""Tokenizer access.  HF tokenizers are used when a model/tokenizer directory is given; the synthetic tasks of the
benchmark configurations (no network, no checkpoint) use ``SyntheticTokenizer``: ids 0..2 are pad/bos/eos, digits
and arithmetic symbols get fixed ids, every other id decodes to ``<id>``.  (The reference loads tokenizers with
``load_tokenizer`` in siirl/models/loader.py.)"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence


class SyntheticTokenizer:
    PAD, BOS, EOS = 0, 1, 2
    _CHARS = "0123456789+-*/= ()?.,:abcdefghijklmnopqrstuvwxyz\n" + "<>{}[]\"'_!#$%&;@|~^ABCDEFGHIJKLMNOPQRSTUVWXYZ\\"

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.pad_token_id, self.bos_token_id, self.eos_token_id = self.PAD, self.BOS, self.EOS
        self.pad_token, self.eos_token = "<pad>", "<eos>"
        self._c2i: Dict[str, int] = {c: 3 + i for i, c in enumerate(self._CHARS)}
        self._i2c = {i: c for c, i in self._c2i.items()}
        self.padding_side = "left"

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = [self._c2i.get(c, 3 + self._CHARS.index("?")) for c in text]
        return ([self.BOS] if add_special_tokens else []) + ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        out = []
        for i in ids:
            i = int(i)
            if i in (self.PAD, self.BOS, self.EOS):
                if not skip_special_tokens:
                    out.append({0: "<pad>", 1: "<bos>", 2: "<eos>"}[i])
            else:
                out.append(self._i2c.get(i, f"<{i}>"))
        return "".join(out)

    def batch_decode(self, seqs, skip_special_tokens: bool = True) -> List[str]:
        return [self.decode(s, skip_special_tokens) for s in seqs]

    def apply_chat_template(self, messages, add_generation_prompt: bool = True, tokenize: bool = False, **_):
        text = "".join(f"{m['role']}:{m['content']}\n" for m in messages)
        if add_generation_prompt:
            text += "assistant:"
        return self.encode(text) if tokenize else text

    def __call__(self, text, **_):
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def __len__(self) -> int:
        return self.vocab_size


def load_tokenizer(path: Optional[str], vocab_size: int = 1024, trust_remote_code: bool = False):
    """HF tokenizer from ``path`` when it is a directory with tokenizer files, else the synthetic tokenizer."""
    if path:
        p = os.path.expanduser(path)
        if os.path.isdir(p) and any(os.path.exists(os.path.join(p, f)) for f in
                                    ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "vocab.json")):
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(p, trust_remote_code=trust_remote_code)
            if tok.pad_token_id is None:
                tok.pad_token = tok.eos_token
            return tok
    return SyntheticTokenizer(vocab_size)
