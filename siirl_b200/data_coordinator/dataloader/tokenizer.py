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


def load_tokenizer(path: Optional[str], vocab_size: int = 1024, trust_remote_code: bool = False, model_args=None):
    """HF tokenizer from ``path`` when it is a directory with tokenizer files, else the synthetic tokenizer.
    ``model_args`` (the ``actor_rollout_ref.model`` group) supplies the loader options of the reference
    (siirl/models/loader.py): ``use_fast_tokenizer``, ``split_special_tokens``, ``new_special_tokens`` (comma
    separated; they must fit the model's vocabulary unless ``resize_vocab`` is set, which this framework does not
    do: the embedding matrix belongs to the checkpoint)."""
    if path:
        p = os.path.expanduser(path)
        if os.path.isdir(p) and any(os.path.exists(os.path.join(p, f)) for f in
                                    ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "vocab.json")):
            from transformers import AutoTokenizer
            kw = {}
            if model_args is not None:
                kw["use_fast"] = bool(getattr(model_args, "use_fast_tokenizer", True))
                if getattr(model_args, "split_special_tokens", False):
                    kw["split_special_tokens"] = True
                trust_remote_code = trust_remote_code or bool(getattr(model_args, "trust_remote_code", False))
            tok = AutoTokenizer.from_pretrained(p, trust_remote_code=trust_remote_code, **kw)
            new = getattr(model_args, "new_special_tokens", None) if model_args is not None else None
            if new:
                names = [t.strip() for t in (new.split(",") if isinstance(new, str) else list(new)) if str(t).strip()]
                added = tok.add_tokens(names, special_tokens=True)
                if added and len(tok) > vocab_size and not getattr(model_args, "resize_vocab", False):
                    raise ValueError(f"model.new_special_tokens adds {added} token(s) beyond the model's vocabulary of "
                                     f"{vocab_size}: the embedding matrix is not resized")
                if added and len(tok) > vocab_size:
                    raise NotImplementedError("model.resize_vocab: growing the embedding matrix is not supported; "
                                              "use tokens inside the checkpoint's vocabulary")
            if tok.pad_token_id is None:
                tok.pad_token = tok.eos_token
            return tok
    return SyntheticTokenizer(vocab_size)
