# SPDX-License-Identifier: Apache-2.0
"""A dependency-free tokenizer for tests, benchmarks and synthetic data.

Words are mapped to ids by a stable hash (so no vocabulary file is needed), special tokens occupy the
first ids, and ``apply_chat_template`` renders messages in a simple ``<|role|> content <|eot|>`` format
and can report per-character offsets, which is all the SFT data factory needs to mask non-assistant
tokens.  It mimics the subset of the Hugging Face tokenizer interface that the data factories use.
"""

from __future__ import annotations

import hashlib
import json
import re
from pathlib import Path
from typing import Any
from typing import Dict
from typing import List
from typing import Optional
from typing import Union

_WORD = re.compile(r"<\|[a-z_]+\|>|\w+|[^\w\s]|\s+")


class FakeTokenizer:
    pad_token = "<|pad|>"
    bos_token = "<|bos|>"
    eos_token = "<|eot|>"
    unk_token = "<|unk|>"
    _specials = ["<|pad|>", "<|bos|>", "<|eot|>", "<|unk|>", "<|system|>", "<|user|>", "<|assistant|>"]
    chat_template = "fake"
    padding_side = "right"

    def __init__(self, vocab_size: int = 1024, name_or_path: str = "fake") -> None:
        assert vocab_size > 16
        self.vocab_size = vocab_size
        self.name_or_path = name_or_path
        self.pad_token_id, self.bos_token_id, self.eos_token_id, self.unk_token_id = 0, 1, 2, 3
        self._special_ids = {s: i for i, s in enumerate(self._specials)}
        self.model_max_length = 1 << 30

    def __len__(self) -> int:
        return self.vocab_size

    def _tok_id(self, piece: str) -> int:
        if piece in self._special_ids:
            return self._special_ids[piece]
        h = int.from_bytes(hashlib.blake2s(piece.encode("utf-8"), digest_size=4).digest(), "little")
        return len(self._specials) + h % (self.vocab_size - len(self._specials))

    def _pieces(self, text: str):
        for m in _WORD.finditer(text):
            if m.group().isspace():
                continue
            yield m.group(), m.start(), m.end()

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = [self._tok_id(p) for p, _, _ in self._pieces(text)]
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: List[int], skip_special_tokens: bool = False) -> str:
        inv = {v: k for k, v in self._special_ids.items()}
        return " ".join(inv.get(int(i), f"w{int(i)}") for i in ids if not (skip_special_tokens and int(i) in inv))

    def __call__(self, text: Union[str, List[str]], add_special_tokens: bool = False, return_offsets_mapping: bool = False,
                 truncation: bool = False, max_length: Optional[int] = None, **_: Any) -> Dict[str, Any]:
        if isinstance(text, list):
            outs = [self(t, add_special_tokens, return_offsets_mapping, truncation, max_length) for t in text]
            return {k: [o[k] for o in outs] for k in outs[0]}
        ids, offs = [], []
        if add_special_tokens:
            ids.append(self.bos_token_id)
            offs.append((0, 0))
        for p, s, e in self._pieces(text):
            ids.append(self._tok_id(p))
            offs.append((s, e))
        if truncation and max_length is not None:
            ids, offs = ids[:max_length], offs[:max_length]
        out: Dict[str, Any] = {"input_ids": ids, "attention_mask": [1] * len(ids)}
        if return_offsets_mapping:
            out["offset_mapping"] = offs
        return out

    def apply_chat_template(self, conversation: List[Dict[str, str]], tokenize: bool = False,
                            add_generation_prompt: bool = False, **_: Any) -> Union[str, List[int]]:
        text = self.bos_token
        for msg in conversation:
            text += f"<|{msg['role']}|> {msg['content']} {self.eos_token}\n"
        if add_generation_prompt:
            text += "<|assistant|> "
        return self.encode(text) if tokenize else text

    def save_pretrained(self, path: Union[str, Path]) -> None:
        Path(path).mkdir(parents=True, exist_ok=True)
        with open(Path(path) / "fake_tokenizer.json", "w") as fh:
            json.dump({"vocab_size": self.vocab_size}, fh)

    @classmethod
    def from_pretrained(cls, path: Union[str, Path]) -> "FakeTokenizer":
        f = Path(path) / "fake_tokenizer.json"
        if f.exists():
            with open(f) as fh:
                return cls(**json.load(fh))
        return cls()
