# SPDX-License-Identifier: Apache-2.0
"""Bi-encoder: one shared text encoder for queries and documents, pooled and (at loss time) L2-normalised.
Behaviour parity: projects/arctic_embed/src/arctic_embed/core/biencoder_model.py:37-134 (first / last / mean
pooling; ``biencoder_config.json`` next to the encoder checkpoint).

The encoder is the native decoder stack (``DecoderModel``) when the architecture is one of the native families, or
any ``transformers.AutoModel`` otherwise.
"""

from __future__ import annotations

import json
from dataclasses import asdict
from dataclasses import dataclass
from pathlib import Path
from typing import Tuple

import torch
import torch.nn as nn
from torch import Tensor


@dataclass
class BiencoderConfig:
    pooling: str = "first"  # first | last | mean
    normalize: bool = False

    def save(self, directory: Path) -> None:
        (Path(directory) / "biencoder_config.json").write_text(json.dumps(asdict(self)))

    @classmethod
    def load(cls, directory: Path) -> "BiencoderConfig":
        return cls(**json.loads((Path(directory) / "biencoder_config.json").read_text()))


def pool(hidden: Tensor, attention_mask: Tensor, how: str) -> Tensor:
    """``hidden [B, S, H]``, ``attention_mask [B, S]`` (1 = token) -> ``[B, H]``."""
    how = {"first_token": "first", "last_token": "last", "average": "mean"}.get(how, how)
    if how == "first":
        return hidden[:, 0]
    if how == "last":
        # index of the last real token, for right- and left-padded rows alike
        S = attention_mask.shape[1]
        last = S - 1 - attention_mask.long().flip(1).argmax(1)
        return hidden[torch.arange(hidden.size(0), device=hidden.device), last]
    if how == "mean":
        m = attention_mask.unsqueeze(-1).to(hidden.dtype)
        return (hidden * m).sum(1) / m.sum(1).clamp(min=1)
    raise ValueError(f"unknown pooling {how!r}")


def first_token_pool(hidden: Tensor, attention_mask: Tensor) -> Tensor:
    return pool(hidden, attention_mask, "first")


def last_token_pool(hidden: Tensor, attention_mask: Tensor) -> Tensor:
    return pool(hidden, attention_mask, "last")


def average_pool(hidden: Tensor, attention_mask: Tensor) -> Tensor:
    return pool(hidden, attention_mask, "mean")


class Biencoder(nn.Module):
    def __init__(self, encoder: nn.Module, config: BiencoderConfig) -> None:
        super().__init__()
        self.encoder = encoder
        self.biencoder_config = config
        self.config = getattr(encoder, "cfg", getattr(encoder, "config", {}))
        self.activation_checkpointing = False

    def encode(self, input_ids: Tensor, attention_mask: Tensor) -> Tensor:
        out = self.encoder(input_ids=input_ids, attention_mask=attention_mask)
        hidden = out if torch.is_tensor(out) else getattr(out, "last_hidden_state", out[0])
        emb = pool(hidden, attention_mask, self.biencoder_config.pooling)
        return torch.nn.functional.normalize(emb, dim=-1) if self.biencoder_config.normalize else emb

    def forward(self, query_input_ids: Tensor, query_attention_mask: Tensor, document_input_ids: Tensor,
                document_attention_mask: Tensor) -> Tuple[Tensor, Tensor]:
        return (self.encode(query_input_ids, query_attention_mask),
                self.encode(document_input_ids, document_attention_mask))

    def zero_units(self):
        enc = self.encoder
        if hasattr(enc, "layers") and hasattr(enc, "embed_tokens"):
            units = [("embed", [enc.embed_tokens], False)]
            units += [(f"layer{i}", [layer], True) for i, layer in enumerate(enc.layers)]
            units.append(("head", [enc.norm], False))
            return units
        return [("encoder", [enc], False)]
