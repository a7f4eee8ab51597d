# SPDX-License-Identifier: Apache-2.0
"""Causal (pre-training style) data: BOS + text + EOS tokenisation, then a token stream cut into rows of
exactly ``max_length`` tokens; documents shorter than a row are packed together and document boundaries
are kept in ``position_ids`` / ``packed_sample_seqlens``.  Parity: arctic_training/data/causal_factory.py:55-228.
"""

from __future__ import annotations

from collections import deque
from typing import Any
from typing import Deque
from typing import Dict
from typing import List

import torch

from ..config.data import DataConfig
from .factory import DataFactory
from .hf_sources import HFDataSourceCausal


class CausalCollator:
    def __call__(self, instances: List[Dict[str, Any]]) -> Dict[str, Any]:
        ids = torch.stack([torch.as_tensor(ex["input_ids"], dtype=torch.long) for ex in instances])
        pos = torch.stack([torch.as_tensor(ex["position_ids"], dtype=torch.long) for ex in instances])
        return {
            "input_ids": ids,
            "labels": ids.clone(),
            "position_ids": pos,
            "packed_sample_seqlens": [list(ex["packed_sample_seqlens"]) for ex in instances],
        }


def _row(pieces: List[List[int]]) -> Dict[str, List[int]]:
    return {
        "input_ids": [t for p in pieces for t in p],
        "position_ids": [i for p in pieces for i in range(len(p))],
        "packed_sample_seqlens": [len(p) for p in pieces],
    }


def slice_and_pack_causal_batch(batch: Dict[str, List[List[int]]], max_length: int,
                                overflow_buffer: List[List[int]]) -> Dict[str, List[List[int]]]:
    """Cut documents into full rows; leftovers wait in ``overflow_buffer`` (shared across calls) until
    together they fill a row.  What remains in the buffer at the very end is dropped."""
    out: Dict[str, List[List[int]]] = {"input_ids": [], "position_ids": [], "packed_sample_seqlens": []}

    def emit(pieces: List[List[int]]) -> None:
        row = _row(pieces)
        for k in out:
            out[k].append(row[k])

    pending: Deque[List[int]] = deque(overflow_buffer)
    pending_len = sum(len(x) for x in pending)
    for doc in batch["input_ids"]:
        full = len(doc) // max_length
        for i in range(full):
            emit([doc[i * max_length : (i + 1) * max_length]])
        tail = doc[full * max_length :]
        if tail:
            pending.append(tail)
            pending_len += len(tail)
        while pending_len >= max_length:
            pieces, used = [], 0
            while used < max_length:
                piece = pending.popleft()
                room = max_length - used
                if len(piece) > room:
                    pending.appendleft(piece[room:])
                    piece = piece[:room]
                pieces.append(piece)
                used += len(piece)
            pending_len -= max_length
            emit(pieces)
    overflow_buffer[:] = list(pending)
    return out


class CausalDataConfig(DataConfig):
    pass


def slice_and_pack_dataset(self, dataset):
    cfg = self.config
    dataset = dataset.shuffle(seed=cfg.seed)
    overflow: List[List[int]] = []
    dataset = dataset.map(
        lambda x: slice_and_pack_causal_batch(x, cfg.max_length, overflow),
        batched=True, batch_size=min(100, len(dataset) + 1), remove_columns=dataset.column_names, desc="Packing dataset",
    )
    if len(dataset) < 1:
        raise ValueError("No data left after packing dataset samples (is max_length larger than the corpus?)")
    return dataset


class CausalDataFactory(DataFactory):
    name = "causal"
    config: CausalDataConfig
    default_source_cls = HFDataSourceCausal
    callbacks = [("post-load", slice_and_pack_dataset)]

    def process(self, dataset):
        if "text" not in dataset.column_names:
            raise ValueError("Dataset must have a 'text' column to tokenize for CausalDataFactory.")
        tok, tcfg = self.tokenizer, self.trainer.config.tokenizer
        nproc = min(self.config.num_proc, max(1, len(dataset) // 64))
        return dataset.select_columns(["text"]).map(
            lambda ex: self.tokenize_text(ex["text"], tok, tcfg),
            remove_columns=["text"], num_proc=nproc if nproc > 1 else None, desc="Tokenizing text",
        )

    @classmethod
    def tokenize_text(cls, text: str, tokenizer: Any, tokenizer_config_at: Any) -> Dict[str, List[int]]:
        kwargs = dict(return_attention_mask=False, add_special_tokens=False, verbose=False)
        kwargs.update(tokenizer_config_at.tokenize_kwargs)
        if tokenizer_config_at.tokenize_kwargs.get("add_special_tokens", False):
            raise ValueError(
                "CausalDataFactory adds BOS/EOS itself; `tokenizer.tokenize_kwargs.add_special_tokens: true` "
                "would insert them twice."
            )
        ids: List[int] = []
        if getattr(tokenizer, "bos_token_id", None) is not None:
            ids.append(tokenizer.bos_token_id)
        ids += list(tokenizer(text, **kwargs)["input_ids"])
        if getattr(tokenizer, "eos_token_id", None) is not None:
            ids.append(tokenizer.eos_token_id)
        return {"input_ids": ids}

    def collate_fn(self):
        return CausalCollator()
