# SPDX-License-Identifier: Apache-2.0
"""Supervised fine-tuning data: chat-template tokenisation with assistant-only labels, length filter,
sample packing and the padding collator.

Behaviour parity: arctic_training/data/sft_factory.py:44-471.  Labels follow the "offset range" rule of
the reference: a token is trained on when its character span lies inside an assistant message, plus the
single token that follows an assistant span (so the end-of-turn token is learnt).  Packing concatenates
samples greedily up to ``max_length``, restarts ``position_ids`` at every sample and records
``packed_sample_seqlens``; the collator pads to a multiple of ``div_length`` (or to ``max_length``), with
-100 for labels and a running ``arange`` for position ids.
"""

from __future__ import annotations

import random
import re
from typing import Any
from typing import Dict
from typing import List
from typing import Literal
from typing import Optional
from typing import Sequence
from typing import Tuple

import torch
from pydantic import Field
from pydantic import model_validator
from typing_extensions import Self

from ..config.data import DataConfig
from ..config.utils import HumanInt
from .factory import DataFactory
from .hf_sources import HFDataSourceInstruct

IGNORE_INDEX = -100
_EMPTY_THINK = re.compile(r"^<think>\s*</think>\s*")


def pad(
    tensors: Sequence[torch.Tensor],
    padding_value: int = 0,
    padding_side: str = "right",
    is_position_id: bool = False,
    divisible_by: Optional[int] = 256,
    max_seq: Optional[int] = None,
) -> torch.Tensor:
    """Stack 1-D tensors into ``[len(tensors), L]`` where ``L`` is ``max_seq`` or the longest length
    rounded up to ``divisible_by``.  Position ids are padded with a plain ``arange`` so that padding never
    looks like thousands of one-token samples to a varlen attention kernel."""
    longest = max(int(t.shape[0]) for t in tensors)
    if max_seq is not None:
        length = max_seq
    elif divisible_by:
        length = -(-longest // divisible_by) * divisible_by
    else:
        length = longest
    if is_position_id:
        out = torch.arange(length, dtype=tensors[0].dtype).repeat(len(tensors), 1)
    else:
        out = torch.full((len(tensors), length), padding_value, dtype=tensors[0].dtype)
    for i, t in enumerate(tensors):
        t = t[:length]
        if padding_side == "right":
            out[i, : t.shape[0]] = t
        elif padding_side == "left":
            out[i, length - t.shape[0] :] = t
        else:
            raise ValueError("padding_side must be 'left' or 'right'")
    return out


class DataCollatorForCausalLM:
    def __init__(self, tokenizer: Any, config: "SFTDataConfig") -> None:
        self.tokenizer = tokenizer
        self.config = config

    def __call__(self, instances: List[Dict[str, Any]]) -> Dict[str, Any]:
        ids = [torch.as_tensor(ex["input_ids"], dtype=torch.long) for ex in instances]
        labels = [torch.as_tensor(ex["labels"], dtype=torch.long) for ex in instances]
        if "position_ids" in instances[0] and instances[0]["position_ids"] is not None:
            pos = [torch.as_tensor(ex["position_ids"], dtype=torch.long) for ex in instances]
            seqlens = [list(ex["packed_sample_seqlens"]) for ex in instances]
        else:
            pos = [torch.arange(len(t), dtype=torch.long) for t in ids]
            seqlens = [[len(t)] for t in ids]
        if self.config.pad_to == "max_length":
            kw: Dict[str, Any] = {"max_seq": self.config.max_length}
        elif self.config.pad_to == "div_length":
            kw = {"divisible_by": self.config.div_length}
        else:
            raise ValueError(f"Unknown pad_to value: {self.config.pad_to}")
        pad_id = getattr(self.tokenizer, "pad_token_id", 0) or 0
        return {
            "input_ids": pad(ids, padding_value=pad_id, **kw),
            "labels": pad(labels, padding_value=IGNORE_INDEX, **kw),
            "position_ids": pad(pos, padding_value=0, is_position_id=True, **kw),
            "packed_sample_seqlens": seqlens,
        }


def pack_sft_batch(
    batch: Dict[str, List[List[int]]],
    max_length: int,
    always_max_length: bool,
    drop_last: bool,
    fuse_positions_prob: float,
    seed: int,
) -> Dict[str, List[List[int]]]:
    """Greedy packing of tokenised samples (in order) into rows of at most ``max_length`` tokens."""
    keys = ("input_ids", "labels", "position_ids", "packed_sample_seqlens", "attention_mask")
    out: Dict[str, List[List[int]]] = {k: [] for k in keys}
    cur: Dict[str, List[int]] = {k: [] for k in keys}
    rng = random.Random(seed)

    def flush() -> None:
        if not cur["input_ids"]:
            return
        if fuse_positions_prob and rng.random() <= fuse_positions_prob:
            cur["position_ids"] = list(range(len(cur["input_ids"])))
        for k in keys:
            out[k].append(cur[k])
            cur[k] = []

    masks = batch.get("attention_mask") or [[1] * len(x) for x in batch["input_ids"]]
    for ids, labels, mask in zip(batch["input_ids"], batch["labels"], masks):
        total = len(cur["input_ids"])
        if total > max_length or (not always_max_length and total + len(ids) > max_length):
            flush()
        cur["input_ids"].extend(ids)
        cur["labels"].extend(labels)
        cur["attention_mask"].extend(mask)
        cur["position_ids"].extend(range(len(ids)))
        cur["packed_sample_seqlens"].append(len(ids))
    if not drop_last:
        flush()
    return out


class SFTDataConfig(DataConfig):
    div_length: HumanInt = 256
    """ Sequences are padded to a multiple of this. """

    mask_inputs: bool = True
    """ Train on assistant tokens only. """

    always_max_length: bool = False
    """ Keep appending samples until a packed row reaches ``max_length``. """

    pad_to: Literal["max_length", "div_length"] = "div_length"
    """ Pad to ``max_length`` or to the next multiple of ``div_length``. """

    filter_samples: bool = True
    """ Drop samples longer than ``max_length``. """

    pack_samples: bool = False
    """ Pack several samples into one row of up to ``max_length`` tokens. """

    drop_last: bool = False
    """ Drop the last (possibly short) packed row. """

    fuse_positions_prob: float = Field(0.0, ge=0.0, le=1.0)
    """ Probability with which a packed row gets contiguous position ids (long-context augmentation). """

    repeat_to_pack_max_length: bool = False
    """ Repeat a small dataset so that a packed row gets close to ``max_length``. """

    ignore_empty_think: bool = False
    """ Do not train on an empty ``<think></think>`` prefix of assistant messages. """

    @model_validator(mode="after")
    def _padding_is_consistent(self) -> Self:
        if self.pad_to == "max_length" and "div_length" in self.model_fields_set and self.max_length % self.div_length:
            lo = self.max_length // self.div_length * self.div_length
            raise ValueError(
                f"You have requested padding sequences to 'max_length', which needs max_length ({self.max_length}) "
                f"divisible by div_length ({self.div_length}); use {lo} or {lo + self.div_length}, or drop div_length."
            )
        return self


def filter_dataset_length(self, dataset):
    if not self.config.filter_samples:
        return dataset
    limit = self.config.max_length
    dataset = dataset.filter(lambda x: len(x["input_ids"]) <= limit, num_proc=_procs(self, dataset), desc="Length filter")
    if len(dataset) < 1:
        raise ValueError(f"No data left after filtering by max length {limit}. Consider increasing `max_length`.")
    return dataset


def _procs(self, dataset) -> Optional[int]:
    n = min(self.config.num_proc, max(1, len(dataset) // 64))
    return n if n > 1 else None


def repeat_dataset(dataset, max_length: int):
    from datasets import concatenate_datasets

    lengths = [len(x) for x in dataset["input_ids"]]
    per_round = sum(lengths)
    repeats = max(1, max_length // per_round)
    remaining = max_length - repeats * per_round
    used, end = 0, 0
    for n in lengths:
        if used + n > remaining:
            break
        used += n
        end += 1
    return concatenate_datasets([dataset] * repeats + [dataset.select(range(end))])


def pack_dataset(self, dataset):
    if not self.config.pack_samples:
        return dataset
    cfg = self.config
    if cfg.repeat_to_pack_max_length:
        dataset = repeat_dataset(dataset, cfg.max_length)
    nproc = _procs(self, dataset)
    batch_size = int(min(len(dataset) // (nproc or 1) + 1, 1000))
    dataset = dataset.shuffle(seed=cfg.seed)
    dataset = dataset.map(
        lambda x: pack_sft_batch(x, cfg.max_length, cfg.always_max_length, cfg.drop_last, cfg.fuse_positions_prob, cfg.seed),
        batched=True, batch_size=batch_size, num_proc=nproc, remove_columns=dataset.column_names, desc="Packing",
    )
    if len(dataset) < 1:
        raise ValueError("No data left after packing dataset samples")
    return dataset


class SFTDataFactory(DataFactory):
    name = "sft"
    config: SFTDataConfig
    default_source_cls = HFDataSourceInstruct
    callbacks = [("post-load", filter_dataset_length), ("post-load", pack_dataset)]

    def process(self, dataset):
        if "messages" not in dataset.column_names:
            raise ValueError("Dataset must have a 'messages' column to tokenize for SFTDataFactory.")
        dataset = dataset.select_columns(["messages"])
        tok, cfg = self.tokenizer, self.config
        return dataset.map(
            lambda ex: dict(self.tokenize_messages(ex["messages"], tok, cfg.mask_inputs, cfg.ignore_empty_think)),
            remove_columns=dataset.column_names, num_proc=_procs(self, dataset), desc="Tokenizing messages",
        )

    @classmethod
    def tokenize_messages(cls, messages: List[Dict[str, str]], tokenizer: Any, mask_inputs: bool = True,
                          ignore_empty_think: bool = False) -> Dict[str, List[int]]:
        text = tokenizer.apply_chat_template(conversation=messages, tokenize=False)
        enc = tokenizer(text, return_offsets_mapping=mask_inputs, add_special_tokens=False)
        enc = {k: enc[k] for k in enc.keys()} if not isinstance(enc, dict) else dict(enc)
        if mask_inputs:
            ranges = cls.get_assistant_start_end_indices(messages, text, ignore_empty_think)
            enc["labels"] = cls.get_masked_labels(enc, ranges)
            del enc["offset_mapping"]
        else:
            enc["labels"] = list(enc["input_ids"])
        enc.setdefault("attention_mask", [1] * len(enc["input_ids"]))
        return enc

    @staticmethod
    def get_assistant_start_end_indices(messages, conversation_text: str, ignore_empty_think: bool = False) -> List[Tuple[int, int]]:
        spans = []
        for msg in messages:
            if msg["role"] != "assistant":
                continue
            content = msg["content"]
            if ignore_empty_think:
                content = _EMPTY_THINK.sub("", content)
            start = conversation_text.find(content)
            spans.append((start, start + len(content)))
        return spans

    @staticmethod
    def get_masked_labels(conversation_ids: Dict[str, Any], assistant_ranges: List[Tuple[int, int]]) -> List[int]:
        labels: List[int] = []
        inside_prev = False
        for tok, (s, e) in zip(conversation_ids["input_ids"], conversation_ids["offset_mapping"]):
            inside = any(s >= a and e <= b for a, b in assistant_ranges)
            # the first token after an assistant span (the end-of-turn marker) is kept as a target
            labels.append(tok if inside or inside_prev else IGNORE_INDEX)
            inside_prev = inside
        return labels

    def collate_fn(self):
        return DataCollatorForCausalLM(tokenizer=self.tokenizer, config=self.config)
